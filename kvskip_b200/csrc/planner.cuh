// Device-side refresh planner: `plan` before the attention pass, `update` after it.
//
// Semantics and float operation order follow format37/kvskip's plan_kernel / update_kernel
// (kernels/kvskip_planner.cu:75-305) so that, given the same inputs, the integer outputs (refresh
// decision, block list, stored set, age, index latch) are identical and the float outputs agree to
// the last bit on the same GPU.  The order that matters:
//   centroid score   lane l multiplies dims 4l..4l+3 (first product rounded, three fused
//                    multiply-adds), 32-lane butterfly, then times 1/n_b;
//   drift estimate   128 "fold slots": slot t folds blocks t, t+128, ... into a running (max, sum);
//                    slots merge per 32 (max, butterfly of rescaled sums), the four groups merge
//                    serially in ascending order;
//   top-p cut        per query head lane l owns blocks l, l+32, ...; 32 bisection steps on the
//                    log-weight threshold in [-80, 0], each a lane-serial sum + butterfly.
// Layout of the work is ours.  Both kernels are chains of dependent memory latencies rather than
// bandwidth: `plan` spreads the centroid scores over ceil(nb/32) CTAs per head and lets the last
// one to finish do the fold; the per-block "attended" flags are staged in shared memory with
// independent coalesced loads, and the fold loads its operands four blocks ahead, so a head costs
// a handful of memory round trips instead of one per block.  No per-head shared-memory table of
// scores is needed, so block counts beyond 3072 (contexts beyond 196 608 tokens) work.
#pragma once
#include "common.cuh"

namespace kvb {

constexpr int PL_THREADS = 128;
constexpr int PL_G = 4;
constexpr int PL_D = 128;

__device__ __forceinline__ bool pl_always(int blk, int nb, int local) { return blk == 0 || blk >= nb - local; }

__device__ __forceinline__ float pl_logit(float x) {
  x = fminf(fmaxf(x, 1e-6f), 1.f - 1e-6f);
  return __logf(x) - __logf(1.f - x);
}

// running log-sum-exp (m, s), s relative to m
__device__ __forceinline__ void pl_fold(float& m, float& s, float e) {
  if (e == -INFINITY) return;
  if (e > m) {
    s = s * __expf(m - e) + 1.f;
    m = e;
  } else {
    s += __expf(e - m);
  }
}

// Ascending compaction of the blocks satisfying `pred` into bi[]; count to *cnt.  Chunked scan:
// thread t owns a contiguous chunk, an inclusive Hillis-Steele scan over the 128 chunk counts
// gives the offsets.  Must be called by all PL_THREADS threads.
template <typename Pred>
__device__ __forceinline__ void pl_compact(int nb, int* bi, int* cnt, int* scan, Pred pred) {
  const int tid = threadIdx.x;
  const int per = (nb + PL_THREADS - 1) / PL_THREADS;
  const int a = min(nb, tid * per), e = min(nb, a + per);
  int c = 0;
  for (int i = a; i < e; ++i) c += pred(i) ? 1 : 0;
  scan[tid] = c;
  __syncthreads();
  for (int o = 1; o < PL_THREADS; o <<= 1) {
    const int add = tid >= o ? scan[tid - o] : 0;
    __syncthreads();
    scan[tid] += add;
    __syncthreads();
  }
  int off = scan[tid] - c;
  for (int i = a; i < e; ++i)
    if (pred(i)) bi[off++] = i;
  if (tid == PL_THREADS - 1) *cnt = scan[PL_THREADS - 1];
}

constexpr int PL_CHUNK = 32;   // blocks whose centroid scores one CTA computes (4 warps x 8 in flight)

// grid (ceil(nb / PL_CHUNK), Hkv, B).  Every CTA computes the centroid scores of its chunk of
// blocks and stores them to cs_now; the last CTA of a (batch, kv head) to finish (counted in
// done[], which it puts back to zero) folds the estimate, decides and writes the block list.
// The arithmetic of a score and of the fold is unchanged, only spread over more SMs: one CTA per
// head reading nb * 512 bytes of key sums is latency-bound at long contexts.
// With a device-resident length (t_dev != nullptr) p.T is the bound the grid was sized for; CTAs
// whose chunk lies beyond the current length leave without being counted.
// With a paged cache (pages != nullptr) p.k is the page pool [pages, Hkv, 64, D] (k_sb = page stride)
// and the key of the new token is row (T-1) % 64 of page pages[b, (T-1) / 64].
__global__ void __launch_bounds__(PL_THREADS) plan_kernel(const kvskip_plan_params p, int* __restrict__ done,
                                                          const int* __restrict__ t_dev,
                                                          const int32_t* __restrict__ pages, const int max_pages,
                                                          const int num_pages) {
  const int chunk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t bh = static_cast<int64_t>(b) * p.Hkv + h;
  float* csum = p.csum + bh * p.NBC * PL_D;
  const uint8_t* keep = p.keep + bh * p.NBC;
  int* bi = p.block_idx + bh * p.NBC;
  __shared__ int scan[PL_THREADS];
  __shared__ float wM[PL_THREADS / 32][PL_G], wS[PL_THREADS / 32][PL_G];
  __shared__ int s_flag;
  pdl_wait_prior();          // the state this kernel reads may come from the previous kernel on the stream
  pdl_launch_dependents();
  const int T = t_dev ? max(1, min(*t_dev, p.T)) : p.T;
  const int nb = (T + TILE - 1) / TILE;
  const int chunks = (nb + PL_CHUNK - 1) / PL_CHUNK;
  if (chunk >= chunks) return;

  const int fl = p.flags[h];
  if (fl & 2) {   // token-index head: index blocks + sink + newest, never refreshes; one CTA does it
    if (chunk != 0) return;
    const uint8_t* ix = p.idx + static_cast<int64_t>(b) * p.NBC;
    pl_compact(nb, bi, p.block_cnt + bh, scan, [&](int i) { return ix[i] || pl_always(i, nb, p.local); });
    if (tid == 0) p.trig[bh] = 0;
    return;
  }
  const bool uni = (fl & 4) || (p.aix && p.aix[bh]);
  const uint8_t* ix = uni ? p.idx + static_cast<int64_t>(b) * p.NBC : nullptr;
  auto attended = [&](int blk) { return keep[blk] || pl_always(blk, nb, p.local) || (uni && ix[blk]); };

  const int blk0 = chunk * PL_CHUNK;
  const int tok_blk = (T - 1) / TILE;
  if (p.add_token && tok_blk >= blk0 && tok_blk < blk0 + PL_CHUNK) {   // D == 128 == PL_THREADS
    int64_t seq = b, row = T - 1;
    if (pages) {
      seq = pages[static_cast<int64_t>(b) * max_pages + tok_blk];
      row = (T - 1) % TILE;
      if (seq < 0 || seq >= num_pages) {   // a table entry outside the pool: nothing is read
        if (tid == 0) atomicCAS(&g_status, 0u, 0x300u);
        seq = -1;
      }
    }
    if (seq >= 0) {
      const __nv_bfloat16* kr = reinterpret_cast<const __nv_bfloat16*>(p.k) + seq * p.k_sb + h * p.k_sh + row * p.k_st;
      csum[static_cast<int64_t>(tok_blk) * PL_D + tid] += __bfloat162float(kr[tid]);
    }
  }
  __syncthreads();

  // 1. centroid scores of this chunk: a warp per block, lane owns dims 4*lane..4*lane+3
  float qv[PL_G][4];
#pragma unroll
  for (int g = 0; g < PL_G; ++g) {
    const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(p.q) + b * p.q_sb + (h * PL_G + g) * p.q_sh + 4 * lane;
#pragma unroll
    for (int e = 0; e < 4; ++e) qv[g][e] = __bfloat162float(qp[e]) * p.scale;
  }
  const int64_t row0 = (static_cast<int64_t>(b) * p.Hq + h * PL_G) * p.NBC;
  // Warp w takes the 8 consecutive blocks blk0 + 8w .. +7: 8 blocks x 4 heads = 32 dot products,
  // each the butterfly sum (lane distances 16, 8, 4, 2, 1) of 32 per-lane partials.  Instead of 32
  // butterflies in which every lane computes every sum, the 32 sums are reduced together: at
  // distance 16 a lane keeps the 16 sums whose index has the lane's bit 4 and hands the other 16
  // to its partner, and so on.  Every addition has the same two operands in the same order as in
  // the butterfly, so the bits are the same; lane j ends up with sum j.
  constexpr int U = PL_CHUNK / 4;
  static_assert(U * PL_G == 32, "one dot product per lane");
  {
    float a[32];   // a[4 * u + g]: this lane's partial of block u, head g
    const int wb = blk0 + warp * U;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int blk = wb + u;
      const float4 c = blk < nb ? *reinterpret_cast<const float4*>(csum + static_cast<int64_t>(blk) * PL_D + 4 * lane)
                                : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int g = 0; g < PL_G; ++g)
        a[4 * u + g] = qv[g][0] * c.x + qv[g][1] * c.y + qv[g][2] * c.z + qv[g][3] * c.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const bool up = (lane & o) != 0;
#pragma unroll
      for (int j = 0; j < o; ++j) {
        const float mine = up ? a[j + o] : a[j];
        const float theirs = up ? a[j] : a[j + o];
        a[j] = mine + __shfl_xor_sync(0xffffffffu, theirs, o);
      }
    }
    const int blk = wb + (lane >> 2), g = lane & 3;
    if (blk < nb) {
      const float inv_n = 1.f / static_cast<float>(blk == nb - 1 ? T - blk * TILE : TILE);
      p.cs_now[row0 + g * p.NBC + blk] = a[0] * inv_n;
    }
  }
  // count this chunk; only the last one of the head goes on
  __threadfence();
  __syncthreads();
  if (tid == 0) s_flag = atomicAdd(&done[bh], 1) == chunks - 1;
  __syncthreads();
  if (!s_flag) return;
  __threadfence();
  if (tid == 0) done[bh] = 0;

  // attended flags of every block into shared memory: independent, coalesced loads
  extern __shared__ unsigned char pl_att[];   // [nb]
  for (int i = tid; i < nb; i += PL_THREADS) pl_att[i] = attended(i) ? 1 : 0;
  __syncthreads();

  // 2. estimate of the mass outside the attended set: fold slot t takes blocks t, t+128, ...
  // (operands of four blocks are loaded before the dependent exp chain of the fold starts)
  float m[PL_G], s[PL_G];
#pragma unroll
  for (int g = 0; g < PL_G; ++g) {
    m[g] = -INFINITY;
    s[g] = 0.f;
  }
  for (int base = tid; base < nb; base += 4 * PL_THREADS) {
    float e[4][PL_G];
    bool use[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int blk = base + j * PL_THREADS;
      use[j] = blk < nb && !pl_att[blk];
      if (use[j]) {
#pragma unroll
        for (int g = 0; g < PL_G; ++g)
          e[j][g] = p.lse_ref[row0 + g * p.NBC + blk] + __ldcg(p.cs_now + row0 + g * p.NBC + blk) -
                    p.cs_ref[row0 + g * p.NBC + blk];
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (use[j]) {
#pragma unroll
        for (int g = 0; g < PL_G; ++g) pl_fold(m[g], s[g], e[j][g]);
      }
  }
  constexpr int NW = PL_THREADS / 32;
#pragma unroll
  for (int g = 0; g < PL_G; ++g) {
    const float M = warp_max(m[g]);
    const float S = warp_sum(s[g] > 0.f ? s[g] * __expf(m[g] - M) : 0.f);
    if (lane == 0) {
      wM[warp][g] = M;
      wS[warp][g] = S;
    }
  }
  __syncthreads();
  if (tid == 0) {
    float miss = 0.f;
    for (int g = 0; g < PL_G; ++g) {
      float M = -INFINITY, S = 0.f;
      for (int w = 0; w < NW; ++w)
        if (wS[w][g] > 0.f) M = fmaxf(M, wM[w][g]);
      for (int w = 0; w < NW; ++w)
        if (wS[w][g] > 0.f) S += wS[w][g] * __expf(wM[w][g] - M);
      if (S > 0.f) {
        const float est = M + __logf(S);
        miss = fmaxf(miss, 1.f / (1.f + __expf(p.lse_att[static_cast<int64_t>(b) * p.Hq + h * PL_G + g] - est)));
      }
    }
    if (p.est) p.est[bh] = miss;
    float dec = miss;
    if (p.calib && p.calib_on)
      dec = p.calib_kind ? miss + p.calib[bh] : 1.f / (1.f + __expf(-(pl_logit(miss) + p.calib[bh])));
    const int a = p.age[bh] + 1;
    const bool tr = dec > p.delta || a >= p.max_age || (fl & 1);
    p.age[bh] = tr ? 0 : a;
    p.trig[bh] = tr ? 1 : 0;
    s_flag = tr ? 1 : 0;
  }
  __syncthreads();

  // 3. block list of the attention pass
  if (s_flag) {
    for (int i = tid; i < nb; i += PL_THREADS) bi[i] = i;
    if (tid == 0) p.block_cnt[bh] = nb;
    return;
  }
  pl_compact(nb, bi, p.block_cnt + bh, scan, [&](int i) { return pl_att[i] != 0; });
}

// The top-p cut of one query head by one warp: 32 bisection steps on the threshold lo in
// [-80, 0] such that mass{y >= lo} >= level > mass{y >= hi}, y = x - lse.  Lane l owns blocks
// l, l+32, ... and sums exp(y) over its members in ascending order, then the butterfly: the order
// of the reference.  exp(y) is the same in every step, so it is evaluated once.  Once no block
// lies between lo and hi every further step sees the same set, so the kept set {y >= lo} can no
// longer change and the loop stops (the 32-step set is identical; lo itself is not an output).
// Register form: R values of y and exp(y) per lane, nb <= 32 R.
// ORDERED = false (block selection of the two-pass V-skip, which has no reference order to keep):
// four interleaved partial sums per lane instead of one chain of R dependent additions.
template <int R, bool ORDERED = true>
__device__ __forceinline__ float pl_bisect_regs(const float* x, const int nb, const int lane, const float lse,
                                                const float level) {
  float y[R], e[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
    y[r] = i < nb ? x[i] - lse : -INFINITY;
    e[r] = i < nb ? __expf(x[i] - lse) : 0.f;
  }
  float lo = -80.f, hi = 0.f;
  int n_lo = 0, n_hi = 0;       // blocks with y >= lo, y >= hi
#pragma unroll
  for (int r = 0; r < R; ++r) {
    n_lo += (y[r] >= lo) ? 1 : 0;
    n_hi += (y[r] >= hi) ? 1 : 0;
  }
  n_lo = __reduce_add_sync(0xffffffffu, n_lo);
  n_hi = __reduce_add_sync(0xffffffffu, n_hi);
  for (int it = 0; it < 32 && n_lo != n_hi; ++it) {
    const float mid = 0.5f * (lo + hi);
    float a = 0.f;
    int n_mid = 0;
    if constexpr (ORDERED) {
#pragma unroll
      for (int r = 0; r < R; ++r)
        if (y[r] >= mid) {
          a += e[r];
          ++n_mid;
        }
    } else {
      float a4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const bool in = y[r] >= mid;
        a4[r & 3] += in ? e[r] : 0.f;
        n_mid += in ? 1 : 0;
      }
      a = (a4[0] + a4[1]) + (a4[2] + a4[3]);
    }
    n_mid = __reduce_add_sync(0xffffffffu, n_mid);
    if (warp_sum(a) >= level) { lo = mid; n_lo = n_mid; } else { hi = mid; n_hi = n_mid; }
  }
  return lo;
}

// Shared-memory form for longer rows: ey[] receives exp(y).
__device__ __forceinline__ float pl_bisect_smem(const float* x, float* ey, const int nb, const int lane,
                                                const float lse, const float level) {
  for (int i = lane; i < nb; i += 32) ey[i] = __expf(x[i] - lse);
  float lo = -80.f, hi = 0.f;
  int n_lo = 0, n_hi = 0;
  for (int i = lane; i < nb; i += 32) {
    n_lo += (x[i] - lse >= lo) ? 1 : 0;
    n_hi += (x[i] - lse >= hi) ? 1 : 0;
  }
  n_lo = __reduce_add_sync(0xffffffffu, n_lo);
  n_hi = __reduce_add_sync(0xffffffffu, n_hi);
  for (int it = 0; it < 32 && n_lo != n_hi; ++it) {
    const float mid = 0.5f * (lo + hi);
    float a = 0.f;
    int n_mid = 0;
    for (int i = lane; i < nb; i += 32)
      if (x[i] - lse >= mid) {
        a += ey[i];
        ++n_mid;
      }
    n_mid = __reduce_add_sync(0xffffffffu, n_mid);
    if (warp_sum(a) >= level) { lo = mid; n_lo = n_mid; } else { hi = mid; n_hi = n_mid; }
  }
  return lo;
}

// With a device-resident length p.T bounds it and gives the row stride of the statistics.
__global__ void __launch_bounds__(PL_THREADS) update_kernel(const kvskip_update_params p,
                                                            const int* __restrict__ t_dev) {
  const int h = blockIdx.x, b = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nbs = (p.T + TILE - 1) / TILE;   // row stride of blk_max / blk_sum
  const int64_t bh = static_cast<int64_t>(b) * p.Hkv + h;
  const int64_t hrow = static_cast<int64_t>(b) * p.Hq + h * PL_G + warp;   // this warp's query head
  extern __shared__ float up_smem[];
  uint8_t* keep = p.keep + bh * p.NBC;
  pdl_wait_prior();          // statistics and decisions come from the kernels before this one
  pdl_launch_dependents();
  const int nb = (t_dev ? max(1, min(*t_dev, p.T)) + TILE - 1 : p.T + TILE - 1) / TILE;
  float* x = up_smem + warp * nb;                                          // block log-weights of the head
  float* ey = up_smem + (PL_G + warp) * nb;                                // exp(x - lse) of the head
  uint8_t* skeep = reinterpret_cast<uint8_t*>(up_smem + 2 * PL_G * nb);   // [nb] union of the new sets
  uint8_t* sflag = skeep + nb;   // [nb] bit 0: stored or always read, bit 1: joined through the token index
  const bool tr = p.trig[bh];
  __shared__ float s_real[PL_G];

  float mx = -INFINITY;
#pragma unroll 8
  for (int i = lane; i < nb; i += 32) {
    const float val = p.blk_max[hrow * nbs + i] + __logf(p.blk_sum[hrow * nbs + i]);   // -inf where not read
    x[i] = val;
    mx = fmaxf(mx, val);
  }
  {  // set membership flags once, with independent coalesced loads, instead of a global load per fold step
    const bool uni = tr && p.calib && ((p.flags[h] & 4) || (p.aix && p.aix[bh]));
    const uint8_t* ix = uni ? p.idx + static_cast<int64_t>(b) * p.NBC : nullptr;
#pragma unroll 4
    for (int i = tid; i < nb; i += PL_THREADS) {
      skeep[i] = 0;
      sflag[i] = ((keep[i] || pl_always(i, nb, p.local)) ? 1 : 0) | ((uni && ix[i]) ? 2 : 0);
    }
  }
  mx = warp_max(mx);
  __syncthreads();

  if (tr && p.calib) {   // mass the old attended set really missed (a refreshing head read every block)
    float mi = -INFINITY, si = 0.f, mo = -INFINITY, so = 0.f;
    for (int i = lane; i < nb; i += 32) {
      if (sflag[i]) pl_fold(mi, si, x[i]);
      else pl_fold(mo, so, x[i]);
    }
    const float Mi = warp_max(mi), Si = warp_sum(si > 0.f ? si * __expf(mi - Mi) : 0.f);
    const float Mo = warp_max(mo), So = warp_sum(so > 0.f ? so * __expf(mo - Mo) : 0.f);
    if (lane == 0) s_real[warp] = So > 0.f ? 1.f / (1.f + __expf((Mi + __logf(Si)) - (Mo + __logf(So)))) : 0.f;
  }
  if (tr) {
    float se = 0.f;
    for (int i = lane; i < nb; i += 32) se += __expf(x[i] - mx);
    const float lse = mx + __logf(warp_sum(se));
    // Top-p cut: lo such that mass{y >= lo} >= level, y = x - lse.  With up to 2048 blocks a lane's
    // values of y and exp(y) stay in registers for all 32 steps; longer rows use shared memory.
    float lo;
    if (nb <= 8 * 32) lo = pl_bisect_regs<8>(x, nb, lane, lse, p.level);
    else if (nb <= 16 * 32) lo = pl_bisect_regs<16>(x, nb, lane, lse, p.level);
    else if (nb <= 24 * 32) lo = pl_bisect_regs<24>(x, nb, lane, lse, p.level);
    else if (nb <= 32 * 32) lo = pl_bisect_regs<32>(x, nb, lane, lse, p.level);
    else if (nb <= 40 * 32) lo = pl_bisect_regs<40>(x, nb, lane, lse, p.level);
    else if (nb <= 48 * 32) lo = pl_bisect_regs<48>(x, nb, lane, lse, p.level);
    else if (nb <= 64 * 32) lo = pl_bisect_regs<64>(x, nb, lane, lse, p.level);
    else lo = pl_bisect_smem(x, ey, nb, lane, lse, p.level);
    for (int i = lane; i < nb; i += 32)
      if (x[i] - lse >= lo) skeep[i] = 1;
    // new references: the centroid scores are fetched eight at a time before anything is stored
    // (the compiler may not move a load above a store through another pointer of the same type,
    // so a load-store loop would pay one memory round trip per iteration)
    constexpr int RU = 8;
    for (int base = lane; base < p.NBC; base += 32 * RU) {
      float c[RU];
#pragma unroll
      for (int j = 0; j < RU; ++j) {
        const int i = base + 32 * j;
        c[j] = i < nb ? p.cs_now[hrow * p.NBC + i] : 0.f;
      }
#pragma unroll
      for (int j = 0; j < RU; ++j) {
        const int i = base + 32 * j;
        if (i < p.NBC) {
          p.lse_ref[hrow * p.NBC + i] = i < nb ? x[i] : -INFINITY;
          p.cs_ref[hrow * p.NBC + i] = c[j];
        }
      }
    }
  }
  __syncthreads();
  if (tr && p.calib && tid == 0) {
    float real = 0.f;
    for (int g = 0; g < PL_G; ++g) real = fmaxf(real, s_real[g]);
    const float est = p.est[bh];
    const float resid = p.calib_kind ? real - est : pl_logit(real) - pl_logit(est);
    float c = p.calib_kind == 2 ? fmaxf((1.f - p.calib_rate) * p.calib[bh], resid)
                                : (1.f - p.calib_rate) * p.calib[bh] + p.calib_rate * resid;
    if (!p.calib_free) c = fmaxf(c, 0.f);
    p.calib[bh] = c;
    if (p.aix && c > p.aix_thr) p.aix[bh] = 1;
  }
  if (tr)
    for (int i = tid; i < p.NBC; i += PL_THREADS) {
      const uint8_t kept = (i < nb && (skeep[i] || pl_always(i, nb, p.local))) ? 1 : 0;
      keep[i] = kept;
      if (i < nb) sflag[i] = kept;
    }
  __syncthreads();
  float m2 = -INFINITY, s2 = 0.f;
  for (int i = lane; i < nb; i += 32)
    if (sflag[i] & 1) pl_fold(m2, s2, x[i]);
  const float M = warp_max(m2);
  const float S = warp_sum(s2 > 0.f ? s2 * __expf(m2 - M) : 0.f);
  if (lane == 0) p.lse_att[hrow] = M + __logf(S);
}

// Token-index blocks of one step: grid (ceil(T/256), n).  A position t < T-1 holding the current
// token marks its own block and the block of t+1.
__global__ void __launch_bounds__(256) index_blocks_kernel(const int64_t* __restrict__ ids, int64_t stride,
                                                           int T, uint8_t* out, int NBC,
                                                           const int* __restrict__ t_dev) {
  if (t_dev) T = max(1, min(*t_dev, T));   // device-resident length, bounded by the launch's T
  const int r = blockIdx.y;
  const int64_t* x = ids + r * stride;
  const int64_t cur = x[T - 1];
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < T - 1 && x[t] == cur) {
    out[static_cast<int64_t>(r) * NBC + t / TILE] = 1;
    out[static_cast<int64_t>(r) * NBC + (t + 1) / TILE] = 1;
  }
}

// Block selection between the two passes of the two-pass V-skip, on the device: what the
// reference's caller does with a dozen torch launches (format37/kvskip kernels/kvskip.py:122-147
// select_blocks, :165-177 the weights of vskip_two_pass, :70-85 make_plan).  Grid (Hkv, B), a warp
// per query head.  Per head: block log-weights x = blk_max + log blk_sum, their log-sum-exp, and
//   rule 0 ("topp")  the fewest heaviest blocks whose mass reaches `value`: the same bisection as
//                    update_kernel's top-p cut (kept set {x - lse >= lo});
//   rule 1 ("tau")   blocks whose weight exp(x - lse) is at least `value`.
// The kv head keeps the union over its four heads plus block 0 and the `local` newest.  Outputs:
// keep u8 [B,Hkv,nb], the ascending block list and its length, and for the second pass the
// weights exp(blk_max - lse_kept) [B,Hkv,nb,4] (0 on blocks not kept), lse_kept = log-sum-exp of
// x over the kept set.
// With a device-resident length (t_dev != nullptr, T_bound its bound) nbs = ceil(T_bound / 64) stays
// the row stride of every array and the selection runs over the blocks of the current length.
__global__ void __launch_bounds__(PL_THREADS) select_kernel(const float* __restrict__ blk_max,
                                                            const float* __restrict__ blk_sum, const int nbs,
                                                            const int Hkv, const int rule, const float value,
                                                            const int local, uint8_t* __restrict__ keep,
                                                            int32_t* __restrict__ block_idx,
                                                            int32_t* __restrict__ block_cnt,
                                                            float* __restrict__ weight,
                                                            const int* __restrict__ t_dev, const int T_bound) {
  const int h = blockIdx.x, b = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t bh = static_cast<int64_t>(b) * Hkv + h;
  const int64_t hrow = bh * PL_G + warp;
  extern __shared__ float sel_smem[];
  float* x = sel_smem + warp * nbs;
  float* ey = sel_smem + (PL_G + warp) * nbs;
  uint8_t* skeep = reinterpret_cast<uint8_t*>(sel_smem + 2 * PL_G * nbs);
  __shared__ int scan[PL_THREADS];
  pdl_wait_prior();          // the statistics come from the kernel before this one
  pdl_launch_dependents();
  const int nb = t_dev ? (max(1, min(*t_dev, T_bound)) + TILE - 1) / TILE : nbs;   // blocks of the current length

  const bool in_regs = nb <= 64 * 32;     // the bisection keeps its values in registers: ey[] is free
  float mx = -INFINITY;
#pragma unroll 16
  for (int i = lane; i < nb; i += 32) {
    const float bm = blk_max[hrow * nbs + i];
    const float val = bm + __logf(blk_sum[hrow * nbs + i]);
    x[i] = val;
    if (in_regs) ey[i] = bm;              // block maxima for the weights, no second trip to global memory
    mx = fmaxf(mx, val);
  }
  for (int i = tid; i < nb; i += PL_THREADS) skeep[i] = pl_always(i, nb, local) ? 1 : 0;
  mx = warp_max(mx);
  __syncthreads();
  float se = 0.f;
  for (int i = lane; i < nb; i += 32) se += __expf(x[i] - mx);
  const float lse = mx + __logf(warp_sum(se));
  float lo;
  if (rule == 0) {
    if (nb <= 8 * 32) lo = pl_bisect_regs<8, false>(x, nb, lane, lse, value);
    else if (nb <= 16 * 32) lo = pl_bisect_regs<16, false>(x, nb, lane, lse, value);
    else if (nb <= 32 * 32) lo = pl_bisect_regs<32, false>(x, nb, lane, lse, value);
    else if (nb <= 64 * 32) lo = pl_bisect_regs<64, false>(x, nb, lane, lse, value);
    else lo = pl_bisect_smem(x, ey, nb, lane, lse, value);
  } else {
    lo = __logf(value);
  }
  for (int i = lane; i < nb; i += 32)
    if (rule == 0 ? (x[i] - lse >= lo) : (__expf(x[i] - lse) >= value)) skeep[i] = 1;
  __syncthreads();
  // weights of the second pass, relative to the mass of the kept set
  float m2 = -INFINITY, s2 = 0.f;
  for (int i = lane; i < nb; i += 32)
    if (skeep[i]) pl_fold(m2, s2, x[i]);
  const float M = warp_max(m2);
  const float S = warp_sum(s2 > 0.f ? s2 * __expf(m2 - M) : 0.f);
  const float lse_kept = M + __logf(S);
  for (int i = lane; i < nb; i += 32)
    weight[(bh * nbs + i) * PL_G + warp] =
        skeep[i] ? __expf((in_regs ? ey[i] : blk_max[hrow * nbs + i]) - lse_kept) : 0.f;
  for (int i = tid; i < nbs; i += PL_THREADS) keep[bh * nbs + i] = i < nb ? skeep[i] : 0;
  for (int i = nb + lane; i < nbs; i += 32) weight[(bh * nbs + i) * PL_G + warp] = 0.f;
  pl_compact(nb, block_idx + bh * nbs, block_cnt + bh, scan, [&](int i) { return skeep[i] != 0; });
}

// The new token's K and V rows into the cache: grid (Hkv, B) x D/8 threads, 16 bytes per thread
// and tensor.  T (or *t_dev) is the length after the append, so the row is T-1; with a page table
// it is row (T-1) % 64 of page pages[b, (T-1) / 64].
__global__ void append_kernel(uint16_t* __restrict__ k, uint16_t* __restrict__ v, const int64_t sb, const int64_t sh,
                              const int64_t st, const uint16_t* __restrict__ k_new, const uint16_t* __restrict__ v_new,
                              const int D, int T, const int* __restrict__ t_dev, const int32_t* __restrict__ pages,
                              const int max_pages, const int num_pages) {
  const int h = blockIdx.x, b = blockIdx.y, Hkv = gridDim.x;
  if (t_dev) T = max(1, min(*t_dev, T));
  int64_t seq = b, row = T - 1;
  if (pages) {
    seq = pages[static_cast<int64_t>(b) * max_pages + (T - 1) / TILE];
    row = (T - 1) % TILE;
    if (seq < 0 || seq >= num_pages) {
      if (threadIdx.x == 0) atomicCAS(&g_status, 0u, 0x301u);
      return;
    }
  }
  const int64_t dst = seq * sb + h * sh + row * st + 8 * threadIdx.x;
  const int64_t src = (static_cast<int64_t>(b) * Hkv + h) * D + 8 * threadIdx.x;
  *reinterpret_cast<uint4*>(k + dst) = *reinterpret_cast<const uint4*>(k_new + src);
  *reinterpret_cast<uint4*>(v + dst) = *reinterpret_cast<const uint4*>(v_new + src);
}

// The device-resident sequence length of a captured decode step: one thread adds delta.
__global__ void advance_kernel(int* t, int delta) { *t += delta; }

}  // namespace kvb
