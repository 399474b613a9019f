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
// bandwidth: `plan` spreads a head's centroid scores over the CTAs of a thread-block cluster, which
// hand scores, fold operands and attended flags to the cluster's first CTA through its shared
// memory (plan_cluster_kernel; plan_kernel, with a counter in global memory, for heads whose table
// does not fit there); every load of a phase is requested before the first is used, and the fold
// is written with selects so that the four query heads' chains overlap.  A head costs a handful of
// memory round trips, whatever its length.
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

// running log-sum-exp (m, s), s relative to m.  Written with selects instead of branches: a warp
// whose lanes disagree on e > m would run both sides one after the other, and the four folds of a
// block (one per query head) could not overlap.  The operations and their operands are those of
//   if (e == -inf) return;  if (e > m) { s = s * exp(m - e) + 1; m = e; } else s += exp(e - m);
__device__ __forceinline__ void pl_fold(float& m, float& s, float e) {
  const bool up = e > m;
  const float t = __expf(up ? m - e : e - m);
  const float s_up = s * t + 1.f, s_same = s + t;
  const bool skip = e == -INFINITY;
  s = skip ? s : (up ? s_up : s_same);
  m = (up && !skip) ? e : m;
}

// Ascending compaction of the blocks satisfying `pred` into bi[]; count to *cnt.  Thread t owns a
// contiguous chunk; the offsets come from a shuffle scan inside each warp and the four warp totals
// in `scan`.  Must be called by all PL_THREADS threads.
template <typename Pred>
__device__ __forceinline__ void pl_compact(int nb, int* bi, int* cnt, int* scan, Pred pred) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int per = (nb + PL_THREADS - 1) / PL_THREADS;
  const int a = min(nb, tid * per), e = min(nb, a + per);
  int c = 0;
  for (int i = a; i < e; ++i) c += pred(i) ? 1 : 0;
  int inc = c;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += up;
  }
  __syncthreads();           // (scan may still be read by an earlier call)
  if (lane == 31) scan[warp] = inc;
  __syncthreads();
  int off = inc - c, total = 0;
#pragma unroll
  for (int w = 0; w < PL_THREADS / 32; ++w) {
    const int t = scan[w];
    if (w < warp) off += t;
    total += t;
  }
  for (int i = a; i < e; ++i)
    if (pred(i)) bi[off++] = i;
  if (tid == 0) *cnt = total;
}

// The end of `plan` for one (batch, kv head), by the CTA that holds the 128 fold slots (m, s): the
// slots merge per warp (max, butterfly of rescaled sums), the four groups merge serially in
// ascending order, the largest miss of the four query heads decides, and the block list is written:
// every block on a refresh, else the attended ones (att[], one byte per block in shared memory).
// lse_att (threads 0..3), calib and age (thread 0) were loaded by the caller ahead of time.
__device__ __forceinline__ void pl_decide_list(const kvskip_plan_params& p, float (&m)[PL_G], float (&s)[PL_G],
                                               const float lse_att, const float calib, const int age, const int fl,
                                               const int nb, const int64_t bh, int* bi, const unsigned char* pl_att,
                                               int* scan, float (*wM)[PL_G], float (*wS)[PL_G], int* s_flag_p) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int& s_flag = *s_flag_p;
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
  if (warp == 0) {   // lane g < 4 merges the four groups of head g in ascending order; the largest miss decides
    float miss = 0.f;
    if (lane < PL_G) {
      const int g = lane;
      float M = -INFINITY, S = 0.f;
      for (int w = 0; w < NW; ++w)
        if (wS[w][g] > 0.f) M = fmaxf(M, wM[w][g]);
      for (int w = 0; w < NW; ++w)
        if (wS[w][g] > 0.f) S += wS[w][g] * __expf(wM[w][g] - M);
      if (S > 0.f) {
        const float est = M + __logf(S);
        miss = fmaxf(miss, 1.f / (1.f + __expf(lse_att - est)));
      }
    }
    miss = warp_max(miss);
    if (lane == 0) {
      if (p.est) p.est[bh] = miss;
      float dec = miss;
      if (p.calib && p.calib_on) dec = p.calib_kind ? miss + calib : 1.f / (1.f + __expf(-(pl_logit(miss) + calib)));
      const int a = age + 1;
      const bool tr = dec > p.delta || a >= p.max_age || (fl & 1);
      p.age[bh] = tr ? 0 : a;
      p.trig[bh] = tr ? 1 : 0;
      s_flag = tr ? 1 : 0;
    }
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

constexpr int PL_CHUNK = 32;   // blocks of one round of a CTA's centroid scores (4 warps x 8 in flight)

// grid (ceil(nb / (32 ROUNDS)), Hkv, B).  Every CTA computes the centroid scores of its chunk of
// 32 ROUNDS blocks and stores them to cs_now; the last CTA of a (batch, kv head) to finish (counted
// in done[], which it puts back to zero) folds the estimate, decides and writes the block list.
// The arithmetic of a score and of the fold is unchanged, only spread over more SMs: one CTA per
// head reading nb * 512 bytes of key sums is latency-bound at long contexts.  ROUNDS is chosen by
// the host so that a launch has a few CTAs per SM: the SMs start a CTA every ~0.4 us each, so a grid
// of thousands of 3 us CTAs is bound by the rate at which CTAs start, not by their work.
// A head costs a fixed number of memory round trips, whatever its length: every load of a phase is
// issued before the first use (no load sits behind a branch on another load's value).
// With a device-resident length (t_dev != nullptr) p.T is the bound the grid was sized for; CTAs
// whose chunk lies beyond the current length leave without being counted.
// With a paged cache (pages != nullptr) p.k is the page pool [pages, Hkv, 64, D] (k_sb = page stride)
// and the key of the new token is row (T-1) % 64 of page pages[b, (T-1) / 64].
template <int ROUNDS>
__global__ void __launch_bounds__(PL_THREADS) plan_kernel(const kvskip_plan_params p, int* __restrict__ done,
                                                          const int* __restrict__ t_dev,
                                                          const int32_t* __restrict__ pages, const int max_pages,
                                                          const int num_pages) {
  constexpr int CHUNK = PL_CHUNK * ROUNDS;
  const int chunk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t bh = static_cast<int64_t>(b) * p.Hkv + h;
  float* csum = p.csum + bh * p.NBC * PL_D;
  const uint8_t* keep = p.keep + bh * p.NBC;
  int* bi = p.block_idx + bh * p.NBC;
  __shared__ int scan[PL_THREADS / 32];
  __shared__ float wM[PL_THREADS / 32][PL_G], wS[PL_THREADS / 32][PL_G];
  __shared__ int s_flag;
  extern __shared__ unsigned char pl_att[];   // [nb] attended flags of the head
  pdl_wait_prior();          // the state this kernel reads may come from the previous kernel on the stream
  pdl_launch_dependents();
  const int T = t_dev ? max(1, min(*t_dev, p.T)) : p.T;
  const int nb = (T + TILE - 1) / TILE;
  const int chunks = (nb + CHUNK - 1) / CHUNK;
  if (chunk >= chunks) return;

  const int fl = p.flags[h];
  const bool latched = p.aix && p.aix[bh];
  if (fl & 2) {   // token-index head: index blocks + sink + newest, never refreshes; one CTA does it
    if (chunk != 0) return;
    const uint8_t* ix = p.idx + static_cast<int64_t>(b) * p.NBC;
    pl_compact(nb, bi, p.block_cnt + bh, scan, [&](int i) { return ix[i] || pl_always(i, nb, p.local); });
    if (tid == 0) p.trig[bh] = 0;
    return;
  }
  const bool uni = (fl & 4) || latched;
  const uint8_t* ix = uni ? p.idx + static_cast<int64_t>(b) * p.NBC : keep;   // (read unconditionally below)

  const int blk0 = chunk * CHUNK;
  const int tok_blk = (T - 1) / TILE;
  if (p.add_token && tok_blk >= blk0 && tok_blk < blk0 + CHUNK) {   // D == 128 == PL_THREADS
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
    __syncthreads();
  }

  // 1. centroid scores of this chunk: a warp per block, lane owns dims 4*lane..4*lane+3
  float qv[PL_G][4];
#pragma unroll
  for (int g = 0; g < PL_G; ++g) {
    const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(p.q) + b * p.q_sb + (h * PL_G + g) * p.q_sh + 4 * lane;
#pragma unroll
    for (int e = 0; e < 4; ++e) qv[g][e] = __bfloat162float(qp[e]) * p.scale;
  }
  const int64_t row0 = (static_cast<int64_t>(b) * p.Hq + h * PL_G) * p.NBC;
  // In a round warp w takes the 8 consecutive blocks blk0 + 32 r + 8w .. +7: 8 blocks x 4 heads =
  // 32 dot products, each the butterfly sum (lane distances 16, 8, 4, 2, 1) of 32 per-lane partials.
  // Instead of 32 butterflies in which every lane computes every sum, the 32 sums are reduced
  // together: at distance 16 a lane keeps the 16 sums whose index has the lane's bit 4 and hands
  // the other 16 to its partner, and so on.  Every addition has the same two operands in the same
  // order as in the butterfly, so the bits are the same; lane j ends up with sum j.  The key sums
  // of the next round are requested before this round's reduction.
  constexpr int U = PL_CHUNK / 4;
  static_assert(U * PL_G == 32, "one dot product per lane");
  auto fetch = [&](float4 (&c)[U], const int r) {
    const int wb = blk0 + r * PL_CHUNK + warp * U;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int blk = wb + u;
      c[u] = blk < nb ? *reinterpret_cast<const float4*>(csum + static_cast<int64_t>(blk) * PL_D + 4 * lane)
                      : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  float4 c[U], cn[U];
  fetch(c, 0);
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
    if (r + 1 < ROUNDS) fetch(cn, r + 1);
    float a[32];   // a[4 * u + g]: this lane's partial of block u, head g
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int g = 0; g < PL_G; ++g)
        a[4 * u + g] = qv[g][0] * c[u].x + qv[g][1] * c[u].y + qv[g][2] * c[u].z + qv[g][3] * c[u].w;
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
    const int blk = blk0 + r * PL_CHUNK + warp * U + (lane >> 2), g = lane & 3;
    if (blk < nb) {
      const float inv_n = 1.f / static_cast<float>(blk == nb - 1 ? T - blk * TILE : TILE);
      p.cs_now[row0 + g * p.NBC + blk] = a[0] * inv_n;
    }
    if (r + 1 < ROUNDS) {
#pragma unroll
      for (int u = 0; u < U; ++u) c[u] = cn[u];
    }
  }
  // count this chunk; only the last one of the head goes on.  While the counter's round trip is
  // under way every CTA stages the head's attended flags (a byte or two per block, from state that
  // no CTA of this launch writes) and the scalars of the decision: the last CTA finds them ready.
  __threadfence();
  __syncthreads();
  int prev = 0;
  if (tid == 0) prev = atomicAdd(&done[bh], 1);
  for (int i = tid; i < nb; i += PL_THREADS) {
    const uint8_t kp = keep[i], xi = ix[i];
    pl_att[i] = (kp || pl_always(i, nb, p.local) || (uni && xi)) ? 1 : 0;
  }
  const float lse_att = tid < PL_G ? p.lse_att[static_cast<int64_t>(b) * p.Hq + h * PL_G + tid] : 0.f;
  const float calib = (tid == 0 && p.calib && p.calib_on) ? p.calib[bh] : 0.f;
  const int age = tid == 0 ? p.age[bh] : 0;
  if (tid == 0) s_flag = prev == chunks - 1;
  __syncthreads();
  if (!s_flag) return;
  __threadfence();
  if (tid == 0) done[bh] = 0;

  // 2. estimate of the mass outside the attended set: fold slot t takes blocks t, t+128, ...
  // The operands of eight blocks are requested at once, attended or not (an unused block costs
  // three loads, a load behind a test of the flag would cost a round trip per block), before the
  // dependent exp chain of the fold starts.
  float m[PL_G], s[PL_G];
#pragma unroll
  for (int g = 0; g < PL_G; ++g) {
    m[g] = -INFINITY;
    s[g] = 0.f;
  }
  constexpr int FJ = 8;
  for (int base = tid; base < nb; base += FJ * PL_THREADS) {
    float ra[FJ][PL_G], rb[FJ][PL_G], rc[FJ][PL_G];
#pragma unroll
    for (int j = 0; j < FJ; ++j) {
      const int64_t at = row0 + min(base + j * PL_THREADS, nb - 1);
#pragma unroll
      for (int g = 0; g < PL_G; ++g) {
        ra[j][g] = __ldg(p.lse_ref + at + g * p.NBC);
        rc[j][g] = __ldg(p.cs_ref + at + g * p.NBC);
      }
    }
#pragma unroll
    for (int j = 0; j < FJ; ++j) {
      const int64_t at = row0 + min(base + j * PL_THREADS, nb - 1);
#pragma unroll
      for (int g = 0; g < PL_G; ++g) rb[j][g] = __ldcg(p.cs_now + at + g * p.NBC);
    }
#pragma unroll
    for (int j = 0; j < FJ; ++j) {
      const int blk = base + j * PL_THREADS;
      if (blk < nb && !pl_att[min(blk, nb - 1)]) {
#pragma unroll
        for (int g = 0; g < PL_G; ++g) pl_fold(m[g], s[g], ra[j][g] + rb[j][g] - rc[j][g]);
      }
    }
  }
  pl_decide_list(p, m, s, lse_att, calib, age, fl, nb, bh, bi, pl_att, scan, wM, wS, &s_flag);
}

// `plan` on a thread-block cluster: grid (C, Hkv, B) with the C CTAs of a (batch, kv head) forming
// one cluster (C = 1, 2, 4 or 8, chosen by the host so that a launch has a few CTAs per SM).  The 32-
// block rounds of the head are dealt out evenly; a CTA computes the centroid scores of its rounds
// (the same arithmetic as plan_kernel), stores them to cs_now for `update`, and puts what the fold
// needs -- e = lse_ref + cs_now - cs_ref per query head and the attended flag of the block --
// straight into the shared memory of the cluster's first CTA.  Every thread then arrives on an
// mbarrier of that CTA (release at cluster scope); the first CTA waits for it (bounded), folds from
// its own shared memory, decides and writes the list.  Against the counter version this takes the
// global-memory hand-over out of a head's chain: no fence + atomic round trip, no reload of three
// arrays by one SM.  The operands of e belong to state no CTA of this launch writes, so they are
// requested together with the key sums.  Shared memory of a CTA: 17 bytes per block of the head.
// Every CTA of a cluster takes the same branches up to its arrival: the only early exit (a token-
// index head) depends on the head alone, and with a device-resident length all CTAs see the same nb.
__global__ void __launch_bounds__(PL_THREADS) plan_cluster_kernel(const kvskip_plan_params p,
                                                                  const int* __restrict__ t_dev,
                                                                  const int32_t* __restrict__ pages,
                                                                  const int max_pages, const int num_pages) {
  const int rank = static_cast<int>(cluster_ctarank()), C = static_cast<int>(cluster_nctarank());
  const int h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t bh = static_cast<int64_t>(b) * p.Hkv + h;
  float* csum = p.csum + bh * p.NBC * PL_D;
  const uint8_t* keep = p.keep + bh * p.NBC;
  int* bi = p.block_idx + bh * p.NBC;
  __shared__ int scan[PL_THREADS / 32];
  __shared__ float wM[PL_THREADS / 32][PL_G], wS[PL_THREADS / 32][PL_G];
  __shared__ int s_flag;
  __shared__ __align__(8) uint64_t arrived;
  extern __shared__ __align__(16) unsigned char pl_dyn[];   // first CTA: e [nbs][4] floats, then attended [nbs]
  const int nbs = (p.T + TILE - 1) / TILE;                  // blocks of the bound: the layout of pl_dyn
  if (rank == 0 && tid == 0 && C > 1) {
    mbar_init(&arrived, static_cast<uint32_t>((C - 1) * PL_THREADS));
    mbar_fence_init();
  }
  cluster_arrive();          // (its wait, below, is what makes the initialised barrier visible to the others)
  pdl_wait_prior();          // the state this kernel reads may come from the previous kernel on the stream
  pdl_launch_dependents();
  const int T = t_dev ? max(1, min(*t_dev, p.T)) : p.T;
  const int nb = (T + TILE - 1) / TILE;
  const int rounds = (nb + PL_CHUNK - 1) / PL_CHUNK;
  const int r0 = rank * rounds / C, r1 = (rank + 1) * rounds / C;   // this CTA's rounds

  const int64_t row0 = (static_cast<int64_t>(b) * p.Hq + h * PL_G) * p.NBC;
  // (read unconditionally, so that a round's loads do not wait for the head's flags)
  const uint8_t* ix = p.idx ? p.idx + static_cast<int64_t>(b) * p.NBC : keep;
  constexpr int U = PL_CHUNK / 4;
  static_assert(U * PL_G == 32, "one dot product per lane");
  // what a lane needs of a round: the key sums of the warp's 8 blocks (its 4 dims each) and, for the
  // (block, head) pair whose score it ends up with, the two references and the block's flags
  struct Round {
    float4 c[U];
    float lref, cref;
    uint8_t kp, xi;
  };
  const int my_u = lane >> 2, my_g = lane & 3;
  auto fetch = [&](Round& x, const int r) {
    const int wb = r * PL_CHUNK + warp * U;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int blk = wb + u;
      x.c[u] = blk < nb ? *reinterpret_cast<const float4*>(csum + static_cast<int64_t>(blk) * PL_D + 4 * lane)
                        : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const int blk = min(wb + my_u, nb - 1);
    x.lref = p.lse_ref[row0 + my_g * p.NBC + blk];
    x.cref = p.cs_ref[row0 + my_g * p.NBC + blk];
    x.kp = keep[blk];
    x.xi = ix[blk];
  };
  // The first round is requested before anything that depends on a load (the head's flags); only
  // the CTA that first adds the new token's key to its block's sum has to wait with it.
  const int tok_blk = (T - 1) / TILE;
  const bool has_tok = p.add_token && tok_blk >= r0 * PL_CHUNK && tok_blk < r1 * PL_CHUNK;
  Round cur, nxt;
  if (!has_tok && r0 < r1) fetch(cur, r0);
  float qv[PL_G][4];
#pragma unroll
  for (int g = 0; g < PL_G; ++g) {
    const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(p.q) + b * p.q_sb + (h * PL_G + g) * p.q_sh + 4 * lane;
#pragma unroll
    for (int e = 0; e < 4; ++e) qv[g][e] = __bfloat162float(qp[e]) * p.scale;
  }

  const int fl = p.flags[h];
  const bool latched = p.aix && p.aix[bh];
  if (fl & 2) {   // token-index head: index blocks + sink + newest, never refreshes; one CTA does it
    if (rank != 0) return;
    pl_compact(nb, bi, p.block_cnt + bh, scan, [&](int i) { return ix[i] || pl_always(i, nb, p.local); });
    if (tid == 0) p.trig[bh] = 0;
    return;
  }
  const bool uni = (fl & 4) || latched;
  // scalars of the decision, ahead of time
  const float lse_att = (rank == 0 && tid < PL_G) ? p.lse_att[static_cast<int64_t>(b) * p.Hq + h * PL_G + tid] : 0.f;
  const float calib = (rank == 0 && tid == 0 && p.calib && p.calib_on) ? p.calib[bh] : 0.f;
  const int age = (rank == 0 && tid == 0) ? p.age[bh] : 0;

  if (has_tok) {   // D == 128 == PL_THREADS
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
    __syncthreads();
    fetch(cur, r0);
  }
  const uint32_t e_remote = cluster_map(smem_u32(pl_dyn), 0);
  const uint32_t att_remote = e_remote + 16u * static_cast<uint32_t>(nbs);
  bool waited = false;
  for (int r = r0; r < r1; ++r) {
    if (r + 1 < r1) fetch(nxt, r + 1);
    float a[32];   // a[4 * u + g]: this lane's partial of block u, head g
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int g = 0; g < PL_G; ++g)
        a[4 * u + g] = qv[g][0] * cur.c[u].x + qv[g][1] * cur.c[u].y + qv[g][2] * cur.c[u].z + qv[g][3] * cur.c[u].w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {   // the 32 butterflies reduced together, see plan_kernel
      const bool up = (lane & o) != 0;
#pragma unroll
      for (int j = 0; j < o; ++j) {
        const float mine = up ? a[j + o] : a[j];
        const float theirs = up ? a[j] : a[j + o];
        a[j] = mine + __shfl_xor_sync(0xffffffffu, theirs, o);
      }
    }
    if (!waited) {           // the first CTA runs and its barrier is initialised: its shared memory may be written
      cluster_wait();
      waited = true;
    }
    const int blk = r * PL_CHUNK + warp * U + my_u;
    if (blk < nb) {
      const float inv_n = 1.f / static_cast<float>(blk == nb - 1 ? T - blk * TILE : TILE);
      const float cs = a[0] * inv_n;
      p.cs_now[row0 + my_g * p.NBC + blk] = cs;
      cluster_st_f32(e_remote + 4u * static_cast<uint32_t>(blk * PL_G + my_g), cur.lref + cs - cur.cref);
      if (my_g == 0)
        cluster_st_u8(att_remote + static_cast<uint32_t>(blk),
                      (cur.kp || pl_always(blk, nb, p.local) || (uni && cur.xi)) ? 1u : 0u);
    }
    cur = nxt;
  }
  if (!waited) cluster_wait();
  if (rank != 0) {
    cluster_mbar_arrive(cluster_map(smem_u32(&arrived), 0));
    return;
  }
  __syncthreads();           // this CTA's own rounds are in its shared memory
  // (The CTAs of a cluster are scheduled together and every one of them arrives unconditionally, so
  // this wait can only run out if a peer is stuck; the bound turns that into status word 0x310 and
  // an unwritten list instead of a hang.)
  if (C > 1 && !cluster_mbar_wait(&arrived, 0, 0x310u)) return;

  // estimate of the mass outside the attended set: fold slot t takes blocks t, t+128, ...
  const float4* e4 = reinterpret_cast<const float4*>(pl_dyn);
  const unsigned char* pl_att = pl_dyn + 16 * static_cast<size_t>(nbs);
  float m[PL_G], s[PL_G];
#pragma unroll
  for (int g = 0; g < PL_G; ++g) {
    m[g] = -INFINITY;
    s[g] = 0.f;
  }
  for (int blk = tid; blk < nb; blk += PL_THREADS) {
    if (pl_att[blk]) continue;
    const float4 e = e4[blk];
    pl_fold(m[0], s[0], e.x);
    pl_fold(m[1], s[1], e.y);
    pl_fold(m[2], s[2], e.z);
    pl_fold(m[3], s[3], e.w);
  }
  pl_decide_list(p, m, s, lse_att, calib, age, fl, nb, bh, bi, pl_att, scan, wM, wS, &s_flag);
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

  // Statistics and flags: sixteen (eight) loads per thread are requested before the first is used.
  float mx = -INFINITY;
  constexpr int XB = 16;
  for (int base = lane; base < nb; base += 32 * XB) {
    float bm[XB], bs[XB];
#pragma unroll
    for (int j = 0; j < XB; ++j) {
      const int i = min(base + 32 * j, nb - 1);
      bm[j] = p.blk_max[hrow * nbs + i];
      bs[j] = p.blk_sum[hrow * nbs + i];
    }
#pragma unroll
    for (int j = 0; j < XB; ++j) {
      const int i = base + 32 * j;
      if (i < nb) {
        const float val = bm[j] + __logf(bs[j]);   // -inf where not read
        x[i] = val;
        mx = fmaxf(mx, val);
      }
    }
  }
  {  // set membership flags once, with independent coalesced loads, instead of a global load per fold step
    const bool uni = tr && p.calib && ((p.flags[h] & 4) || (p.aix && p.aix[bh]));
    const uint8_t* ix = uni ? p.idx + static_cast<int64_t>(b) * p.NBC : keep;   // (loaded either way: no load behind a branch)
    constexpr int FB = 8;
    for (int base = tid; base < nb; base += PL_THREADS * FB) {
      uint8_t kp[FB], xi[FB];
#pragma unroll
      for (int j = 0; j < FB; ++j) {
        const int i = min(base + PL_THREADS * j, nb - 1);
        kp[j] = keep[i];
        xi[j] = ix[i];
      }
#pragma unroll
      for (int j = 0; j < FB; ++j) {
        const int i = base + PL_THREADS * j;
        if (i < nb) {
          skeep[i] = 0;
          sflag[i] = ((kp[j] || pl_always(i, nb, p.local)) ? 1 : 0) | ((uni && xi[j]) ? 2 : 0);
        }
      }
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
