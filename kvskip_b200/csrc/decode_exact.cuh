// Split-K flash-decoding on CUDA cores with the reference's float operation order
// ("exact-order" path): scores, block maxima and block sums come out bit-identical to
// format37/kvskip's decode_kernel (kernels/kvskip_kernel.cu:69-292) compiled for the same GPU,
// which is what lets the refresh planner downstream reproduce the reference's decisions.
//
// Data movement is sm_100a-native: one elected thread streams 64-token K (and V) blocks with
// tiled TMA loads (cp.async.bulk.tensor, 4-D map over [B,Hkv,T,D], rows past T zero-filled by the
// copy engine) into a ring of shared-memory stages, each guarded by an mbarrier that the copy
// completes by byte count.  One CTA per (split, kv head, batch) serves the four query heads of
// the KV head, so every block is read once.
//
// Arithmetic order kept from the reference (it defines the bits of the statistics):
//   score(row)  eight fused-multiply-add chains, chain j over dims 8j..8j+7 (then 64+8j.. for
//               D = 128), merged by a distance-4, 2, 1 butterfly;
//   block max   order free;  block sum: token i paired with token i+32, then a 32-lane butterfly;
//   running l   l * 2^(m_old - m_new) + butterfly(pair sums), per block in list order.
#pragma once
#include "common.cuh"

namespace kvb {

constexpr int EX_THREADS = 128;   // 4 warps; warp g owns query head g in the softmax phase

template <int D, bool LOAD_V>
struct ExactCfg {
  static constexpr int kTileBytes = TILE * D * 2;
  static constexpr int kStageBytes = kTileBytes * (LOAD_V ? 2 : 1);
  // ring depth: two stages of K+V (64 KB), so three CTAs fit on an SM.  This path is bound by its
  // own instruction stream (one warp per scheduler and CTA); more resident CTAs hide more latency
  // than a deeper ring does (measured: 2.3 -> 4.1 TB/s at batch 1 / 64k with 54 splits, 2.9 -> 5.3
  // TB/s at batch 16 / 32k), so the front end sizes the split count for three CTAs per SM.
  static constexpr int kStages = (D == 128) ? (LOAD_V ? 2 : 4) : (LOAD_V ? 4 : 8);
  static constexpr int kAuxFloats = 4 * TILE /*scores*/ + TILE * 4 /*probs*/ + 4 /*alpha*/ + 8 /*m,l*/;
  static constexpr int kSmemBytes = kStages * kStageBytes + kAuxFloats * 4 + kStages * 8 + 128;
};

struct TmaMaps {
  CUtensorMap k;
  CUtensorMap v;
};

template <int D, bool MASKED, bool STATS, bool LOAD_V>
__global__ void __launch_bounds__(EX_THREADS, 3)
decode_exact_kernel(const kvskip_params p, const __grid_constant__ TmaMaps maps) {
  using Cfg = ExactCfg<D, LOAD_V>;
  constexpr int G = 4;
  constexpr int S = Cfg::kStages;
  constexpr int CH = D / 64;    // 16-byte chunks of a key row per lane in the score phase
  constexpr int DPL = D / 32;   // value dims per lane in the PV phase

  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* tiles = smem;
  float* sS = reinterpret_cast<float*>(smem + S * Cfg::kStageBytes);   // [G][TILE] scores, log2 units
  float* sP = sS + G * TILE;                                            // [TILE][G] probabilities
  float* sA = sP + TILE * G;                                            // [G] rescale of this block
  float* sML = sA + G;                                                  // [G][2]
  uint64_t* full = reinterpret_cast<uint64_t*>(sML + 2 * G);           // [S]

  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quad = lane >> 3, j = lane & 7;

  int n_items;
  const int32_t* list = nullptr;
  if constexpr (MASKED) {
    n_items = p.block_cnt[b * p.Hkv + h];
    list = p.block_idx + static_cast<int64_t>(b * p.Hkv + h) * p.max_blocks;
  } else {
    n_items = (p.T + TILE - 1) / TILE;
  }
  const int per = (n_items + p.num_splits - 1) / p.num_splits;
  const int i0 = min(n_items, split * per);
  const int n = min(n_items, i0 + per) - i0;

  if (tid == 0) {
    tma_prefetch_desc(&maps.k);
    if constexpr (LOAD_V) tma_prefetch_desc(&maps.v);
    for (int s = 0; s < S; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  __syncthreads();

  auto block_at = [&](int i) -> int { return MASKED ? list[i0 + i] : i0 + i; };
  auto issue = [&](int i) {   // thread 0 only
    const int s = i % S;
    const int t0 = block_at(i) * TILE;
    unsigned char* dst = tiles + s * Cfg::kStageBytes;
    mbar_expect_tx(&full[s], Cfg::kStageBytes);
    tma_load_4d(dst, &maps.k, &full[s], 0, t0, h, b);
    if constexpr (LOAD_V) tma_load_4d(dst + Cfg::kTileBytes, &maps.v, &full[s], 0, t0, h, b);
  };
  if (tid == 0)
    for (int i = 0; i < S - 1 && i < n; ++i) issue(i);

  // the four queries, scaled to log2 units, in the score-phase lane layout
  float qr[G][CH * 8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const uint16_t* qp = p.q + b * p.q_sb + (h * G + g) * p.q_sh;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const uint4 w = *reinterpret_cast<const uint4*>(qp + c * 64 + 8 * j);
      const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        qr[g][c * 8 + 2 * e] = bf_lo(ww[e]) * p.scale_log2;
        qr[g][c * 8 + 2 * e + 1] = bf_hi(ww[e]) * p.scale_log2;
      }
    }
  }

  float m_run = -INFINITY, l_run = 0.f;   // of query head `warp`
  float acc[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < DPL; ++e) acc[g][e] = 0.f;

  bool alive = true;
  for (int i = 0; i < n; ++i) {
    const int s = i % S;
    if (!mbar_wait(&full[s], (i / S) & 1, 0x100u + s)) { alive = false; break; }
    const int blk = block_at(i);
    const int t0 = blk * TILE;
    const uint16_t* tK = reinterpret_cast<const uint16_t*>(tiles + s * Cfg::kStageBytes);
    if constexpr (MASKED && STATS) {
      // statistics of the blocks the list skips: -inf / 0 between the previous listed block and this
      // one (the last item also covers the tail), so the caller need not pre-fill the arrays
      const int prev = (i0 + i) > 0 ? list[i0 + i - 1] : -1;
      const int next = (i0 + i + 1 == n_items) ? p.nb : blk;
      for (int o = tid; o < (next - prev - 1) * G; o += EX_THREADS) {
        const int gblk = prev + 1 + o / G;
        if (gblk == blk) continue;
        const int64_t at = (static_cast<int64_t>(b) * p.Hq + h * G + o % G) * p.nb + gblk;
        p.blk_max[at] = -INFINITY;
        p.blk_sum[at] = 0.f;
      }
    }

    // ---- scores: warp w covers rows 16w..16w+15, four rows per pass, eight lanes per row
#pragma unroll
    for (int pass = 0; pass < TILE / 16; ++pass) {
      const int r = warp * 16 + pass * 4 + quad;
      float sc[G];
#pragma unroll
      for (int g = 0; g < G; ++g) sc[g] = 0.f;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const uint4 w = *reinterpret_cast<const uint4*>(tK + r * D + c * 64 + 8 * j);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float lo = bf_lo(ww[e]), hi = bf_hi(ww[e]);
#pragma unroll
          for (int g = 0; g < G; ++g) sc[g] = fmaf(qr[g][c * 8 + 2 * e], lo, sc[g]);
#pragma unroll
          for (int g = 0; g < G; ++g) sc[g] = fmaf(qr[g][c * 8 + 2 * e + 1], hi, sc[g]);
        }
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1)
#pragma unroll
        for (int g = 0; g < G; ++g) sc[g] += __shfl_xor_sync(0xffffffffu, sc[g], o);
      if (j < G) {
        const float val = j == 0 ? sc[0] : j == 1 ? sc[1] : j == 2 ? sc[2] : sc[3];
        sS[j * TILE + r] = (t0 + r < p.T) ? val : -INFINITY;
      }
    }
    __syncthreads();   // scores visible; every warp has also finished the PV phase of block i-1
    if (tid == 0 && i + S - 1 < n) issue(i + S - 1);   // refills the stage block i-1 used

    // ---- online softmax of head `warp`; lane holds tokens lane and lane+32
    {
      const int g = warp;
      const float s0 = sS[g * TILE + lane], s1 = sS[g * TILE + lane + 32];
      const float mt = warp_max(fmaxf(s0, s1));
      const float m_new = fmaxf(m_run, mt);
      const float mu = (m_new == -INFINITY) ? 0.f : m_new;
      const float p0 = ex2(s0 - mu), p1 = ex2(s1 - mu);
      const float lt = warp_sum(p0 + p1);
      const float alpha = ex2(m_run - mu);
      l_run = l_run * alpha + lt;
      m_run = m_new;
      sP[lane * G + g] = p0;
      sP[(lane + 32) * G + g] = p1;
      if (lane == 0) sA[g] = alpha;
      if constexpr (STATS) {
        const float mtu = (mt == -INFINITY) ? 0.f : mt;
        const float e0 = ex2(s0 - mtu), e1 = ex2(s1 - mtu);
        const float st = warp_sum(e0 + e1);
        const int64_t hq = static_cast<int64_t>(b) * p.Hq + h * G + g;
        if (lane == 0) {
          p.blk_max[hq * p.nb + blk] = mt * LN2;
          p.blk_sum[hq * p.nb + blk] = st;
        }
        if (p.p_out) {
          __half* po = reinterpret_cast<__half*>(p.p_out) + hq * p.t_pad + t0;
          po[lane] = __float2half_rn(e0);
          po[lane + 32] = __float2half_rn(e1);
        }
      }
    }
    __syncthreads();

    // ---- PV: warp w accumulates rows 16w..16w+15, lane owns dims DPL*lane..
    if constexpr (LOAD_V) {
      const uint16_t* tV = reinterpret_cast<const uint16_t*>(tiles + s * Cfg::kStageBytes + Cfg::kTileBytes);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float a = sA[g];
#pragma unroll
        for (int e = 0; e < DPL; ++e) acc[g][e] *= a;
      }
#pragma unroll
      for (int rr = 0; rr < 16; ++rr) {
        const int r = warp * 16 + rr;
        float vf[DPL];
        if constexpr (DPL == 4) {
          const uint2 w = *reinterpret_cast<const uint2*>(tV + r * D + 4 * lane);
          vf[0] = bf_lo(w.x); vf[1] = bf_hi(w.x); vf[2] = bf_lo(w.y); vf[3] = bf_hi(w.y);
        } else {
          const uint32_t w = *reinterpret_cast<const uint32_t*>(tV + r * D + 2 * lane);
          vf[0] = bf_lo(w); vf[1] = bf_hi(w);
        }
        const float4 pr = *reinterpret_cast<const float4*>(sP + r * G);
        const float pg[4] = {pr.x, pr.y, pr.z, pr.w};
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
          for (int e = 0; e < DPL; ++e) acc[g][e] = fmaf(pg[g], vf[e], acc[g][e]);
      }
    }
  }
  (void)alive;   // after a timed-out wait the partial state is still written; g_status says so
  if constexpr (MASKED && STATS) {
    if (n_items == 0 && split == 0)   // empty list: the first split clears every block of this KV head
      for (int o = tid; o < p.nb * G; o += EX_THREADS) {
        const int64_t at = (static_cast<int64_t>(b) * p.Hq + h * G + o % G) * p.nb + o / G;
        p.blk_max[at] = -INFINITY;
        p.blk_sum[at] = 0.f;
      }
  }

  // ---- epilogue: sum the four warps' accumulators through shared memory (tile ring is idle:
  // every issued load has been waited for)
  if (lane == 0) {
    sML[2 * warp] = m_run;
    sML[2 * warp + 1] = l_run;
  }
  __syncthreads();
  if constexpr (LOAD_V) {
    float* red = reinterpret_cast<float*>(tiles);   // [4 warps][G][D]
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int e = 0; e < DPL; ++e) red[(warp * G + g) * D + DPL * lane + e] = acc[g][e];
    __syncthreads();
    for (int o = tid; o < G * D; o += EX_THREADS) {
      const int g = o / D, d = o % D;
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) sum += red[(w * G + g) * D + d];
      const int64_t hq = static_cast<int64_t>(b) * p.Hq + h * G + g;
      if (p.num_splits == 1) {
        const float l = sML[2 * g + 1];
        const float o32 = l > 0.f ? sum / l : 0.f;
        reinterpret_cast<__nv_bfloat16*>(p.out)[hq * D + d] = __float2bfloat16(o32);
        if (p.out_f32) p.out_f32[hq * D + d] = o32;
      } else {
        p.part_acc[(hq * p.num_splits + split) * D + d] = sum;
      }
    }
  }
  if (tid < G) {
    const int64_t hq = static_cast<int64_t>(b) * p.Hq + h * G + tid;
    const float m = sML[2 * tid], l = sML[2 * tid + 1];
    if (p.num_splits == 1) {
      if (p.lse) p.lse[hq] = l > 0.f ? (m + log2f(l)) * LN2 : -INFINITY;
    } else {
      p.part_ml[(hq * p.num_splits + split) * 2] = m;
      p.part_ml[(hq * p.num_splits + split) * 2 + 1] = l;
    }
  }
}

// Split merge: one CTA per (b, query head), one thread per dim; global max over the splits, then
// l and acc summed over s = 0..S-1 in that order (kernels/kvskip_kernel.cu:294-314).
// Rows are laid out [row][S] in part_ml / part_acc when row_major, else [S][row] (gathered shards).
template <int D>
__global__ void __launch_bounds__(D) merge_kernel(const float* __restrict__ part_acc,
                                                  const float* __restrict__ part_ml, int S, int64_t N,
                                                  bool split_inner, uint16_t* out, float* out_f32,
                                                  float* lse) {
  const int64_t row = blockIdx.x;
  const int d = threadIdx.x;
  auto ml_at = [&](int s, int c) -> float {
    return split_inner ? part_ml[(row * S + s) * 2 + c] : part_ml[(static_cast<int64_t>(s) * N + row) * 2 + c];
  };
  auto acc_at = [&](int s) -> float {
    return split_inner ? part_acc[(row * S + s) * D + d] : part_acc[(static_cast<int64_t>(s) * N + row) * D + d];
  };
  float m = -INFINITY;
  for (int s = 0; s < S; ++s) m = fmaxf(m, ml_at(s, 0));
  const float mu = (m == -INFINITY) ? 0.f : m;
  float l = 0.f, acc = 0.f;
  for (int s = 0; s < S; ++s) {
    const float w = ex2(ml_at(s, 0) - mu);
    l += ml_at(s, 1) * w;
    acc += acc_at(s) * w;
  }
  const float o32 = l > 0.f ? acc / l : 0.f;
  if (out) reinterpret_cast<__nv_bfloat16*>(out)[row * D + d] = __float2bfloat16(o32);
  if (out_f32) out_f32[row * D + d] = o32;
  if (d == 0 && lse) lse[row] = l > 0.f ? (m + log2f(l)) * LN2 : -INFINITY;
}

// Sequence shards: a rank's normalised result as the triple the merge consumes, packed per row as
// [acc(D) | m | l] with acc = out, m = lse / ln 2, l = 1 (l = 0, m = -inf for a rank that read nothing).
template <int D>
__global__ void __launch_bounds__(D) pack_partial_kernel(const float* __restrict__ out_f32,
                                                         const float* __restrict__ lse, float* __restrict__ packed) {
  const int64_t row = blockIdx.x;
  const int d = threadIdx.x;
  pdl_wait_prior();
  packed[row * (D + 2) + d] = out_f32[row * D + d];
  if (d == 0) {
    const float x = lse[row];
    const bool empty = x == -INFINITY;
    packed[row * (D + 2) + D] = empty ? -INFINITY : x * LOG2E;
    packed[row * (D + 2) + D + 1] = empty ? 0.f : 1.f;
  }
}

// merge_kernel for R packed partials [R][N][D+2], ascending r.
template <int D>
__global__ void __launch_bounds__(D) merge_packed_kernel(const float* __restrict__ parts, int R, int64_t N,
                                                         uint16_t* out, float* out_f32, float* lse) {
  const int64_t row = blockIdx.x;
  const int d = threadIdx.x;
  constexpr int W = D + 2;
  float m = -INFINITY;
  for (int r = 0; r < R; ++r) m = fmaxf(m, parts[(static_cast<int64_t>(r) * N + row) * W + D]);
  const float mu = (m == -INFINITY) ? 0.f : m;
  float l = 0.f, acc = 0.f;
  for (int r = 0; r < R; ++r) {
    const float* pr = parts + (static_cast<int64_t>(r) * N + row) * W;
    const float w = ex2(pr[D] - mu);
    l += pr[D + 1] * w;
    acc += pr[d] * w;
  }
  const float o32 = l > 0.f ? acc / l : 0.f;
  if (out) reinterpret_cast<__nv_bfloat16*>(out)[row * D + d] = __float2bfloat16(o32);
  if (out_f32) out_f32[row * D + d] = o32;
  if (d == 0 && lse) lse[row] = l > 0.f ? (m + log2f(l)) * LN2 : -INFINITY;
}

// ---- sequence shards, exchange and merge in one kernel over peer memory ----------------------
// One process per GPU.  Every rank owns a symmetric buffer of 8-byte words [2][R][N][D+2] and
// knows the peers' addresses of theirs.  A word is (value bits, step number): the flag travels with
// the data in one 8-byte store, which arrives whole, so no fence, no separate flag array and no
// second round trip are needed -- a reader polls the word itself until it carries the step number
// it waits for.  Row `row` of this rank's result is packed as [acc(D) | m | l] (acc = out,
// m = lse / ln 2, l = 1) and stored word by word into slot [seq & 1][rank][row] of EVERY rank's
// buffer (plain 8-byte stores, over NVLink for the peers); the same CTA then reads the R triples
// of its row from ITS OWN buffer, waiting for each word, and merges them in ascending rank order
// (the arithmetic of merge_packed_kernel, so the bits equal the all-gather path).  Two buffer sets
// alternate by the parity of seq: a rank can be at most one step ahead of a peer, because
// finishing a step needs the peer's words of that step.  Every wait is bounded (`spin` polls); on
// expiry the status word is set to 0x500 + peer and that peer counts as having read nothing.
constexpr int XCHG_MAX_RANKS = 8;
struct XchgPeers {
  float* buf[XCHG_MAX_RANKS];            // 8-byte words; declared float* for the C ABI's sake
  unsigned int* flags[XCHG_MAX_RANKS];   // unused (kept so that the parameter block keeps its shape)
};

__device__ __forceinline__ void ll_store(float* buf, const int64_t word, const float val, const unsigned int seq) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(reinterpret_cast<uint2*>(buf) + word),
               "r"(__float_as_uint(val)), "r"(seq)
               : "memory");
}
// Waits until the word carries `seq`; false (and val = 0) after `spin` polls.
__device__ __forceinline__ bool ll_load(const float* buf, const int64_t word, const unsigned int seq,
                                        const unsigned int spin, float& val) {
  const uint2* w = reinterpret_cast<const uint2*>(buf) + word;
  for (unsigned int it = 0; it < spin; ++it) {
    unsigned int x, y;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(x), "=r"(y) : "l"(w) : "memory");
    if (y == seq) {
      val = __uint_as_float(x);
      return true;
    }
    if (it > 256) __nanosleep(64);
  }
  val = 0.f;
  return false;
}

template <int D>
__global__ void __launch_bounds__(D) exchange_merge_kernel(const float* __restrict__ out_f32,
                                                           const float* __restrict__ lse, const XchgPeers peers,
                                                           int rank, int R, int64_t N, unsigned int seq,
                                                           unsigned int spin, uint16_t* out, float* res_f32,
                                                           float* res_lse) {
  constexpr int W = D + 2;
  const int64_t row = blockIdx.x;
  const int d = threadIdx.x;
  pdl_wait_prior();
  const int64_t par = static_cast<int64_t>(seq & 1u) * R;
  const int64_t slot = ((par + rank) * N + row) * W;
  const float val = out_f32[row * D + d];
  float mval = 0.f, lval = 0.f;
  if (d == 0) {
    const float x = lse[row];
    mval = x == -INFINITY ? -INFINITY : x * LOG2E;
    lval = x == -INFINITY ? 0.f : 1.f;
  }
  for (int r = 0; r < R; ++r) {
    ll_store(peers.buf[r], slot + d, val, seq);
    if (d == 0) {
      ll_store(peers.buf[r], slot + D, mval, seq);
      ll_store(peers.buf[r], slot + D + 1, lval, seq);
    }
  }
  // the R triples of this row from this rank's own buffer
  const float* mine = peers.buf[rank];
  float mr[XCHG_MAX_RANKS], lr[XCHG_MAX_RANKS], ar[XCHG_MAX_RANKS];
  float m = -INFINITY;
  for (int r = 0; r < R; ++r) {
    const int64_t w0 = ((par + r) * N + row) * W;
    const bool ok = ll_load(mine, w0 + D, seq, spin, mr[r]) & ll_load(mine, w0 + D + 1, seq, spin, lr[r]) &
                    ll_load(mine, w0 + d, seq, spin, ar[r]);
    if (!ok) {
      atomicCAS(&g_status, 0u, 0x500u + r);
      mr[r] = -INFINITY;
      lr[r] = ar[r] = 0.f;
    }
    m = fmaxf(m, mr[r]);
  }
  const float mu = (m == -INFINITY) ? 0.f : m;
  float l = 0.f, acc = 0.f;
  for (int r = 0; r < R; ++r) {
    const float w = ex2(mr[r] - mu);
    l += lr[r] * w;
    acc += ar[r] * w;
  }
  const float o32 = l > 0.f ? acc / l : 0.f;
  if (out) reinterpret_cast<__nv_bfloat16*>(out)[row * D + d] = __float2bfloat16(o32);
  if (res_f32) res_f32[row * D + d] = o32;
  if (d == 0 && res_lse) res_lse[row] = l > 0.f ? (m + log2f(l)) * LN2 : -INFINITY;
}

}  // namespace kvb
