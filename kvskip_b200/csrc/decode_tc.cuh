// Split-K flash-decoding, fast path: warp-specialised, TMA-fed, tensor-core arithmetic.
//
// Why tensor cores on an HBM-bound kernel: the CUDA-core formulation needs ~3850 warp
// instructions per 64-token block (measured with ncu on the exact-order kernel: 30 % issue-slot
// use with one warp per scheduler, DRAM at 34 % of peak), i.e. >= 960 issue cycles per block per
// SM against ~1450 cycles of HBM time per block per SM at full bandwidth -- the grouped q.K and
// P.V products are issue-bound.  With the tokens of a block on the M axis of mma.m16n8k16
// (S^T = K Q^T, O^T = V^T P^T; the 4 query heads padded to N = 8) the same block costs ~400 warp
// instructions, and the kernel goes back to being bound by the loads.
//
// Structure of one CTA (one (split, kv head, batch) triple, all 4 query heads of the KV head):
//   * warp TC_CONSUMERS is the producer: one lane walks the CTA's block range (or its slice of the
//     block list) and issues, per block, four tiled TMA loads (K and V, two 64-dim halves each,
//     128-byte swizzle so ldmatrix is bank-conflict free) into a 6-stage ring (one stage per consumer warp); every stage has a
//     `full` mbarrier completed by the copy engine's byte count and an `empty` mbarrier the
//     consuming warp arrives on.
//   * warps 0..TC_CONSUMERS-1 are consumers.  A consumer owns whole blocks (block i of the range
//     goes to warp i mod TC_CONSUMERS) and keeps its own running max / sum / accumulator for the 4
//     heads, so nothing inside the loop synchronises across warps and block statistics are
//     warp-local.  Per block: 32 ldmatrix + 32 MMA for the scores, online softmax on the
//     accumulator fragments (shuffles only across the 8 lanes that share a head), P split into
//     bf16 high + low parts (fp32-grade weights), movmatrix to turn the score fragment into the B
//     operand, 32 ldmatrix.trans + 64 MMA for the output.
//   * epilogue: the consumers' states are merged through shared memory in warp order, then
//     written as the final output (one split) or as this split's partial (max, sum, acc).
// D = 128 and D = 64 (half-size stages, two per consumer warp), G = 4.  Scores differ from the exact-order path in the last bits (the tensor
// core's accumulation order); outputs and block log-sum-exps stay within the 2e-3 tolerance.
#pragma once
#include "common.cuh"
#include "decode_exact.cuh"

namespace kvb {

// Consumer warps.  The stage count of every configuration is a multiple of this, so all uses of a
// stage are consumed by the same warp: an mbarrier wait names a phase by its parity only, and a
// warp that never saw the previous use of a stage could otherwise pass a wait for the next one.
constexpr int TC_CONSUMERS = 6;
constexpr int TC_THREADS = (TC_CONSUMERS + 1) * 32;
constexpr int TC_HALF_BYTES = TILE * 64 * 2;        // one TMA box: 64 tokens x 64 dims bf16 = 8 KB

// NC consumer warps and NC (K+V) or 2*NC (K only) stages.  NC = 6 fills an SM with one CTA (198 KB):
// used when the grid is a single wave.  NC = 3 is half of that, two CTAs per SM: used when the grid
// has more CTAs than SMs, so that while one CTA of an SM sets up, drains or merges, the other one
// streams -- the fixed cost of a CTA (about 6 us: launch, first TMA round trip, merge, fence and
// counter) is as long as streaming 9 blocks, and block lists of a refresh step are short.
// D = 64 (one 64-dim half per tensor): stages are half as large and twice as many, two per consumer.
template <int NC, bool LOAD_V, int D = 128>
struct TcCfg {
  static_assert(D == 64 || D == 128, "head dims with a tensor-core path");
  static constexpr int kHalves = D / 64;                            // 64-dim TMA boxes per tensor and block
  static constexpr int kThreads = (NC + 1) * 32;
  static constexpr int kStageBytes = TC_HALF_BYTES * kHalves * (LOAD_V ? 2 : 1);
  static constexpr int kStages = (LOAD_V ? NC : 2 * NC) * (2 / kHalves);
  static constexpr int kRedBytes = NC * 4 * D * 4;                  // epilogue staging, aliases the ring
  static constexpr int kAuxBytes = NC * 8 * 4 + 2 * kStages * 8;
  static_assert(kStages % NC == 0, "a stage must always be consumed by the same warp");
  static_assert(kRedBytes <= kStages * kStageBytes, "epilogue staging fits in the ring");
  static constexpr int kSmemBytes = kStages * kStageBytes + kAuxBytes + 1024 /* alignment slack */;
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movm_t(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
// (lo, hi) floats -> packed bf16x2 (lo in the low half), round to nearest even
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// max / sum over the 8 lanes that share lane % 4 (= the same pair of heads)
__device__ __forceinline__ float quadcol_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
}
__device__ __forceinline__ float quadcol_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  return v + __shfl_xor_sync(0xffffffffu, v, 16);
}

// ---- one 64-token block for one consumer warp: scores, online softmax (+ statistics), output.
// kbase: shared-memory address of the stage (K halves, then V halves); state in m_run / l_run / acc.
template <bool STATS, bool LOAD_V, int D = 128>
__device__ __forceinline__ void tc_block(const kvskip_params& p, const uint32_t kbase, const uint32_t (&bq)[D / 16][2],
                                         const int blk, const int64_t hq0, const int lane, const int T,
                                         float (&m_run)[2], float (&l_run)[2], float (&acc)[D / 16][4]) {
  constexpr int KS = D / 16;                   // 16-dim steps of the score product = 16-dim tiles of the output
  const int lrow = lane & 7, lmat = lane >> 3;
  const bool col_ok = (lane & 3) < 2;          // this thread's two columns are real heads
  const int head0 = 2 * (lane & 3);
  const int t0 = blk * TILE;
  // ---- S^T = K Q^T: 4 tiles of 16 tokens x 8 heads
  float sc[4][4];
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int c = 0; c < 4; ++c) sc[mt][c] = 0.f;
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const uint32_t hbase = kbase + (ks >> 2) * TC_HALF_BYTES;
    const int chunk = (ks & 3) * 2 + (lmat >> 1);
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
      const int row = mt * 16 + (lmat & 1) * 8 + lrow;
      uint32_t a[4];
      ldsm_x4(a, hbase + row * 128 + ((chunk ^ lrow) << 4));
      mma_bf16(sc[mt], a, bq[ks][0], bq[ks][1]);
    }
  }
  // scale to log2 units, mask the tokens past T (last block only)
  const bool ragged = t0 + TILE > T;
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float v = sc[mt][c] * p.scale_log2;
      if (ragged && t0 + mt * 16 + (lane >> 2) + (c >> 1) * 8 >= T) v = -INFINITY;
      sc[mt][c] = v;
    }
  // ---- online softmax, two heads per thread
  float mb[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    float v = fmaxf(sc[0][e], sc[0][e + 2]);
#pragma unroll
    for (int mt = 1; mt < 4; ++mt) v = fmaxf(v, fmaxf(sc[mt][e], sc[mt][e + 2]));
    mb[e] = quadcol_max(v);
  }
  float alpha[2], mu[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const float m_new = fmaxf(m_run[e], mb[e]);
    mu[e] = (m_new == -INFINITY) ? 0.f : m_new;
    alpha[e] = ex2(m_run[e] - mu[e]);
    m_run[e] = m_new;
  }
  if constexpr (STATS) {
    float es[2] = {0.f, 0.f};
    const float mtu[2] = {mb[0] == -INFINITY ? 0.f : mb[0], mb[1] == -INFINITY ? 0.f : mb[1]};
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float ev = ex2(sc[mt][c] - mtu[c & 1]);
        es[c & 1] += ev;
        if (p.p_out && col_ok) {
          __half* po = reinterpret_cast<__half*>(p.p_out) + (hq0 + head0 + (c & 1)) * p.t_pad + t0;
          po[mt * 16 + (lane >> 2) + (c >> 1) * 8] = __float2half_rn(ev);
        }
      }
    es[0] = quadcol_sum(es[0]);
    es[1] = quadcol_sum(es[1]);
    if (lane < 2) {   // lanes 0 and 1 hold heads (0,1) and (2,3)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        p.blk_max[(hq0 + head0 + e) * p.nb + blk] = mb[e] * LN2;
        p.blk_sum[(hq0 + head0 + e) * p.nb + blk] = es[e];
      }
    }
  }
  float ls[2] = {0.f, 0.f};
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float pv = ex2(sc[mt][c] - mu[c & 1]);
      sc[mt][c] = pv;
      ls[c & 1] += pv;
    }
  l_run[0] = l_run[0] * alpha[0] + ls[0];
  l_run[1] = l_run[1] * alpha[1] + ls[1];

  if constexpr (LOAD_V) {
    // ---- O^T = alpha * O^T + V^T P^T
    if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
      for (int mt = 0; mt < KS; ++mt) {
        acc[mt][0] *= alpha[0]; acc[mt][1] *= alpha[1];
        acc[mt][2] *= alpha[0]; acc[mt][3] *= alpha[1];
      }
    }
    const uint32_t vbase = kbase + (D / 64) * TC_HALF_BYTES;
#pragma unroll
    for (int kt = 0; kt < 4; ++kt) {
      // P of tokens kt*16..+15 as high + low bf16 parts, transposed into the B layout
      const uint32_t h0 = pack_bf16(sc[kt][0], sc[kt][1]);
      const uint32_t h1 = pack_bf16(sc[kt][2], sc[kt][3]);
      const uint32_t l0 = pack_bf16(sc[kt][0] - bf_lo(h0), sc[kt][1] - bf_hi(h0));
      const uint32_t l1 = pack_bf16(sc[kt][2] - bf_lo(h1), sc[kt][3] - bf_hi(h1));
      const uint32_t bh0 = movm_t(h0), bh1 = movm_t(h1), bl0 = movm_t(l0), bl1 = movm_t(l1);
      const int tok = kt * 16 + (lmat >> 1) * 8 + lrow;
#pragma unroll
      for (int mt = 0; mt < KS; ++mt) {
        const int dchunk = mt * 2 + (lmat & 1);
        uint32_t a[4];
        ldsm_x4_t(a, vbase + (dchunk >> 3) * TC_HALF_BYTES + tok * 128 + (((dchunk & 7) ^ lrow) << 4));
        mma_bf16(acc[mt], a, bh0, bh1);
        mma_bf16(acc[mt], a, bl0, bl1);
      }
    }
  }
}

// Q^T as the B operand of the score MMA: column n = lane/4 is a head (4..7 are zero padding),
// rows k = 2*(lane%4)+{0,1} (+8) of each 16-dim step
template <int KS>
__device__ __forceinline__ void tc_load_q(const kvskip_params& p, const int b, const int h, const int lane,
                                          uint32_t (&bq)[KS][2]) {
  const int head = lane >> 2;
  const uint16_t* qp = p.q + b * p.q_sb + (h * 4 + (head & 3)) * p.q_sh + 2 * (lane & 3);
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    bq[ks][0] = head < 4 ? *reinterpret_cast<const uint32_t*>(qp + ks * 16) : 0u;
    bq[ks][1] = head < 4 ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8) : 0u;
  }
}

// Statistics of the blocks a list skips: -inf / 0 between the previous listed block and this one
// (the last item also covers the tail), so the caller need not pre-fill the arrays.
__device__ __forceinline__ void tc_fill_gap(const kvskip_params& p, const int32_t* list, const int pos,
                                            const int n_items, const int blk, const int64_t hq0, const int lane) {
  const int prev = pos > 0 ? list[pos - 1] : -1;
  const int next = (pos + 1 == n_items) ? p.nb : blk;
  for (int gblk = prev + 1 + lane; gblk < next; gblk += 32) {
    if (gblk == blk) continue;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      p.blk_max[(hq0 + g) * p.nb + gblk] = -INFINITY;
      p.blk_sum[(hq0 + g) * p.nb + gblk] = 0.f;
    }
  }
}

// Sequence shards: the cross-GPU exchange inside the attention kernel.  With R > 0 the CTA that
// merges the splits of a (batch, kv head) does not write the result but stores it, as the packed
// triple (acc = out, m = lse / ln 2, l = 1) of exchange_merge_kernel, into every rank's buffer
// over NVLink (plain peer stores of (value, step number) words), then reads the R triples of its
// rows from its own rank's buffer, waiting -- bounded -- for each word, and merges them in
// ascending rank order.  Same buffers, slots and arithmetic as exchange_merge_kernel, so the two
// give the same bits.
struct XchgArgs {
  XchgPeers peers;
  int rank;
  int R;                 // 0: no exchange
  long long N;           // rows of the exchange (B * Hq)
  unsigned int seq;
  unsigned int spin;     // polls of a peer's flag before the wait gives up (status word 0x510 + peer)
};

// Look-ahead of a producer thread over the blocks of its piece.  The number of block i comes from
// the list (a load) and, with a paged cache, its page from the table (a second load that depends on
// the first); asked for when the block is due, each costs the producer a memory round trip per
// block between a stage becoming free and its refill.  Here the list is read eight blocks ahead and
// the table four, so that in steady state both values are in registers when the stage is free.
template <bool MASKED>
struct BlockAhead {
  static constexpr int LA = 4;
  int blk[2 * LA];
  int pg[LA];
  const int32_t* list;   // entries of this piece (MASKED), first at list[0]
  const int32_t* table;  // page table row of the sequence, or null
  int first, n, seq;

  __device__ __forceinline__ int entry(const int j) const {
    if (j >= n) return 0;
    return MASKED ? list[j] : first + j;
  }
  __device__ __forceinline__ int page(const int b) const { return table ? table[b] : seq; }
  // first: number of the piece's first block when there is no list; seq: what `page` is without a table
  __device__ __forceinline__ void init(const int32_t* list_, const int32_t* table_, const int first_, const int n_,
                                       const int seq_) {
    list = list_, table = table_, first = first_, n = n_, seq = seq_;
#pragma unroll
    for (int j = 0; j < 2 * LA; ++j) blk[j] = entry(j);
#pragma unroll
    for (int j = 0; j < LA; ++j) pg[j] = page(blk[j]);
  }
  // block i (calls in order i = 0, 1, ...): its number and page; requests those of later blocks
  __device__ __forceinline__ void next(const int i, int& b_out, int& pg_out) {
    b_out = blk[0];
    pg_out = pg[0];
#pragma unroll
    for (int j = 0; j + 1 < 2 * LA; ++j) blk[j] = blk[j + 1];
    blk[2 * LA - 1] = entry(i + 2 * LA);
#pragma unroll
    for (int j = 0; j + 1 < LA; ++j) pg[j] = pg[j + 1];
    pg[LA - 1] = page(blk[LA - 1]);
  }
};

// Merge of the S pieces of one (query head, output element) on the tensor-core path: global max,
// then the rescaled sums in FOUR interleaved chains (pieces s = k mod 4 in ascending order, combined
// as (c0 + c1) + (c2 + c3)): four independent chains of loads and additions instead of one, which
// matters when the CTA that merges is the tail of the launch (a head cut into 43 pieces).  Every
// in-kernel merge of this path and tc_merge_kernel use this order, so they give the same bits.
// ml: (m, l) pairs of the pieces; acc: this element of piece 0, pieces `stride` floats apart.
__device__ __forceinline__ void tc_merge_pieces(const float* ml, const float* acc, const int stride, const int S,
                                                float& m_out, float& l_out, float& a_out) {
  float m = -INFINITY;
  for (int s = 0; s < S; ++s) m = fmaxf(m, __ldcg(ml + 2 * s));
  const float mu = (m == -INFINITY) ? 0.f : m;
  float l[4] = {0.f, 0.f, 0.f, 0.f}, a[4] = {0.f, 0.f, 0.f, 0.f};
  int s = 0;
  for (; s + 4 <= S; s += 4) {
    float w[4], pl[4], x[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      w[u] = __ldcg(ml + 2 * (s + u));
      pl[u] = __ldcg(ml + 2 * (s + u) + 1);
      x[u] = __ldcg(acc + static_cast<int64_t>(s + u) * stride);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float ww = ex2(w[u] - mu);
      l[u] += pl[u] * ww;
      a[u] += x[u] * ww;
    }
  }
  for (int u = 0; s < S; ++s, ++u) {
    const float ww = ex2(__ldcg(ml + 2 * s) - mu);
    l[u] += __ldcg(ml + 2 * s + 1) * ww;
    a[u] += __ldcg(acc + static_cast<int64_t>(s) * stride) * ww;
  }
  m_out = m;
  l_out = (l[0] + l[1]) + (l[2] + l[3]);
  a_out = (a[0] + a[1]) + (a[2] + a[3]);
}

// tc_merge_pieces for E (query head, output element) pairs at once, with the loads of eight pieces
// of all E pairs requested before the first is used: the CTA that merges a head is the tail of its
// launch, and a merge that asks for four values at a time spends a memory round trip on every four
// pieces of every element.  Every chain sees the same operands in the same order as in
// tc_merge_pieces, so the bits are the same.
template <int E>
__device__ __forceinline__ void tc_merge_pieces_n(const float* const (&ml)[E], const float* const (&acc)[E],
                                                  const int stride, const int S, float (&m_out)[E], float (&l_out)[E],
                                                  float (&a_out)[E]) {
  constexpr int MB = 16, PB = 8;
  float m[E], mu[E];
#pragma unroll
  for (int e = 0; e < E; ++e) m[e] = -INFINITY;
  for (int s0 = 0; s0 < S; s0 += MB) {
    float v[E][MB];
#pragma unroll
    for (int e = 0; e < E; ++e)
#pragma unroll
      for (int u = 0; u < MB; ++u) v[e][u] = s0 + u < S ? __ldcg(ml[e] + 2 * (s0 + u)) : -INFINITY;
#pragma unroll
    for (int e = 0; e < E; ++e)
#pragma unroll
      for (int u = 0; u < MB; ++u) m[e] = fmaxf(m[e], v[e][u]);
  }
  float l[E][4], a[E][4];
#pragma unroll
  for (int e = 0; e < E; ++e) {
    mu[e] = (m[e] == -INFINITY) ? 0.f : m[e];
#pragma unroll
    for (int u = 0; u < 4; ++u) l[e][u] = a[e][u] = 0.f;
  }
  int s = 0;
  for (; s + PB <= S; s += PB) {
    float w[E][PB], pl[E][PB], x[E][PB];
#pragma unroll
    for (int e = 0; e < E; ++e)
#pragma unroll
      for (int u = 0; u < PB; ++u) {
        w[e][u] = __ldcg(ml[e] + 2 * (s + u));
        pl[e][u] = __ldcg(ml[e] + 2 * (s + u) + 1);
        x[e][u] = __ldcg(acc[e] + static_cast<int64_t>(s + u) * stride);
      }
#pragma unroll
    for (int e = 0; e < E; ++e)
#pragma unroll
      for (int u = 0; u < PB; ++u) {
        const float ww = ex2(w[e][u] - mu[e]);
        l[e][u & 3] += pl[e][u] * ww;
        a[e][u & 3] += x[e][u] * ww;
      }
  }
  {   // the last 0..7 pieces: chains 0, 1, 2, 3, 0, ... as above
    float w[E][PB], pl[E][PB], x[E][PB];
#pragma unroll
    for (int e = 0; e < E; ++e)
#pragma unroll
      for (int u = 0; u < PB; ++u) {
        const int su = min(s + u, S - 1);
        w[e][u] = __ldcg(ml[e] + 2 * su);
        pl[e][u] = __ldcg(ml[e] + 2 * su + 1);
        x[e][u] = __ldcg(acc[e] + static_cast<int64_t>(su) * stride);
      }
#pragma unroll
    for (int e = 0; e < E; ++e)
#pragma unroll
      for (int u = 0; u < PB; ++u)
        if (s + u < S) {
          const float ww = ex2(w[e][u] - mu[e]);
          l[e][u & 3] += pl[e][u] * ww;
          a[e][u & 3] += x[e][u] * ww;
        }
  }
#pragma unroll
  for (int e = 0; e < E; ++e) {
    m_out[e] = m[e];
    l_out[e] = (l[e][0] + l[e][1]) + (l[e][2] + l[e][3]);
    a_out[e] = (a[e][0] + a[e][1]) + (a[e][2] + a[e][3]);
  }
}

// The same merge as a kernel of its own (the fallback when a launch cannot use the device counters):
// one CTA per (b, query head), one thread per dim; part_acc [rows][S][D], part_ml [rows][S][2].
template <int D>
__global__ void __launch_bounds__(D) tc_merge_kernel(const float* __restrict__ part_acc,
                                                     const float* __restrict__ part_ml, int S, uint16_t* out,
                                                     float* out_f32, float* lse) {
  const int64_t row = blockIdx.x;
  const int d = threadIdx.x;
  float m, l, a;
  tc_merge_pieces(part_ml + row * S * 2, part_acc + row * S * D + d, D, S, m, l, a);
  const float o32 = l > 0.f ? a / l : 0.f;
  if (out) reinterpret_cast<__nv_bfloat16*>(out)[row * D + d] = __float2bfloat16(o32);
  if (out_f32) out_f32[row * D + d] = o32;
  if (d == 0 && lse) lse[row] = l > 0.f ? (m + log2f(l)) * LN2 : -INFINITY;
}

// One element of this rank's packed row (acc = out, then m = lse / ln 2 and l = 1) into every
// rank's buffer as (value, step number) words: plain 8-byte stores, to peer memory over NVLink for
// r != rank.
__device__ __forceinline__ void xchg_store(const XchgArgs& xa, const int64_t hq, const int d, const float o32,
                                           const float lse_nat) {
  constexpr int D = 128, XW = D + 2;
  const int64_t slot = ((static_cast<int64_t>(xa.seq & 1u) * xa.R + xa.rank) * xa.N + hq) * XW;
  for (int r = 0; r < xa.R; ++r) {
    ll_store(xa.peers.buf[r], slot + d, o32, xa.seq);
    if (d == 0) {
      ll_store(xa.peers.buf[r], slot + D, lse_nat == -INFINITY ? -INFINITY : lse_nat * LOG2E, xa.seq);
      ll_store(xa.peers.buf[r], slot + D + 1, lse_nat == -INFINITY ? 0.f : 1.f, xa.seq);
    }
  }
}

// After the four rows of (batch b, kv head h) were stored with xchg_store by this CTA: read the R
// triples of those rows from this rank's own buffer, waiting -- bounded -- for every word to carry
// this step's number, and merge them in ascending rank order (the arithmetic of
// merge_packed_kernel).  No fence and no flag: the step number travels inside every word.
// Called by every thread of the CTA.
template <int THREADS>
__device__ __forceinline__ void xchg_finish(const kvskip_params& p, const XchgArgs& xa, const int b, const int h,
                                            const int tid) {
  constexpr int G = 4, D = 128, XW = D + 2;
  const int64_t hq0x = static_cast<int64_t>(b) * p.Hq + h * G;
  const float* mine = xa.peers.buf[xa.rank];
  const int64_t par = static_cast<int64_t>(xa.seq & 1u) * xa.R;
  for (int o = tid; o < G * D; o += THREADS) {
    const int g = o / D, d = o % D;
    const int64_t row = hq0x + g;
    float mr[XCHG_MAX_RANKS], lr[XCHG_MAX_RANKS], ar[XCHG_MAX_RANKS];
    float m = -INFINITY;
    for (int r = 0; r < xa.R; ++r) {
      const int64_t w0 = ((par + r) * xa.N + row) * XW;
      const bool ok = ll_load(mine, w0 + D, xa.seq, xa.spin, mr[r]) & ll_load(mine, w0 + D + 1, xa.seq, xa.spin, lr[r]) &
                      ll_load(mine, w0 + d, xa.seq, xa.spin, ar[r]);
      if (!ok) {
        atomicCAS(&g_status, 0u, 0x510u + r);
        mr[r] = -INFINITY;
        lr[r] = ar[r] = 0.f;
      }
      m = fmaxf(m, mr[r]);
    }
    const float mu = (m == -INFINITY) ? 0.f : m;
    float l = 0.f, acc2 = 0.f;
    for (int r = 0; r < xa.R; ++r) {
      const float w = ex2(mr[r] - mu);
      l += lr[r] * w;
      acc2 += ar[r] * w;
    }
    const float o32 = l > 0.f ? acc2 / l : 0.f;
    reinterpret_cast<__nv_bfloat16*>(p.out)[row * D + d] = __float2bfloat16(o32);
    if (p.out_f32) p.out_f32[row * D + d] = o32;
    if (d == 0 && p.lse) p.lse[row] = l > 0.f ? (m + log2f(l)) * LN2 : -INFINITY;
  }
}

template <int NC, bool MASKED, bool STATS, bool LOAD_V, int D = 128>
__global__ void __launch_bounds__((NC + 1) * 32, NC <= 3 ? 2 : 1)
decode_tc_kernel(const kvskip_params p, const __grid_constant__ TmaMaps maps, int* __restrict__ split_done,
                 const int min_blocks, const int* __restrict__ t_dev, const int32_t* __restrict__ pages,
                 const int max_pages, const XchgArgs xa) {
  using Cfg = TcCfg<NC, LOAD_V, D>;
  constexpr int G = 4, KS = D / 16, HV = D / 64;   // HV: 64-dim halves per tensor and block
  constexpr int S = Cfg::kStages;
  constexpr int TC_THREADS = Cfg::kThreads;   // shadows the 6-consumer constant inside this kernel

  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* ring = smem;                                              // [S] stages, 1024-byte aligned
  float* sM = reinterpret_cast<float*>(smem + S * Cfg::kStageBytes);       // [NC][4]
  float* sL = sM + NC * 4;                                                 // [NC][4]
  uint64_t* full = reinterpret_cast<uint64_t*>(sL + NC * 4);               // [S]
  uint64_t* empty = full + S;                                              // [S]

  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    tma_prefetch_desc(&maps.k);
    if constexpr (LOAD_V) tma_prefetch_desc(&maps.v);
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  // Launched with programmatic stream serialisation: everything above overlaps the tail of the
  // previous kernel on the stream; nothing that kernel may have written is read before this wait.
  pdl_wait_prior();
  pdl_launch_dependents();

  // Length of the sequences: p.T, or, with a device-resident length, the value at t_dev (p.T is
  // then the bound the grid, the tensor maps and the statistics stride p.nb were sized for).
  const int T = t_dev ? max(1, min(*t_dev, p.T)) : p.T;
  int n_items;
  const int32_t* list = nullptr;
  if constexpr (MASKED) {
    n_items = p.block_cnt[b * p.Hkv + h];
    list = p.block_idx + static_cast<int64_t>(b * p.Hkv + h) * p.max_blocks;
  } else {
    n_items = (T + TILE - 1) / TILE;
  }
  // Splits actually used for this (batch, kv head).  A block list can be much shorter than the
  // length the grid was sized for (a head that does not refresh reads a tenth of the blocks a
  // refreshing one reads): with the merge inside the kernel the list is cut into at most
  // ceil(n_items / min_blocks) pieces and the surplus CTAs leave at once, instead of every CTA
  // paying its fixed cost for a handful of blocks.
  int S_use = p.num_splits;
  if (MASKED && LOAD_V && split_done != nullptr && min_blocks > 1)
    S_use = max(1, min(p.num_splits, (n_items + min_blocks - 1) / min_blocks));
  if (split >= S_use) return;
  const int per = (n_items + S_use - 1) / S_use;
  const int i0 = min(n_items, split * per);
  const int n = min(n_items, i0 + per) - i0;


  // per-thread state of a consumer: two heads (columns 2*(lane&3), +1 of the 8-wide N axis)
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};            // thread-partial sums, reduced across lanes in the epilogue
  float acc[KS][4];                       // O^T fragments: D/16 tiles of 16 dims x 8 heads
#pragma unroll
  for (int mt = 0; mt < KS; ++mt)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[mt][c] = 0.f;

  if (warp == NC) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      BlockAhead<MASKED> ahead;
      ahead.init(MASKED ? list + i0 : nullptr, pages ? pages + static_cast<int64_t>(b) * max_pages : nullptr, i0, n, b);
      for (int i = 0; i < n; ++i) {
        const int s = i % S;
        if (i >= S && !mbar_wait(&empty[s], ((i / S) - 1) & 1, 0x200u + s)) break;
        // contiguous cache: rows blk*64.. of sequence b; paged cache: the whole page the table
        // names for block blk (the maps then run over pages instead of sequences; an entry
        // outside the pool is out of bounds for the map and reads as zeros)
        int blk, bp;
        ahead.next(i, blk, bp);
        const int t0 = pages ? 0 : blk * TILE;
        unsigned char* dst = ring + s * Cfg::kStageBytes;
        mbar_expect_tx(&full[s], Cfg::kStageBytes);
#pragma unroll
        for (int hv = 0; hv < HV; ++hv) tma_load_4d(dst + hv * TC_HALF_BYTES, &maps.k, &full[s], 64 * hv, t0, h, bp);
        if constexpr (LOAD_V) {
#pragma unroll
          for (int hv = 0; hv < HV; ++hv)
            tma_load_4d(dst + (HV + hv) * TC_HALF_BYTES, &maps.v, &full[s], 64 * hv, t0, h, bp);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    uint32_t bq[KS][2];
    tc_load_q<KS>(p, b, h, lane, bq);
    const int64_t hq0 = static_cast<int64_t>(b) * p.Hq + h * G;
    const int head0 = 2 * (lane & 3);

    for (int i = warp; i < n; i += NC) {
      const int s = i % S;
      const int blk = MASKED ? list[i0 + i] : i0 + i;
      if constexpr (MASKED && STATS) tc_fill_gap(p, list, i0 + i, n_items, blk, hq0, lane);
      if (!mbar_wait(&full[s], (i / S) & 1, 0x210u + s)) break;
      const uint32_t kbase = smem_u32(ring + s * Cfg::kStageBytes);
      if constexpr (LOAD_V) {
        // Device-resident length or paged cache: the tensor map reaches past T, so the rows of the
        // last block beyond T hold whatever the cache holds there.  Their weights are zero, but
        // 0 x NaN is not: clear those V rows (whole 128-byte rows of both halves, so the swizzle
        // is moot).
        if ((t_dev != nullptr || pages != nullptr) && blk * TILE + TILE > T) {
          const int r0 = T - blk * TILE;
          unsigned char* vst = ring + s * Cfg::kStageBytes + HV * TC_HALF_BYTES;
          for (int o = r0 * 128 + lane * 16; o < TILE * 128; o += 32 * 16) {
#pragma unroll
            for (int hv = 0; hv < HV; ++hv) *reinterpret_cast<uint4*>(vst + hv * TC_HALF_BYTES + o) = make_uint4(0u, 0u, 0u, 0u);
          }
          fence_proxy_async_smem();   // ordered before the next bulk load into this stage
          __syncwarp();
        }
      }

      tc_block<STATS, LOAD_V, D>(p, kbase, bq, blk, hq0, lane, T, m_run, l_run, acc);
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
    if constexpr (MASKED && STATS) {
      // an empty list: the first split clears every block of this KV head
      if (n_items == 0 && split == 0 && warp == 0)
        for (int gblk = lane; gblk < p.nb; gblk += 32)
#pragma unroll
          for (int g = 0; g < G; ++g) {
            p.blk_max[(hq0 + g) * p.nb + gblk] = -INFINITY;
            p.blk_sum[(hq0 + g) * p.nb + gblk] = 0.f;
          }
    }
    if constexpr (!MASKED && STATS) {
      // device-resident length: blocks between the current and the provisioned length are unread
      if (t_dev != nullptr && split == 0 && warp == 0)
        for (int gblk = n_items + lane; gblk < p.nb; gblk += 32)
#pragma unroll
          for (int g = 0; g < G; ++g) {
            p.blk_max[(hq0 + g) * p.nb + gblk] = -INFINITY;
            p.blk_sum[(hq0 + g) * p.nb + gblk] = 0.f;
          }
    }
    l_run[0] = quadcol_sum(l_run[0]);
    l_run[1] = quadcol_sum(l_run[1]);
    if (lane < 2) {
      sM[warp * 4 + head0] = m_run[0];
      sM[warp * 4 + head0 + 1] = m_run[1];
      sL[warp * 4 + head0] = l_run[0];
      sL[warp * 4 + head0 + 1] = l_run[1];
    }
  }
  __syncthreads();   // every block has been consumed: the ring is free for the merge of the warps

  const bool xchg = LOAD_V && D == 128 && xa.R > 0;   // the cross-GPU exchange exists for D = 128
  if constexpr (LOAD_V) {
    float* red = reinterpret_cast<float*>(ring);   // [NC][G][D]
    if (warp < NC && (lane & 3) < 2) {
      const int head0 = 2 * (lane & 3);
#pragma unroll
      for (int mt = 0; mt < KS; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c)
          red[(warp * G + head0 + (c & 1)) * D + mt * 16 + (lane >> 2) + (c >> 1) * 8] = acc[mt][c];
    }
    __syncthreads();
    for (int o = tid; o < G * D; o += TC_THREADS) {
      const int g = o / D, d = o % D;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < NC; ++w) M = fmaxf(M, sM[w * 4 + g]);
      const float mu = (M == -INFINITY) ? 0.f : M;
      float sum = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < NC; ++w) {
        const float f = ex2(sM[w * 4 + g] - mu);
        sum += red[(w * G + g) * D + d] * f;
        l += sL[w * 4 + g] * f;
      }
      const int64_t hq = static_cast<int64_t>(b) * p.Hq + h * G + g;
      if (S_use == 1) {
        const float o32 = l > 0.f ? sum / l : 0.f;
        if (!xchg) {
          reinterpret_cast<__nv_bfloat16*>(p.out)[hq * D + d] = __float2bfloat16(o32);
          if (p.out_f32) p.out_f32[hq * D + d] = o32;
        } else if constexpr (D == 128) {   // a head this rank reads in one piece (a short or empty list): its row goes to the peers from here
          xchg_store(xa, hq, d, o32, l > 0.f ? (M + log2f(l)) * LN2 : -INFINITY);
        }
      } else {
        p.part_acc[(hq * p.num_splits + split) * D + d] = sum;
      }
    }
  }
  if (tid < G) {
    float M = -INFINITY;
    for (int w = 0; w < NC; ++w) M = fmaxf(M, sM[w * 4 + tid]);
    const float mu = (M == -INFINITY) ? 0.f : M;
    float l = 0.f;
    for (int w = 0; w < NC; ++w) l += sL[w * 4 + tid] * ex2(sM[w * 4 + tid] - mu);
    const int64_t hq = static_cast<int64_t>(b) * p.Hq + h * G + tid;
    if (S_use == 1) {
      if (p.lse && !xchg) p.lse[hq] = l > 0.f ? (M + log2f(l)) * LN2 : -INFINITY;
    } else {
      p.part_ml[(hq * p.num_splits + split) * 2] = M;
      p.part_ml[(hq * p.num_splits + split) * 2 + 1] = l;
    }
  }

  // ---- split merge by the last CTA of this (batch, kv head) to finish: same arithmetic and the
  // same ascending-split order as merge_kernel, without a second launch.  split_done[] counts the
  // finished splits and is put back to zero by the CTA that merges.
  if constexpr (LOAD_V) {
    if (S_use == 1) {
      if constexpr (D == 128)
        if (xchg) xchg_finish<TC_THREADS>(p, xa, b, h, tid);
    } else if (split_done != nullptr) {
      __shared__ int s_last;
      __threadfence();            // this CTA's partials are visible device-wide before it is counted
      __syncthreads();
      if (tid == 0) s_last = atomicAdd(&split_done[b * p.Hkv + h], 1) == S_use - 1;
      __syncthreads();
      if (s_last) {
        __threadfence();
        const int S2 = S_use;             // partials used; their stride stays p.num_splits
        constexpr int E = (G * D + TC_THREADS - 1) / TC_THREADS;   // elements of the head per thread, merged together
        const float* ml[E];
        const float* pa[E];
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const int o = min(tid + e * TC_THREADS, G * D - 1);
          const int64_t hq = static_cast<int64_t>(b) * p.Hq + h * G + o / D;
          ml[e] = p.part_ml + hq * p.num_splits * 2;
          pa[e] = p.part_acc + hq * p.num_splits * D + o % D;
        }
        float mm[E], ll[E], aa[E];
        tc_merge_pieces_n<E>(ml, pa, D, S2, mm, ll, aa);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const int o = tid + e * TC_THREADS;
          if (o >= G * D) continue;
          const int g = o / D, d = o % D;
          const int64_t hq = static_cast<int64_t>(b) * p.Hq + h * G + g;
          const float m = mm[e], l = ll[e], a = aa[e];
          const float o32 = l > 0.f ? a / l : 0.f;
          const float lse_nat = l > 0.f ? (m + log2f(l)) * LN2 : -INFINITY;
          if (!xchg) {
            reinterpret_cast<__nv_bfloat16*>(p.out)[hq * D + d] = __float2bfloat16(o32);
            if (p.out_f32) p.out_f32[hq * D + d] = o32;
            if (d == 0 && p.lse) p.lse[hq] = lse_nat;
          } else if constexpr (D == 128) {
            xchg_store(xa, hq, d, o32, lse_nat);
          }
        }
        if constexpr (D == 128)
          if (xchg) xchg_finish<TC_THREADS>(p, xa, b, h, tid);
        if (tid == 0) split_done[b * p.Hkv + h] = 0;
      }
    }
  }
}

}  // namespace kvb
