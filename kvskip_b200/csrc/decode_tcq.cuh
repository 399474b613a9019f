// Masked split-K decode as ONE persistent CTA per SM that pulls (kv head, piece) items from a
// device-side queue and never lets its shared-memory ring run dry between items.
//
// Why: with block lists the work per (batch, kv head) differs by an order of magnitude (a head
// that refreshes reads every block, the others a tenth) and the one-piece-per-CTA kernel
// (decode_tc.cuh) pays its fixed part -- CTA launch, barrier set-up, first DRAM round trip, merge
// of the consumer warps, fence and counter: about 6 us -- once per piece of 24 blocks (16 us of
// streaming), plus the rounding of the piece count to waves of CTAs.  Here the producer lane
// fetches the next item while the loads of the current one are still being issued, the ring of
// six 32 KB stages carries blocks of consecutive items back to back, the consumer warps hand
// their per-piece state to a seventh "merger" warp through a double-buffered staging area and go
// straight on to the next item, and the merger warp does everything that has a global-memory round
// trip in it (partial store, fence, counter, merge of a head's pieces) off the consumers' path.
//
// Results are bit-identical to decode_tc_kernel<6, MASKED, STATS, true> for the same num_splits
// and min_blocks: a list is cut into the same pieces, block i of a piece is folded by "virtual
// warp" i mod 6 in the same order (the physical warp is rotated so that ring stage s is always
// consumed by warp s: an mbarrier wait names a phase by parity only), the six states merge in
// virtual-warp order, a head's pieces merge in the same order (tc_merge_pieces).  Which SM processes which piece
// depends on timing; what is computed does not.
//
// Warps: 0..5 consumers, 6 producer (one lane), 7 merger.  D = 128, G = 4, V always loaded.
#pragma once
#include "decode_tc.cuh"

namespace kvb {

// Development aid, compiled out by default: with -DKVB_TIMELINE every CTA records %globaltimer stamps
// and counts (entry, first item, first data, last block consumed, exit; items, blocks, skipped ids)
// into g_timeline, which kvskip_debug_timeline() copies out.
#ifdef KVB_TIMELINE
__device__ unsigned long long g_timeline[256 * 16];
__device__ __forceinline__ unsigned long long tl_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define KVB_TL(slot, value) g_timeline[blockIdx.x * 16 + (slot)] = (value)
#else
#define KVB_TL(slot, value) ((void)0)
#endif

struct TcqItem {
  int b, h;
  int i0, n;          // list positions [i0, i0 + n) (dense: blocks)
  int n_items;        // length of the head's list
  int S_use, piece;   // pieces of this head, index of this one
  int stop;           // 1: no more items
};

struct TcqCfg {
  static constexpr int kConsumers = 6;
  static constexpr int kThreads = 8 * 32;
  static constexpr int kStages = 6;
  static constexpr int kStageBytes = 4 * TC_HALF_BYTES;                       // K + V of one block: 32 KB
  static constexpr int kQueueDepth = 4;                                        // item descriptors in flight
  static constexpr int kStageAcc = 2 * kConsumers * 4 * 128 * 4;               // [2][6][4][128] floats
  static constexpr int kStageMl = 2 * 2 * kConsumers * 4 * 4;                  // sM, sL: [2][6][4] floats each
  static constexpr int kBars = (2 * kStages + 2 * kQueueDepth + 4) * 8;
  static constexpr int kMaxHeads = 1024;                                       // (batch, kv head) pairs of a launch
  static constexpr int kTable = (2 * kMaxHeads + 16) * 4;                      // item prefix sums + scan scratch
  static constexpr int kSmemBytes = kStages * kStageBytes + kStageAcc + kStageMl +
                                    kQueueDepth * static_cast<int>(sizeof(TcqItem)) + kBars + kTable + 1024;
  static_assert(kMaxHeads % kThreads == 0, "heads are dealt to threads in equal runs");
  static_assert(kSmemBytes <= 232448, "one CTA per SM: at most 227 KB of shared memory");
};

template <bool MASKED, bool STATS>
__global__ void __launch_bounds__(TcqCfg::kThreads, 1)
decode_tcq_kernel(const kvskip_params p, const __grid_constant__ TmaMaps maps, int* __restrict__ split_done,
                  int* __restrict__ queue, const int min_blocks, const int* __restrict__ t_dev,
                  const int32_t* __restrict__ pages, const int max_pages) {
  constexpr int G = 4, D = 128, NC = TcqCfg::kConsumers, S = TcqCfg::kStages, QD = TcqCfg::kQueueDepth;

  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* ring = smem;
  float* stg = reinterpret_cast<float*>(smem + S * TcqCfg::kStageBytes);        // [2][NC][G][D]
  float* sM = stg + 2 * NC * G * D;                                              // [2][NC][G]
  float* sL = sM + 2 * NC * G;                                                   // [2][NC][G]
  TcqItem* items = reinterpret_cast<TcqItem*>(sL + 2 * NC * G);                  // [QD]
  uint64_t* full = reinterpret_cast<uint64_t*>(items + QD);                      // [S]
  uint64_t* empty = full + S;                                                    // [S]
  uint64_t* ifull = empty + S;                                                   // [QD]
  uint64_t* iempty = ifull + QD;                                                 // [QD]
  uint64_t* done = iempty + QD;                                                  // [2] staging written by the consumers
  uint64_t* freeb = done + 2;                                                    // [2] staging read by the merger
  int* pfx = reinterpret_cast<int*>(freeb + 2);                                  // [2][kMaxHeads] item prefix sums
  int* wsum = pfx + 2 * TcqCfg::kMaxHeads;                                       // [16] scan scratch

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
#ifdef KVB_TIMELINE
    KVB_TL(0, tl_now());
    unsigned int smid;
    asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
    KVB_TL(9, smid);
#endif
    tma_prefetch_desc(&maps.k);
    tma_prefetch_desc(&maps.v);
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < QD; ++s) {
      mbar_init(&ifull[s], 1);
      mbar_init(&iempty[s], NC + 1);        // six consumer warps and the merger read every descriptor
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&done[s], NC);
      mbar_init(&freeb[s], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  pdl_wait_prior();
  pdl_launch_dependents();

  const int T = t_dev ? max(1, min(*t_dev, p.T)) : p.T;
  const int BH = p.B * p.Hkv;

  // ---- item table: every CTA computes the same one.  Items are (head, piece) pairs; the heads whose
  // pieces are long (lists longer than num_splits * min_blocks: the refreshing heads) come first,
  // then the others, so that the work left for the end of the launch comes in short pieces.
  // pfx[0][bh], pfx[1][bh]: inclusive prefix sums of the piece counts of the long / the other heads.
  auto pieces_of = [&](int n_items) {
    int S_use = p.num_splits;
    if (min_blocks > 1) S_use = max(1, min(p.num_splits, (n_items + min_blocks - 1) / min_blocks));
    return S_use;
  };
  const int long_len = p.num_splits * max(min_blocks, 1);
  {
    constexpr int PER = TcqCfg::kMaxHeads / TcqCfg::kThreads;      // heads per thread
    int cl[PER], cs[PER], sl = 0, ss = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int bh = tid * PER + j;
      cl[j] = cs[j] = 0;
      if (bh < BH) {
        const int n_items = MASKED ? p.block_cnt[bh] : (T + TILE - 1) / TILE;
        const int c = pieces_of(n_items);
        if (n_items > long_len) cl[j] = c; else cs[j] = c;
      }
      sl += cl[j];
      ss += cs[j];
    }
    int il = sl, is = ss;                                           // inclusive scan over the threads
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int tl = __shfl_up_sync(0xffffffffu, il, o), ts = __shfl_up_sync(0xffffffffu, is, o);
      if (lane >= o) { il += tl; is += ts; }
    }
    if (lane == 31) { wsum[warp] = il; wsum[8 + warp] = is; }
    __syncthreads();
    int ol = 0, os = 0;
    for (int w = 0; w < warp; ++w) { ol += wsum[w]; os += wsum[8 + w]; }
    int rl = ol + il - sl, rs = os + is - ss;                       // exclusive offsets of this thread's first head
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int bh = tid * PER + j;
      rl += cl[j];
      rs += cs[j];
      if (bh < BH) { pfx[bh] = rl; pfx[TcqCfg::kMaxHeads + bh] = rs; }
    }
    __syncthreads();
  }

  if (warp == NC) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      const int total_long = pfx[BH - 1], total = total_long + pfx[TcqCfg::kMaxHeads + BH - 1];
      const int last_fetch = total + static_cast<int>(gridDim.x) - 1;
      int gi = 0, it = 0;
      int id = atomicAdd(queue, 1);
      bool ok = true;
#ifdef KVB_TIMELINE
      KVB_TL(1, tl_now());
#endif
      while (ok) {
        if (id >= total) {
          if (id == last_fetch) *queue = 0;              // every CTA has made its final fetch: ready for the next launch
          break;
        }
        // item id -> (head, piece): the first head whose inclusive prefix exceeds the index
        const int* pf = id < total_long ? pfx : pfx + TcqCfg::kMaxHeads;
        const int k = id < total_long ? id : id - total_long;
        int lo = 0, hi = BH - 1;
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          if (pf[mid] > k) hi = mid; else lo = mid + 1;
        }
        const int bh = lo;
        const int n_items = MASKED ? p.block_cnt[bh] : (T + TILE - 1) / TILE;
        const int S_use = pieces_of(n_items);
        const int piece = k - (pf[bh] - S_use);
#ifdef KVB_TIMELINE
        if (it == 0) KVB_TL(2, tl_now());
#endif
        const int per = (n_items + S_use - 1) / S_use;
        const int i0 = min(n_items, piece * per);
        const int n = min(n_items, i0 + per) - i0;
        const int b = bh / p.Hkv, h = bh % p.Hkv;
        const int qi = it % QD;
        if (it >= QD && !mbar_wait(&iempty[qi], ((it / QD) - 1) & 1, 0x220u + qi)) break;
        items[qi] = TcqItem{b, h, i0, n, n_items, S_use, piece, 0};
        mbar_arrive(&ifull[qi]);
        const int next = atomicAdd(queue, 1);            // in flight while this item's loads are issued
        const int32_t* list = MASKED ? p.block_idx + static_cast<int64_t>(bh) * p.max_blocks : nullptr;
        BlockAhead<MASKED> ahead;
        ahead.init(MASKED ? list + i0 : nullptr, pages ? pages + static_cast<int64_t>(b) * max_pages : nullptr, i0, n, b);
        for (int i = 0; i < n; ++i) {
          const int g2 = gi + i, s = g2 % S;
          if (g2 >= S && !mbar_wait(&empty[s], ((g2 / S) - 1) & 1, 0x200u + s)) { ok = false; break; }
          int blk, bp;
          ahead.next(i, blk, bp);
          const int t0 = pages ? 0 : blk * TILE;
          unsigned char* dst = ring + s * TcqCfg::kStageBytes;
          mbar_expect_tx(&full[s], TcqCfg::kStageBytes);
          tma_load_4d(dst, &maps.k, &full[s], 0, t0, h, bp);
          tma_load_4d(dst + TC_HALF_BYTES, &maps.k, &full[s], 64, t0, h, bp);
          tma_load_4d(dst + 2 * TC_HALF_BYTES, &maps.v, &full[s], 0, t0, h, bp);
          tma_load_4d(dst + 3 * TC_HALF_BYTES, &maps.v, &full[s], 64, t0, h, bp);
        }
        gi += n;
        ++it;
        id = next;
      }
#ifdef KVB_TIMELINE
      KVB_TL(3, tl_now());
      KVB_TL(6, static_cast<unsigned long long>(it));
      KVB_TL(7, static_cast<unsigned long long>(gi));
#endif
      // the end of this CTA's item stream, for the consumers and the merger
      const int qi = it % QD;
      if (it < QD || mbar_wait(&iempty[qi], ((it / QD) - 1) & 1, 0x228u + qi)) {
        items[qi] = TcqItem{0, 0, 0, 0, 0, 0, 0, 1};
        mbar_arrive(&ifull[qi]);
      }
    }
  } else if (warp < NC) {
    // ------------------------------------------------------------------ consumers
    const int head0 = 2 * (lane & 3);
    int gi = 0;
    for (int it = 0;; ++it) {
      const int qi = it % QD;
      if (!mbar_wait(&ifull[qi], (it / QD) & 1, 0x230u + qi)) break;
      const TcqItem d = items[qi];
      __syncwarp();
      if (lane == 0) mbar_arrive(&iempty[qi]);
      if (d.stop) break;
      const int b = d.b, h = d.h;
      const int32_t* list = MASKED ? p.block_idx + static_cast<int64_t>(b * p.Hkv + h) * p.max_blocks : nullptr;
      const int64_t hq0 = static_cast<int64_t>(b) * p.Hq + h * G;
      uint32_t bq[8][2];
      tc_load_q<8>(p, b, h, lane, bq);
      float m_run[2] = {-INFINITY, -INFINITY};
      float l_run[2] = {0.f, 0.f};
      float acc[8][4];
#pragma unroll
      for (int mt = 0; mt < 8; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[mt][c] = 0.f;
      // virtual warp of this piece: block i is folded by virtual warp i mod 6, which is the physical
      // warp that owns ring stage (gi + i) mod 6
      const int v = (warp - gi % NC + NC) % NC;
      bool ok = true;
      for (int i = v; i < d.n; i += NC) {
        const int g2 = gi + i, s = g2 % S;               // s == warp
        const int blk = MASKED ? list[d.i0 + i] : d.i0 + i;
        if constexpr (MASKED && STATS) tc_fill_gap(p, list, d.i0 + i, d.n_items, blk, hq0, lane);
        if (!mbar_wait(&full[s], (g2 / S) & 1, 0x210u + s)) { ok = false; break; }
        const uint32_t kbase = smem_u32(ring + s * TcqCfg::kStageBytes);
        if ((t_dev != nullptr || pages != nullptr) && blk * TILE + TILE > T) {
          // rows of the last block beyond the length: weights are zero, but the cache may hold NaN there
          const int r0 = T - blk * TILE;
          unsigned char* vst = ring + s * TcqCfg::kStageBytes + 2 * TC_HALF_BYTES;
          for (int o = r0 * 128 + lane * 16; o < TILE * 128; o += 32 * 16) {
            *reinterpret_cast<uint4*>(vst + o) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(vst + TC_HALF_BYTES + o) = make_uint4(0u, 0u, 0u, 0u);
          }
          fence_proxy_async_smem();
          __syncwarp();
        }
#ifdef KVB_TIMELINE
        if (g2 == 0 && lane == 0) KVB_TL(4, tl_now());
#endif
        tc_block<STATS, true>(p, kbase, bq, blk, hq0, lane, T, m_run, l_run, acc);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
#ifdef KVB_TIMELINE
        if (lane == 0) g_timeline[blockIdx.x * 16 + 10 + (warp % 6 == 0 ? 0 : 1)] = tl_now();   // last block done (warp 0 / others)
#endif
      }
      if (!ok) break;
      gi += d.n;
      if constexpr (MASKED && STATS) {
        if (d.n_items == 0 && d.piece == 0 && v == 0)    // an empty list: every block of this KV head is unread
          for (int gblk = lane; gblk < p.nb; gblk += 32)
#pragma unroll
            for (int g = 0; g < G; ++g) {
              p.blk_max[(hq0 + g) * p.nb + gblk] = -INFINITY;
              p.blk_sum[(hq0 + g) * p.nb + gblk] = 0.f;
            }
      }
      if constexpr (!MASKED && STATS) {
        if (t_dev != nullptr && d.piece == 0 && v == 0)
          for (int gblk = d.n_items + lane; gblk < p.nb; gblk += 32)
#pragma unroll
            for (int g = 0; g < G; ++g) {
              p.blk_max[(hq0 + g) * p.nb + gblk] = -INFINITY;
              p.blk_sum[(hq0 + g) * p.nb + gblk] = 0.f;
            }
      }
      // hand the state of virtual warp v to the merger
      const int buf = it & 1;
      if (it >= 2 && !mbar_wait(&freeb[buf], ((it >> 1) - 1) & 1, 0x240u + buf)) break;
      l_run[0] = quadcol_sum(l_run[0]);
      l_run[1] = quadcol_sum(l_run[1]);
      if (lane < 2) {
        sM[(buf * NC + v) * G + head0] = m_run[0];
        sM[(buf * NC + v) * G + head0 + 1] = m_run[1];
        sL[(buf * NC + v) * G + head0] = l_run[0];
        sL[(buf * NC + v) * G + head0 + 1] = l_run[1];
      }
      if ((lane & 3) < 2) {
        float* red = stg + static_cast<size_t>(buf * NC + v) * G * D;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt)
#pragma unroll
          for (int c = 0; c < 4; ++c) red[(head0 + (c & 1)) * D + mt * 16 + (lane >> 2) + (c >> 1) * 8] = acc[mt][c];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&done[buf]);
    }
  } else {
    // ------------------------------------------------------------------ merger
    for (int it = 0;; ++it) {
      const int qi = it % QD;
      if (!mbar_wait(&ifull[qi], (it / QD) & 1, 0x250u + qi)) break;
      const TcqItem d = items[qi];
      __syncwarp();
      if (lane == 0) mbar_arrive(&iempty[qi]);
      if (d.stop) break;
      const int buf = it & 1;
      if (!mbar_wait(&done[buf], (it >> 1) & 1, 0x260u + buf)) break;
      // the six states of the piece, merged in virtual-warp order; lane owns outputs lane + 32 j
      const float* red = stg + static_cast<size_t>(buf) * NC * G * D;
      const float* bM = sM + buf * NC * G;
      const float* bL = sL + buf * NC * G;
      float sum[16], Mg[G], Lg[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NC; ++w) M = fmaxf(M, bM[w * G + g]);
        const float mu = (M == -INFINITY) ? 0.f : M;
        float l = 0.f;
#pragma unroll
        for (int w = 0; w < NC; ++w) l += bL[w * G + g] * ex2(bM[w * G + g] - mu);
        Mg[g] = M;
        Lg[g] = l;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int o = lane + 32 * j, g = o >> 7, dd = o & 127;       // g == j / 4
        const float mu = (Mg[g] == -INFINITY) ? 0.f : Mg[g];
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < NC; ++w) a += red[(w * G + g) * D + dd] * ex2(bM[w * G + g] - mu);
        sum[j] = a;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&freeb[buf]);                       // the staging buffer can be written again
      const int64_t hq0 = static_cast<int64_t>(d.b) * p.Hq + d.h * G;
      if (d.S_use == 1) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int o = lane + 32 * j, g = o >> 7, dd = o & 127;
          const float o32 = Lg[g] > 0.f ? sum[j] / Lg[g] : 0.f;
          reinterpret_cast<__nv_bfloat16*>(p.out)[(hq0 + g) * D + dd] = __float2bfloat16(o32);
          if (p.out_f32) p.out_f32[(hq0 + g) * D + dd] = o32;
        }
        if (lane < G && p.lse) p.lse[hq0 + lane] = Lg[lane] > 0.f ? (Mg[lane] + log2f(Lg[lane])) * LN2 : -INFINITY;
        continue;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int o = lane + 32 * j, g = o >> 7, dd = o & 127;
        p.part_acc[((hq0 + g) * p.num_splits + d.piece) * D + dd] = sum[j];
      }
      if (lane < G) {
        p.part_ml[((hq0 + lane) * p.num_splits + d.piece) * 2] = Mg[lane];
        p.part_ml[((hq0 + lane) * p.num_splits + d.piece) * 2 + 1] = Lg[lane];
      }
      __threadfence();              // this piece's partial is visible device-wide before it is counted
      __syncwarp();
      int last = 0;
      if (lane == 0) last = atomicAdd(&split_done[d.b * p.Hkv + d.h], 1) == d.S_use - 1;
      last = __shfl_sync(0xffffffffu, last, 0);
      if (!last) continue;
      __threadfence();
      // merge of the head's pieces in the order of tc_merge_pieces (four interleaved chains per output
      // element: pieces s = u mod 4 ascending, combined (c0 + c1) + (c2 + c3)).  This warp is the tail
      // of the head (and, for the last head, of the launch), so it is written for few memory round
      // trips: the maxima of all four query heads in one, then two query heads at a time, a lane
      // owning four consecutive outputs of each (one 16-byte load per piece) and up to 12 pieces of
      // both heads requested before any of them is used.
      {
        const int Su = d.S_use, ns = p.num_splits;
        constexpr int BATCH = 12;                         // pieces in flight: a multiple of 4 (chain u = s mod 4)
        float mh[G];
#pragma unroll
        for (int g = 0; g < G; ++g) mh[g] = -INFINITY;
        for (int s0 = 0; s0 < Su; s0 += BATCH) {
          float t[G][BATCH];
#pragma unroll
          for (int g = 0; g < G; ++g)
#pragma unroll
            for (int u = 0; u < BATCH; ++u)
              t[g][u] = s0 + u < Su ? __ldcg(p.part_ml + ((hq0 + g) * ns + s0 + u) * 2) : -INFINITY;
#pragma unroll
          for (int g = 0; g < G; ++g)
#pragma unroll
            for (int u = 0; u < BATCH; ++u) mh[g] = fmaxf(mh[g], t[g][u]);
        }
#pragma unroll 1
        for (int g0 = 0; g0 < G; g0 += 2) {
          float l[2][4], a[2][4][4], mu[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float m = g0 == 0 ? mh[e] : mh[2 + e];
            mu[e] = (m == -INFINITY) ? 0.f : m;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              l[e][u] = 0.f;
#pragma unroll
              for (int j = 0; j < 4; ++j) a[e][u][j] = 0.f;
            }
          }
          for (int s0 = 0; s0 < Su; s0 += BATCH) {
            float w[2][BATCH], pl[2][BATCH];
            float4 x[2][BATCH];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int64_t hq = hq0 + g0 + e;
              const float* ml = p.part_ml + hq * ns * 2;
              const float* pa = p.part_acc + hq * ns * D + 4 * lane;
#pragma unroll
              for (int u = 0; u < BATCH; ++u) {
                const int s2 = min(s0 + u, Su - 1);
                w[e][u] = __ldcg(ml + 2 * s2);
                pl[e][u] = __ldcg(ml + 2 * s2 + 1);
                x[e][u] = __ldcg(reinterpret_cast<const float4*>(pa + static_cast<int64_t>(s2) * D));
              }
            }
#pragma unroll
            for (int e = 0; e < 2; ++e)
#pragma unroll
              for (int u = 0; u < BATCH; ++u) {
                if (s0 + u < Su) {
                  const float ww = ex2(w[e][u] - mu[e]);
                  l[e][u & 3] += pl[e][u] * ww;
                  a[e][u & 3][0] += x[e][u].x * ww;
                  a[e][u & 3][1] += x[e][u].y * ww;
                  a[e][u & 3][2] += x[e][u].z * ww;
                  a[e][u & 3][3] += x[e][u].w * ww;
                }
              }
          }
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int64_t hq = hq0 + g0 + e;
            const float m = g0 == 0 ? mh[e] : mh[2 + e];
            const float lt = (l[e][0] + l[e][1]) + (l[e][2] + l[e][3]);
            float o32[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float at = (a[e][0][j] + a[e][1][j]) + (a[e][2][j] + a[e][3][j]);
              o32[j] = lt > 0.f ? at / lt : 0.f;
            }
            __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(p.out) + hq * D + 4 * lane);
            ob[0] = __floats2bfloat162_rn(o32[0], o32[1]);
            ob[1] = __floats2bfloat162_rn(o32[2], o32[3]);
            if (p.out_f32)
              *reinterpret_cast<float4*>(p.out_f32 + hq * D + 4 * lane) = make_float4(o32[0], o32[1], o32[2], o32[3]);
            if (lane == 0 && p.lse) p.lse[hq] = lt > 0.f ? (m + log2f(lt)) * LN2 : -INFINITY;
          }
        }
      }
      if (lane == 0) split_done[d.b * p.Hkv + d.h] = 0;
    }
#ifdef KVB_TIMELINE
    if (lane == 0) KVB_TL(5, tl_now());
#endif
  }
}

}  // namespace kvb
