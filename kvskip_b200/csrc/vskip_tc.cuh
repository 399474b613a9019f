// Single-pass V-skip on the tensor-core path (D = 128, G = 4).
//
// Same rule as vskip1_kernel (vskip.cuh): all of K is streamed; the V block of a tile is fetched
// only if the tile is block 0, one of the `local` newest, or some query head of the group gives
// it  lse_block - lse0 >= log2(tau); a skipped block contributes neither to the output nor to the
// normaliser.  Layout as decode_tc_kernel: a producer warp feeds a K ring (one 16 KB stage per
// consumer warp); a consumer warp owns whole blocks, so the vote is warp-local (`__any_sync`).
// The warp that voted "yes" issues the TMA load of that V block itself into its private V buffer
// and retires the P.V product one block later, after the scores of its next block, so the V load
// overlaps useful work and skipped V bytes never leave HBM.
#pragma once
#include "decode_tc.cuh"

namespace kvb {

struct Vs1TcCfg {
  static constexpr int kKBytes = 2 * TC_HALF_BYTES;          // one K block
  static constexpr int kVBytes = 2 * TC_HALF_BYTES;          // one V block
  static constexpr int kAuxBytes = TC_CONSUMERS * 8 * 4 + 4 * 4 + (3 * TC_CONSUMERS + 1) * 8 + 64;
  static constexpr int kSmemBytes = TC_CONSUMERS * (kKBytes + kVBytes) + kAuxBytes + 1024;
};

__global__ void __launch_bounds__(TC_THREADS, 1)
vskip1_tc_kernel(const kvskip_params p, const __grid_constant__ TmaMaps maps, int* __restrict__ split_done,
                 const int32_t* __restrict__ pages, const int max_pages, const int* __restrict__ t_dev) {
  constexpr int G = 4, D = 128;
  constexpr int NC = TC_CONSUMERS;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* ringK = smem;                                             // [NC] key stages
  unsigned char* bufV = smem + NC * Vs1TcCfg::kKBytes;                     // [NC] value buffers, one per warp
  float* sM = reinterpret_cast<float*>(bufV + NC * Vs1TcCfg::kVBytes);     // [NC][4]
  float* sL = sM + NC * 4;                                                 // [NC][4]
  float* sLse0 = sL + NC * 4;                                              // [4] sink-block lse (log2 units)
  uint64_t* kfull = reinterpret_cast<uint64_t*>(sLse0 + 4);                // [NC]
  uint64_t* kempty = kfull + NC;                                           // [NC]
  uint64_t* vfull = kempty + NC;                                           // [NC]
  uint64_t* pro = vfull + NC;                                              // sink-block prologue

  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool sink_rule = p.lse_prev == nullptr;

  if (tid == 0) {
    tma_prefetch_desc(&maps.k);
    tma_prefetch_desc(&maps.v);
    for (int s = 0; s < NC; ++s) {
      mbar_init(&kfull[s], 1);
      mbar_init(&kempty[s], 1);
      mbar_init(&vfull[s], 1);
    }
    mbar_init(pro, 1);
    mbar_fence_init();
  }
  __syncthreads();
  pdl_wait_prior();          // nothing written by the previous kernel on the stream is read above
  pdl_launch_dependents();
  // the length: p.T, or the value at t_dev (p.T is then the bound the grid and the maps were sized for)
  const int T = t_dev ? max(1, min(*t_dev, p.T)) : p.T;
  const int nb = (T + TILE - 1) / TILE;
  const int per = (nb + p.num_splits - 1) / p.num_splits;
  const int i0 = min(nb, split * per);
  const int n = min(nb, i0 + per) - i0;
  // contiguous cache: rows blk*64.. of sequence b; paged cache (pages != nullptr): the whole page
  // the table names for block blk -- the maps then run over the page pool
  auto row_of = [&](int blk) { return pages ? 0 : blk * TILE; };
  auto seq_of = [&](int blk) { return pages ? pages[static_cast<int64_t>(b) * max_pages + blk] : b; };

  const int lrow = lane & 7, lmat = lane >> 3;
  const int64_t hq0 = static_cast<int64_t>(b) * p.Hq + h * G;
  const bool col_ok = (lane & 3) < 2;
  const int head0 = 2 * (lane & 3);

  // Q^T fragments (B operand of the score MMA), as in decode_tc_kernel
  uint32_t bq[8][2];
  {
    const int head = lane >> 2;
    const uint16_t* qp = p.q + b * p.q_sb + (h * G + (head & 3)) * p.q_sh + 2 * (lane & 3);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      bq[ks][0] = head < G ? *reinterpret_cast<const uint32_t*>(qp + ks * 16) : 0u;
      bq[ks][1] = head < G ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8) : 0u;
    }
  }
  // scores of one K block in log2 units, tokens past T masked
  auto scores = [&](uint32_t kbase, int t0, float (&sc)[4][4]) {
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int c = 0; c < 4; ++c) sc[mt][c] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
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
    const bool ragged = t0 + TILE > T;
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float v = sc[mt][c] * p.scale_log2;
        if (ragged && t0 + mt * 16 + (lane >> 2) + (c >> 1) * 8 >= T) v = -INFINITY;
        sc[mt][c] = v;
      }
  };
  // block max and block log-sum-exp of this thread's two heads
  auto block_lse = [&](const float (&sc)[4][4], float (&mb)[2], float (&lse_b)[2]) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float v = fmaxf(sc[0][e], sc[0][e + 2]);
#pragma unroll
      for (int mt = 1; mt < 4; ++mt) v = fmaxf(v, fmaxf(sc[mt][e], sc[mt][e + 2]));
      mb[e] = quadcol_max(v);
    }
    const float mtu[2] = {mb[0] == -INFINITY ? 0.f : mb[0], mb[1] == -INFINITY ? 0.f : mb[1]};
    float es[2] = {0.f, 0.f};
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int c = 0; c < 4; ++c) es[c & 1] += ex2(sc[mt][c] - mtu[c & 1]);
    lse_b[0] = mtu[0] + log2f(quadcol_sum(es[0]));
    lse_b[1] = mtu[1] + log2f(quadcol_sum(es[1]));
  };

  // ---- normaliser estimate: the sink block's lse, computed once per CTA by warp 0
  if (sink_rule) {
    if (warp == NC && lane == 0) {
      mbar_expect_tx(pro, Vs1TcCfg::kKBytes);
      tma_load_4d(ringK, &maps.k, pro, 0, 0, h, seq_of(0));
      tma_load_4d(ringK + TC_HALF_BYTES, &maps.k, pro, 64, 0, h, seq_of(0));
    }
    if (warp == 0) {
      if (mbar_wait(pro, 0, 0x340u)) {
        float sc[4][4], mb[2], lb[2];
        scores(smem_u32(ringK), 0, sc);
        block_lse(sc, mb, lb);
        if (lane < 2) {
          sLse0[head0] = lb[0];
          sLse0[head0 + 1] = lb[1];
        }
      }
    }
    __syncthreads();   // lse0 visible; stage 0 free again
  }

  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float acc[8][4];
#pragma unroll
  for (int mt = 0; mt < 8; ++mt)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[mt][c] = 0.f;

  if (warp == NC) {
    if (lane == 0) {
      for (int i = 0; i < n; ++i) {
        const int s = i % NC;
        if (i >= NC && !mbar_wait(&kempty[s], ((i / NC) - 1) & 1, 0x350u + s)) break;
        const int t0 = row_of(i0 + i), bp = seq_of(i0 + i);
        mbar_expect_tx(&kfull[s], Vs1TcCfg::kKBytes);
        tma_load_4d(ringK + s * Vs1TcCfg::kKBytes, &maps.k, &kfull[s], 0, t0, h, bp);
        tma_load_4d(ringK + s * Vs1TcCfg::kKBytes + TC_HALF_BYTES, &maps.k, &kfull[s], 64, t0, h, bp);
      }
    }
  } else {
    float lse0[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      if (!col_ok) lse0[e] = INFINITY;                       // padding columns never vote
      else if (sink_rule) lse0[e] = sLse0[head0 + e];
      else lse0[e] = p.lse_prev[hq0 + head0 + e] * LOG2E;
    }
    const uint32_t vbase = smem_u32(bufV + warp * Vs1TcCfg::kVBytes);
    uint32_t pend_b[4][4];          // P of the pending block as B fragments: [16-token step][hi0, hi1, lo0, lo1]
    float pend_alpha[2] = {1.f, 1.f};
    bool pending = false;
    int pend_rows = TILE;
    uint32_t vphase = 0;
    int loaded = 0;
    bool ok = true;

    auto retire = [&]() {           // acc = alpha * acc + V^T P^T for the pending block
      if (!mbar_wait(&vfull[warp], vphase ^ 1u, 0x360u + warp)) { ok = false; return; }
      if ((pages != nullptr || t_dev != nullptr) && pend_rows < TILE) {
        // paged cache: the rows of the last page past the sequence hold stale data; their weights
        // are zero but 0 x NaN is not, so clear them (whole 128-byte rows of both halves)
        unsigned char* vb = bufV + warp * Vs1TcCfg::kVBytes;
        for (int o = pend_rows * 128 + lane * 16; o < TILE * 128; o += 32 * 16) {
          *reinterpret_cast<uint4*>(vb + o) = make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4*>(vb + TC_HALF_BYTES + o) = make_uint4(0u, 0u, 0u, 0u);
        }
        fence_proxy_async_smem();   // every writing lane: ordered before the next bulk load into this buffer
        __syncwarp();
      }
      if (__any_sync(0xffffffffu, pend_alpha[0] != 1.f || pend_alpha[1] != 1.f)) {
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
          acc[mt][0] *= pend_alpha[0]; acc[mt][1] *= pend_alpha[1];
          acc[mt][2] *= pend_alpha[0]; acc[mt][3] *= pend_alpha[1];
        }
      }
#pragma unroll
      for (int kt = 0; kt < 4; ++kt) {
        const int tok = kt * 16 + (lmat >> 1) * 8 + lrow;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
          const int dchunk = mt * 2 + (lmat & 1);
          uint32_t a[4];
          ldsm_x4_t(a, vbase + (dchunk >> 3) * TC_HALF_BYTES + tok * 128 + (((dchunk & 7) ^ lrow) << 4));
          mma_bf16(acc[mt], a, pend_b[kt][0], pend_b[kt][1]);
          mma_bf16(acc[mt], a, pend_b[kt][2], pend_b[kt][3]);
        }
      }
      pending = false;
    };

    for (int i = warp; i < n && ok; i += NC) {
      const int s = i % NC;                                  // == warp
      const int blk = i0 + i;
      if (!mbar_wait(&kfull[s], (i / NC) & 1, 0x370u + s)) break;
      float sc[4][4], mb[2], lse_b[2];
      scores(smem_u32(ringK + s * Vs1TcCfg::kKBytes), blk * TILE, sc);
      __syncwarp();
      if (lane == 0) mbar_arrive(&kempty[s]);                // the key block is not needed any more
      block_lse(sc, mb, lse_b);
      const bool vote = (lse_b[0] - lse0[0] >= p.log2_tau) || (lse_b[1] - lse0[1] >= p.log2_tau);
      const bool need = blk == 0 || blk >= nb - p.local || __any_sync(0xffffffffu, vote);
      if (pending) retire();                                 // frees the V buffer and brings acc up to date
      if (!ok) break;
      if (need) {
        float alpha[2], mu[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float m_new = fmaxf(m_run[e], mb[e]);
          mu[e] = (m_new == -INFINITY) ? 0.f : m_new;
          alpha[e] = ex2(m_run[e] - mu[e]);
          m_run[e] = m_new;
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
        pend_alpha[0] = alpha[0];
        pend_alpha[1] = alpha[1];
#pragma unroll
        for (int kt = 0; kt < 4; ++kt) {
          const uint32_t h0 = pack_bf16(sc[kt][0], sc[kt][1]);
          const uint32_t h1 = pack_bf16(sc[kt][2], sc[kt][3]);
          const uint32_t l0 = pack_bf16(sc[kt][0] - bf_lo(h0), sc[kt][1] - bf_hi(h0));
          const uint32_t l1 = pack_bf16(sc[kt][2] - bf_lo(h1), sc[kt][3] - bf_hi(h1));
          pend_b[kt][0] = movm_t(h0);
          pend_b[kt][1] = movm_t(h1);
          pend_b[kt][2] = movm_t(l0);
          pend_b[kt][3] = movm_t(l1);
        }
        __syncwarp();                                        // every lane is done reading the V buffer
        if (lane == 0) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          mbar_expect_tx(&vfull[warp], Vs1TcCfg::kVBytes);
          const int tv = row_of(blk), bv = seq_of(blk);
          tma_load_4d(bufV + warp * Vs1TcCfg::kVBytes, &maps.v, &vfull[warp], 0, tv, h, bv);
          tma_load_4d(bufV + warp * Vs1TcCfg::kVBytes + TC_HALF_BYTES, &maps.v, &vfull[warp], 64, tv, h, bv);
        }
        vphase ^= 1u;                                        // retire() waits for parity vphase ^ 1
        pending = true;
        pend_rows = min(TILE, T - blk * TILE);               // rows of the block that hold tokens
        ++loaded;
      }
    }
    if (pending && ok) retire();
    if (lane == 0 && p.vcount && loaded) atomicAdd(p.vcount + b * p.Hkv + h, loaded);
    l_run[0] = quadcol_sum(l_run[0]);
    l_run[1] = quadcol_sum(l_run[1]);
    if (lane < 2) {
      sM[warp * 4 + head0] = m_run[0];
      sM[warp * 4 + head0 + 1] = m_run[1];
      sL[warp * 4 + head0] = l_run[0];
      sL[warp * 4 + head0 + 1] = l_run[1];
    }
  }
  __syncthreads();

  // ---- merge of the consumer warps, then of the splits (as decode_tc_kernel)
  float* red = reinterpret_cast<float*>(ringK);   // [NC][G][D]
  if (warp < NC && (lane & 3) < 2) {
#pragma unroll
    for (int mt = 0; mt < 8; ++mt)
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
    const int64_t hq = hq0 + g;
    if (p.num_splits == 1) {
      const float o32 = l > 0.f ? sum / l : 0.f;
      reinterpret_cast<__nv_bfloat16*>(p.out)[hq * D + d] = __float2bfloat16(o32);
      if (p.out_f32) p.out_f32[hq * D + d] = o32;
    } else {
      p.part_acc[(hq * p.num_splits + split) * D + d] = sum;
    }
  }
  if (tid < G) {
    float M = -INFINITY;
    for (int w = 0; w < NC; ++w) M = fmaxf(M, sM[w * 4 + tid]);
    const float mu = (M == -INFINITY) ? 0.f : M;
    float l = 0.f;
    for (int w = 0; w < NC; ++w) l += sL[w * 4 + tid] * ex2(sM[w * 4 + tid] - mu);
    const int64_t hq = hq0 + tid;
    if (p.num_splits == 1) {
      if (p.lse) p.lse[hq] = l > 0.f ? (M + log2f(l)) * LN2 : -INFINITY;
    } else {
      p.part_ml[(hq * p.num_splits + split) * 2] = M;
      p.part_ml[(hq * p.num_splits + split) * 2 + 1] = l;
    }
  }
  if (p.num_splits > 1 && split_done != nullptr) {
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(&split_done[b * p.Hkv + h], 1) == p.num_splits - 1;
    __syncthreads();
    if (s_last) {
      __threadfence();
      const int S2 = p.num_splits;
      for (int o = tid; o < G * D; o += TC_THREADS) {
        const int g = o / D, d = o % D;
        const int64_t hq = hq0 + g;
        const float* ml = p.part_ml + hq * S2 * 2;
        float m = -INFINITY;
        for (int s2 = 0; s2 < S2; ++s2) m = fmaxf(m, __ldcg(ml + 2 * s2));
        const float mu = (m == -INFINITY) ? 0.f : m;
        float l = 0.f, a = 0.f;
        for (int s2 = 0; s2 < S2; ++s2) {
          const float w = ex2(__ldcg(ml + 2 * s2) - mu);
          l += __ldcg(ml + 2 * s2 + 1) * w;
          a += __ldcg(p.part_acc + (hq * S2 + s2) * D + d) * w;
        }
        const float o32 = l > 0.f ? a / l : 0.f;
        reinterpret_cast<__nv_bfloat16*>(p.out)[hq * D + d] = __float2bfloat16(o32);
        if (p.out_f32) p.out_f32[hq * D + d] = o32;
        if (d == 0 && p.lse) p.lse[hq] = l > 0.f ? (m + log2f(l)) * LN2 : -INFINITY;
      }
      if (tid == 0) split_done[b * p.Hkv + h] = 0;
    }
  }
}

}  // namespace kvb
