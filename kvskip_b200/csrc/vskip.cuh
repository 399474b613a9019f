// Single-pass V-skip and the second pass of the two-pass V-skip, plus the streaming-read probe.
//
// vskip1: all of K is streamed (TMA ring); the V block of a tile is requested only after the
// tile's block log-sum-exp has been compared with the normaliser estimate (vote per query head,
// OR over the group, block 0 and the `local` newest blocks always pass), so skipped V bytes never
// leave HBM.  A skipped block contributes neither to the output nor to the normaliser.  Rule and
// arithmetic follow format37/kvskip's vskip1_kernel (kernels/kvskip_kernel.cu:482-704); the PV of
// tile i runs one iteration later so the V load overlaps the next tile's scores.
//
// pv: out = sum over listed blocks of blk_scale * P * V with P (fp16) from a statistics pass
// (kernels/kvskip_kernel.cu:316-431); weights are already normalised, splits just add.
#pragma once
#include "common.cuh"
#include "decode_exact.cuh"

namespace kvb {

template <int D>
struct Vskip1Cfg {
  static constexpr int kTileBytes = TILE * D * 2;
  static constexpr int kKStages = 6;
  static constexpr int kAuxFloats = 4 * TILE + 2 * TILE * 4 + 2 * 4 + 8 + 4;
  static constexpr int kSmemBytes = (kKStages + 2) * kTileBytes + kAuxFloats * 4 + (kKStages + 3) * 8 + 128;
};

template <int D>
__global__ void __launch_bounds__(EX_THREADS, 1)
vskip1_kernel(const kvskip_params p, const __grid_constant__ TmaMaps maps) {
  using Cfg = Vskip1Cfg<D>;
  constexpr int G = 4;
  constexpr int SK = Cfg::kKStages;
  constexpr int CH = D / 64;
  constexpr int DPL = D / 32;

  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* sK = smem;                                   // [SK] key tiles
  unsigned char* sV = smem + SK * Cfg::kTileBytes;            // [2] value tiles
  float* sS = reinterpret_cast<float*>(sV + 2 * Cfg::kTileBytes);   // [G][TILE]
  float* sP = sS + G * TILE;                                  // [2][TILE][G]
  float* sA = sP + 2 * TILE * G;                              // [2][G]
  float* sML = sA + 2 * G;                                    // [G][2]
  int* sVote = reinterpret_cast<int*>(sML + 2 * G);           // [G]
  uint64_t* kfull = reinterpret_cast<uint64_t*>(sVote + G);   // [SK]
  uint64_t* vfull = kfull + SK;                               // [2]
  uint64_t* pro = vfull + 2;                                  // sink-block prologue

  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quad = lane >> 3, j = lane & 7;
  const int nb = (p.T + TILE - 1) / TILE;
  const int per = (nb + p.num_splits - 1) / p.num_splits;
  const int i0 = min(nb, split * per);
  const int n = min(nb, i0 + per) - i0;

  if (tid == 0) {
    tma_prefetch_desc(&maps.k);
    tma_prefetch_desc(&maps.v);
    for (int s = 0; s < SK; ++s) mbar_init(&kfull[s], 1);
    mbar_init(&vfull[0], 1);
    mbar_init(&vfull[1], 1);
    mbar_init(pro, 1);
    mbar_fence_init();
  }
  __syncthreads();

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

  auto scores = [&](const uint16_t* tK, int t0) {
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
  };

  // normaliser estimate of this warp's head, log2 units
  float lse0;
  if (p.lse_prev) {
    lse0 = p.lse_prev[static_cast<int64_t>(b) * p.Hq + h * G + warp] * LOG2E;
  } else {
    if (tid == 0) {
      mbar_expect_tx(pro, Cfg::kTileBytes);
      tma_load_4d(sK, &maps.k, pro, 0, 0, h, b);
    }
    mbar_wait(pro, 0, 0x300u);
    scores(reinterpret_cast<const uint16_t*>(sK), 0);
    __syncthreads();
    const float s0 = sS[warp * TILE + lane], s1 = sS[warp * TILE + lane + 32];
    const float m0 = warp_max(fmaxf(s0, s1));
    lse0 = m0 + log2f(warp_sum(ex2(s0 - m0) + ex2(s1 - m0)));
    __syncthreads();   // stage 0 and the score buffer are reused below
  }

  auto issue_k = [&](int i) {
    const int s = i % SK;
    mbar_expect_tx(&kfull[s], Cfg::kTileBytes);
    tma_load_4d(sK + s * Cfg::kTileBytes, &maps.k, &kfull[s], 0, (i0 + i) * TILE, h, b);
  };
  if (tid == 0)
    for (int i = 0; i < SK - 1 && i < n; ++i) issue_k(i);

  float m_run = -INFINITY, l_run = 0.f;
  float acc[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < DPL; ++e) acc[g][e] = 0.f;
  int loaded = 0;
  uint32_t vphase[2] = {0u, 0u};     // parity the next load into each V buffer completes
  uint32_t vwait[2] = {0u, 0u};      // parity to wait for the latest load of each V buffer
  bool need_prev = false;

  auto pv_tile = [&](int buf) {
    const uint16_t* tV = reinterpret_cast<const uint16_t*>(sV + buf * Cfg::kTileBytes);
    const float* tP = sP + buf * TILE * G;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float a = sA[buf * G + g];
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
      const float4 pr = *reinterpret_cast<const float4*>(tP + r * G);
      const float pg[4] = {pr.x, pr.y, pr.z, pr.w};
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < DPL; ++e) acc[g][e] = fmaf(pg[g], vf[e], acc[g][e]);
    }
  };

  for (int i = 0; i < n; ++i) {
    const int s = i % SK;
    if (!mbar_wait(&kfull[s], (i / SK) & 1, 0x310u + s)) break;
    const int blk = i0 + i;
    const int buf = i & 1;
    scores(reinterpret_cast<const uint16_t*>(sK + s * Cfg::kTileBytes), blk * TILE);
    __syncthreads();
    if (tid == 0 && i + SK - 1 < n) issue_k(i + SK - 1);
    const int g = warp;
    const float s0 = sS[g * TILE + lane], s1 = sS[g * TILE + lane + 32];
    const float mt = warp_max(fmaxf(s0, s1));
    const float mtu = (mt == -INFINITY) ? 0.f : mt;
    const float lse_b = mtu + log2f(warp_sum(ex2(s0 - mtu) + ex2(s1 - mtu)));
    if (lane == 0) sVote[g] = (lse_b - lse0 >= p.log2_tau) ? 1 : 0;
    __syncthreads();
    bool need = blk == 0 || blk >= nb - p.local;
#pragma unroll
    for (int w = 0; w < G; ++w) need = need || sVote[w];
    if (need) {
      const float m_new = fmaxf(m_run, mt);
      const float mu = (m_new == -INFINITY) ? 0.f : m_new;
      const float p0 = ex2(s0 - mu), p1 = ex2(s1 - mu);
      const float alpha = ex2(m_run - mu);
      l_run = l_run * alpha + warp_sum(p0 + p1);
      m_run = m_new;
      sP[(buf * TILE + lane) * G + g] = p0;
      sP[(buf * TILE + lane + 32) * G + g] = p1;
      if (lane == 0) sA[buf * G + g] = alpha;
      if (tid == 0) {
        mbar_expect_tx(&vfull[buf], Cfg::kTileBytes);
        tma_load_4d(sV + buf * Cfg::kTileBytes, &maps.v, &vfull[buf], 0, blk * TILE, h, b);
      }
      vwait[buf] = vphase[buf];
      vphase[buf] ^= 1u;
      ++loaded;
    }
    if (i > 0 && need_prev) {
      if (!mbar_wait(&vfull[buf ^ 1], vwait[buf ^ 1], 0x320u + (buf ^ 1))) break;
      pv_tile(buf ^ 1);
    }
    need_prev = need;
  }
  if (n > 0 && need_prev) {
    const int buf = (n - 1) & 1;
    __syncthreads();   // probabilities of the last tile visible to every warp
    if (mbar_wait(&vfull[buf], vwait[buf], 0x330u + buf)) pv_tile(buf);
  }

  if (lane == 0) {
    sML[2 * warp] = m_run;
    sML[2 * warp + 1] = l_run;
  }
  if (tid == 0 && p.vcount) atomicAdd(p.vcount + b * p.Hkv + h, loaded);
  __syncthreads();
  float* red = reinterpret_cast<float*>(sK);
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

template <int D>
struct PvCfg {
  static constexpr int kTileBytes = TILE * D * 2;
  static constexpr int kStages = 8;
  static constexpr int kSmemBytes = kStages * kTileBytes + 2 * 4 * TILE * 4 + kStages * 8 + 128;
};

template <int D>
__global__ void __launch_bounds__(EX_THREADS, 1)
pv_kernel(const kvskip_params p, const __grid_constant__ TmaMaps maps) {
  using Cfg = PvCfg<D>;
  constexpr int G = 4;
  constexpr int S = Cfg::kStages;
  constexpr int DPL = D / 32;
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* sV = smem;
  float* sP = reinterpret_cast<float*>(smem + S * Cfg::kTileBytes);   // [2][G][TILE], weight applied
  uint64_t* full = reinterpret_cast<uint64_t*>(sP + 2 * G * TILE);

  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_items = p.block_cnt[b * p.Hkv + h];
  const int32_t* list = p.block_idx + static_cast<int64_t>(b * p.Hkv + h) * p.max_blocks;
  const int per = (n_items + p.num_splits - 1) / p.num_splits;
  const int i0 = min(n_items, split * per);
  const int n = min(n_items, i0 + per) - i0;
  const int64_t hq0 = static_cast<int64_t>(b) * p.Hq + h * G;

  if (tid == 0) {
    tma_prefetch_desc(&maps.v);
    for (int s = 0; s < S; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  auto issue = [&](int i) {
    const int s = i % S;
    mbar_expect_tx(&full[s], Cfg::kTileBytes);
    tma_load_4d(sV + s * Cfg::kTileBytes, &maps.v, &full[s], 0, list[i0 + i] * TILE, h, b);
  };
  if (tid == 0)
    for (int i = 0; i < S - 1 && i < n; ++i) issue(i);

  // thread (warp g, lane) stages tokens 2*lane, 2*lane+1 of head g, already times the block weight
  auto fetch = [&](int i, float& w0, float& w1) {
    const int blk = list[i0 + i];
    const float f = p.blk_scale[((static_cast<int64_t>(b) * p.Hkv + h) * p.nb + blk) * G + warp];
    const __half2 hh = *reinterpret_cast<const __half2*>(reinterpret_cast<const __half*>(p.p_in) +
                                                          (hq0 + warp) * p.t_pad + blk * TILE + 2 * lane);
    w0 = __half2float(__low2half(hh)) * f;
    w1 = __half2float(__high2half(hh)) * f;
  };
  float w0 = 0.f, w1 = 0.f;
  if (n > 0) {
    fetch(0, w0, w1);
    sP[warp * TILE + 2 * lane] = w0;
    sP[warp * TILE + 2 * lane + 1] = w1;
  }
  float acc[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < DPL; ++e) acc[g][e] = 0.f;

  for (int i = 0; i < n; ++i) {
    __syncthreads();   // weights of tile i staged; everyone is past the PV of tile i-1
    if (tid == 0 && i + S - 1 < n) issue(i + S - 1);
    if (i + 1 < n) fetch(i + 1, w0, w1);
    const int s = i % S;
    if (!mbar_wait(&full[s], (i / S) & 1, 0x400u + s)) break;
    const uint16_t* tV = reinterpret_cast<const uint16_t*>(sV + s * Cfg::kTileBytes);
    const float* tP = sP + (i & 1) * G * TILE;
    const int t0 = list[i0 + i] * TILE;
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
      const bool ok = t0 + r < p.T;   // P beyond T is not defined: the row is zero-filled, skip it
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pg = ok ? tP[g * TILE + r] : 0.f;
#pragma unroll
        for (int e = 0; e < DPL; ++e) acc[g][e] = fmaf(pg, vf[e], acc[g][e]);
      }
    }
    if (i + 1 < n) {
      float* nP = sP + ((i + 1) & 1) * G * TILE;
      nP[warp * TILE + 2 * lane] = w0;
      nP[warp * TILE + 2 * lane + 1] = w1;
    }
  }
  __syncthreads();
  float* red = reinterpret_cast<float*>(sV);
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
    const int64_t hq = hq0 + g;
    if (p.num_splits == 1) {
      reinterpret_cast<__nv_bfloat16*>(p.out)[hq * D + d] = __float2bfloat16(sum);
      if (p.out_f32) p.out_f32[hq * D + d] = sum;
    } else {
      p.part_acc[(hq * p.num_splits + split) * D + d] = sum;
    }
  }
}

template <int D>
__global__ void __launch_bounds__(D) sum_splits_kernel(const kvskip_params p) {
  const int64_t hq = blockIdx.x;
  const int d = threadIdx.x;
  float acc = 0.f;
  for (int s = 0; s < p.num_splits; ++s) acc += p.part_acc[(hq * p.num_splits + s) * D + d];
  reinterpret_cast<__nv_bfloat16*>(p.out)[hq * D + d] = __float2bfloat16(acc);
  if (p.out_f32) p.out_f32[hq * D + d] = acc;
}

// Streaming read through the copy engine: the ceiling of what the attention kernels' own loads can
// reach.  Every CTA pulls 32 KB pieces (piece c, c + grid, ...) with 1-D bulk copies into a ring of
// RB_STAGES stages; a consumer warp touches one word per lane of a piece and frees the stage.
// Nothing else is done with the data.  Bytes beyond the last whole piece are left out (the caller
// counts whole pieces).  Waits are bounded like everywhere else.
constexpr int RB_PIECE = 32768;
constexpr int RB_STAGES = 6;
constexpr int RB_SMEM = RB_STAGES * RB_PIECE + 2 * RB_STAGES * 8 + 128;
__global__ void __launch_bounds__(64) read_bulk_kernel(const unsigned char* __restrict__ x, int64_t pieces,
                                                       uint32_t* out) {
  extern __shared__ unsigned char rb_raw[];
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(rb_raw) + 127) & ~uintptr_t(127));
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + RB_STAGES * RB_PIECE);
  uint64_t* empty = full + RB_STAGES;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < RB_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  const int64_t first = blockIdx.x, step = gridDim.x;
  const int64_t n = first < pieces ? (pieces - first + step - 1) / step : 0;
  if (warp == 0) {
    if (lane == 0)
      for (int64_t i = 0; i < n; ++i) {
        const int s = static_cast<int>(i % RB_STAGES);
        if (i >= RB_STAGES && !mbar_wait(&empty[s], ((i / RB_STAGES) - 1) & 1, 0x600u + s)) break;
        mbar_expect_tx(&full[s], RB_PIECE);
        bulk_load_1d(ring + s * RB_PIECE, x + (first + i * step) * RB_PIECE, RB_PIECE, &full[s]);
      }
  } else {
    uint32_t fold = 0;
    for (int64_t i = 0; i < n; ++i) {
      const int s = static_cast<int>(i % RB_STAGES);
      if (!mbar_wait(&full[s], (i / RB_STAGES) & 1, 0x610u + s)) break;
      fold ^= *reinterpret_cast<const uint32_t*>(ring + s * RB_PIECE + lane * 1024);
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
    if (fold == 0x9e3779b9u) out[0] = fold;   // keeps the reads alive; practically never true
  }
}

// Streaming read: 16-byte loads, grid-stride, four independent loads in flight per thread.
__global__ void __launch_bounds__(256) read_kernel(const uint4* __restrict__ x, int64_t n16, uint32_t* out) {
  uint32_t fold = 0;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n16; i += 4 * stride) {
    uint4 a[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(a[u].x), "=r"(a[u].y), "=r"(a[u].z), "=r"(a[u].w)
                   : "l"(x + i + u * stride));
#pragma unroll
    for (int u = 0; u < 4; ++u) fold ^= a[u].x ^ a[u].y ^ a[u].z ^ a[u].w;
  }
  for (; i < n16; i += stride) {
    uint4 a;
    asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w)
                 : "l"(x + i));
    fold ^= a.x ^ a.y ^ a.z ^ a.w;
  }
  if (fold == 0x9e3779b9u) out[0] = fold;   // keeps the loads alive; practically never true
}

}  // namespace kvb
