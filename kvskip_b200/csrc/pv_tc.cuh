// Second pass of the two-pass V-skip on tensor cores (D = 128, G = 4): out = sum over the listed
// blocks of (P * block weight) V, P in fp16 from the statistics pass.
//
// What it computes is what format37/kvskip's pv_kernel computes (kernels/kvskip_kernel.cu:319-445:
// per listed block the fp16 weights of the 64 tokens times blk_scale[b, kv head, block, head],
// times the V rows, summed over blocks; partial sums per split added in ascending split order).
// The layout of the work is the one of decode_tc_kernel: a producer warp feeds a ring of V blocks
// with TMA, six consumer warps each own every sixth block, O^T = V^T W^T by mma.m16n8k16 with the
// tokens on the K axis.  The B operand (weights: k = token, n = head) is built straight from
// global memory -- a thread needs two adjacent tokens of one head, which is one half2 of P -- and
// split into bf16 high + low parts so the weights keep fp32-grade precision.  The sum over splits
// runs inside the kernel (last CTA of a head), as in the decode kernel.
#pragma once
#include "decode_tc.cuh"

namespace kvb {

using PvTcCfg = TcCfg<TC_CONSUMERS, false>;   // 12 stages of one V block (16 KB)

__global__ void __launch_bounds__(TC_THREADS, 1)
pv_tc_kernel(const kvskip_params p, const __grid_constant__ TmaMaps maps, int* __restrict__ split_done,
             const int* __restrict__ t_dev) {
  using Cfg = PvTcCfg;
  constexpr int G = 4, D = 128, NC = TC_CONSUMERS;
  constexpr int S = Cfg::kStages;

  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* ring = smem;                                              // [S] stages of V, 1024-byte aligned
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S * Cfg::kStageBytes + NC * 8 * 4);   // [S]
  uint64_t* empty = full + S;                                              // [S]

  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    tma_prefetch_desc(&maps.v);
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  pdl_wait_prior();          // P, the block weights and the list come from earlier work on the stream
  pdl_launch_dependents();

  const int T = t_dev ? max(1, min(*t_dev, p.T)) : p.T;   // device-resident length: p.T is its bound
  const int n_items = p.block_cnt[b * p.Hkv + h];
  const int32_t* list = p.block_idx + static_cast<int64_t>(b * p.Hkv + h) * p.max_blocks;
  const int per = (n_items + p.num_splits - 1) / p.num_splits;
  const int i0 = min(n_items, split * per);
  const int n = min(n_items, i0 + per) - i0;
  const int64_t hq0 = static_cast<int64_t>(b) * p.Hq + h * G;

  float acc[8][4];                        // O^T fragments: 8 tiles of 16 dims x 8 heads
#pragma unroll
  for (int mt = 0; mt < 8; ++mt)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[mt][c] = 0.f;

  if (warp == NC) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      BlockAhead<true> ahead;   // list entries eight blocks ahead of the stage they are needed for
      ahead.init(list + i0, nullptr, i0, n, b);
      for (int i = 0; i < n; ++i) {
        const int s = i % S;
        if (i >= S && !mbar_wait(&empty[s], ((i / S) - 1) & 1, 0x420u + s)) break;
        int blk_i, unused;
        ahead.next(i, blk_i, unused);
        const int t0 = blk_i * TILE;
        unsigned char* dst = ring + s * Cfg::kStageBytes;
        mbar_expect_tx(&full[s], Cfg::kStageBytes);
        tma_load_4d(dst, &maps.v, &full[s], 0, t0, h, b);
        tma_load_4d(dst + TC_HALF_BYTES, &maps.v, &full[s], 64, t0, h, b);
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const int lrow = lane & 7, lmat = lane >> 3;
    const int head = lane >> 2;            // column of the B operand; 4..7 are padding
    const __half* pin = reinterpret_cast<const __half*>(p.p_in) + (hq0 + (head & 3)) * p.t_pad;
    const float* scl = p.blk_scale + (static_cast<int64_t>(b) * p.Hkv + h) * p.nb * G + (head & 3);

    // A warp's blocks are a chain list entry -> (block weight, P of its 64 tokens) -> MMA.  Walked one
    // block at a time that is two memory round trips per block and warp, which bounded the kernel
    // (0.4 us per block and CTA whatever the bandwidth).  So the chain is pipelined: the list entry is
    // read two blocks ahead and the block's weight and P (eight half2 per thread) one block ahead,
    // while the current block is multiplied.
    struct Raw {
      float f;
      __half2 hh[4][2];
    };
    auto fetch = [&](Raw& r, const int blk) {
      r.f = head < G ? scl[static_cast<int64_t>(blk) * G] : 0.f;
#pragma unroll
      for (int kt = 0; kt < 4; ++kt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tok = kt * 16 + e * 8 + 2 * (lane & 3);          // first of this thread's two tokens
          r.hh[kt][e] = head < G ? *reinterpret_cast<const __half2*>(pin + blk * TILE + tok) : __half2{};
        }
    };
    const int last = i0 + n - 1;
    int blk = warp < n ? list[min(i0 + warp, last)] : 0;
    int blk_next = warp < n ? list[min(i0 + warp + NC, last)] : 0;
    Raw cur, nxt;
    if (warp < n) fetch(cur, blk);
    for (int i = warp; i < n; i += NC) {
      const int s = i % S;
      const int t0 = blk * TILE;
      const int blk_after = list[min(i0 + i + 2 * NC, last)];
      if (i + NC < n) fetch(nxt, blk_next);
      // weights of this block as B fragments (high and low bf16 parts)
      uint32_t bhi[4][2], blo[4][2];
      {
        const float f = cur.f;
#pragma unroll
        for (int kt = 0; kt < 4; ++kt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int tok = kt * 16 + e * 8 + 2 * (lane & 3);
            // P beyond T is not defined (the statistics pass never wrote it): those weights are zero
            const float w0 = (head < G && t0 + tok < T) ? __half2float(__low2half(cur.hh[kt][e])) * f : 0.f;
            const float w1 = (head < G && t0 + tok + 1 < T) ? __half2float(__high2half(cur.hh[kt][e])) * f : 0.f;
            const uint32_t hi = pack_bf16(w0, w1);
            bhi[kt][e] = hi;
            blo[kt][e] = pack_bf16(w0 - bf_lo(hi), w1 - bf_hi(hi));
          }
      }
      if (!mbar_wait(&full[s], (i / S) & 1, 0x430u + s)) break;
      const uint32_t vbase = smem_u32(ring + s * Cfg::kStageBytes);
      if (t_dev != nullptr && t0 + TILE > T) {
        // device-resident length: the map reaches past T, where the cache holds anything (their
        // weights are zero, but 0 x NaN is not): clear those rows of both halves
        unsigned char* vst = ring + s * Cfg::kStageBytes;
        for (int o = (T - t0) * 128 + lane * 16; o < TILE * 128; o += 32 * 16) {
          *reinterpret_cast<uint4*>(vst + o) = make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4*>(vst + TC_HALF_BYTES + o) = make_uint4(0u, 0u, 0u, 0u);
        }
        fence_proxy_async_smem();   // ordered before the next bulk load into this stage
        __syncwarp();
      }
#pragma unroll
      for (int kt = 0; kt < 4; ++kt) {
        const int tok = kt * 16 + (lmat >> 1) * 8 + lrow;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
          const int dchunk = mt * 2 + (lmat & 1);
          uint32_t a[4];
          ldsm_x4_t(a, vbase + (dchunk >> 3) * TC_HALF_BYTES + tok * 128 + (((dchunk & 7) ^ lrow) << 4));
          mma_bf16(acc[mt], a, bhi[kt][0], bhi[kt][1]);
          mma_bf16(acc[mt], a, blo[kt][0], blo[kt][1]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
      cur = nxt;
      blk = blk_next;
      blk_next = blk_after;
    }
  }
  __syncthreads();   // every block has been consumed: the ring is free for the sum over the warps

  float* red = reinterpret_cast<float*>(ring);   // [NC][G][D]
  if (warp < NC && (lane & 3) < 2) {
    const int head0 = 2 * (lane & 3);
#pragma unroll
    for (int mt = 0; mt < 8; ++mt)
#pragma unroll
      for (int c = 0; c < 4; ++c)
        red[(warp * G + head0 + (c & 1)) * D + mt * 16 + (lane >> 2) + (c >> 1) * 8] = acc[mt][c];
  }
  __syncthreads();
  for (int o = tid; o < G * D; o += TC_THREADS) {
    const int g = o / D, d = o % D;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < NC; ++w) sum += red[(w * G + g) * D + d];
    const int64_t hq = hq0 + g;
    if (p.num_splits == 1) {
      reinterpret_cast<__nv_bfloat16*>(p.out)[hq * D + d] = __float2bfloat16(sum);
      if (p.out_f32) p.out_f32[hq * D + d] = sum;
    } else {
      p.part_acc[(hq * p.num_splits + split) * D + d] = sum;
    }
  }

  // ---- sum over the splits by the last CTA of this (batch, kv head) to finish, ascending order
  if (p.num_splits > 1 && split_done != nullptr) {
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(&split_done[b * p.Hkv + h], 1) == p.num_splits - 1;
    __syncthreads();
    if (s_last) {
      __threadfence();
      for (int o = tid; o < G * D; o += TC_THREADS) {
        const int g = o / D, d = o % D;
        const int64_t hq = hq0 + g;
        float a = 0.f;
        for (int s2 = 0; s2 < p.num_splits; ++s2) a += __ldcg(p.part_acc + (hq * p.num_splits + s2) * D + d);
        reinterpret_cast<__nv_bfloat16*>(p.out)[hq * D + d] = __float2bfloat16(a);
        if (p.out_f32) p.out_f32[hq * D + d] = a;
      }
      if (tid == 0) split_done[b * p.Hkv + h] = 0;
    }
  }
}

}  // namespace kvb
