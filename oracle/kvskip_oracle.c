/*
 * CPU restatement of kvskip's decode-attention hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker used by the tests, by the smoke run and by the CPU-baseline leg of
 * the benchmark.  The product (the CUDA library) never links, loads or calls it.
 *
 * Two families of functions:
 *   kvo_*_f64   exact-arithmetic semantics in double precision (what the answer should be);
 *               follows the reference's own fp64 checker bench/harness.py:99-131 and the kernel
 *               semantics of kernels/kvskip_kernel.cu (masked lists, -inf/0 on unread blocks,
 *               V-skip vote and renormalisation).
 *   kvo_*_f32   float restatement that keeps the reference kernels' operation ORDER (which
 *               partial sums are formed, in which order they are merged), so integer outputs
 *               (block lists, refresh decisions, stored sets, index latches) come out identical
 *               unless an approximate exp/log on the GPU lands across a threshold.
 *               Follows kernels/kvskip_kernel.cu:106-218,294-314 and
 *               kernels/kvskip_planner.cu:58-305.
 *
 * Parity pin: every function here is checked against golden vectors produced by importing the
 * reference's Python path (bench/harness.py, kernels/kvskip.py selectors, src/kvskip_attn.py
 * refresh_pre_step, src/lab.py index_steps) on CPU; see tests/golden/make_golden.py.
 *
 * bf16 tensors travel as uint16_t bit patterns.  All strides are in ELEMENTS.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define KVO_BLOCK 64
#define KVO_LN2 0.6931471805599453f
#define KVO_LOG2E 1.4426950408889634f

static inline float bf16f(uint16_t b) {
  union { uint32_t u; float f; } c;
  c.u = ((uint32_t)b) << 16;
  return c.f;
}

static inline uint16_t f2bf16(float f) { /* round to nearest even, as __float2bfloat16 */
  union { uint32_t u; float f; } c;
  c.f = f;
  if ((c.u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((c.u >> 16) | 0x40);
  uint32_t r = ((c.u >> 16) & 1u) + 0x7fffu;
  return (uint16_t)((c.u + r) >> 16);
}

int kvo_version(void) { return 3; }

/* Threads of the parallel loops from now on (a launcher may have exported OMP_NUM_THREADS=1). */
void kvo_set_num_threads(int n) {
#ifdef _OPENMP
  extern void omp_set_num_threads(int);
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int kvo_num_threads(void) {
#ifdef _OPENMP
  extern int omp_get_max_threads(void);
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void kvo_f32_to_bf16(const float* x, uint16_t* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) y[i] = f2bf16(x[i]);
}

/* ------------------------------------------------------------------------------------------
 * Attention, double precision.
 *
 * q [B,Hq,D] (q_sb, q_sh); k, v [B,Hkv,T,D] (sb, sh, st), D contiguous.
 * block_idx/block_cnt NULL -> every block; else per (b, kv head) the first block_cnt entries of
 * block_idx[b,h,:] are the blocks read (kernels/kvskip_kernel.cu:91-101,120).
 * Outputs (any may be NULL): out [B,Hq,D], lse [B,Hq] (natural log; -inf if nothing read),
 * blk_max / blk_sum [B,Hq,nb]: max score (scale applied) and sum exp(s - max) of each block that
 * was read, -inf / 0 elsewhere (kvskip_kernel.cu:203-211, kvskip_ext.cpp:51-54).
 * Tokens >= T of the last block score -inf (kvskip_kernel.cu:183).
 * ---------------------------------------------------------------------------------------- */
void kvo_decode_f64(const uint16_t* q, int64_t q_sb, int64_t q_sh,
                    const uint16_t* k, int64_t k_sb, int64_t k_sh, int64_t k_st,
                    const uint16_t* v, int64_t v_sb, int64_t v_sh, int64_t v_st,
                    int B, int Hq, int Hkv, int T, int D, double scale,
                    const int32_t* block_idx, const int32_t* block_cnt, int max_blocks,
                    double* out, double* lse, double* blk_max, double* blk_sum) {
  const int G = Hq / Hkv;
  const int nb = (T + KVO_BLOCK - 1) / KVO_BLOCK;
  if (blk_max) for (int64_t i = 0; i < (int64_t)B * Hq * nb; ++i) blk_max[i] = -INFINITY;
  if (blk_sum) for (int64_t i = 0; i < (int64_t)B * Hq * nb; ++i) blk_sum[i] = 0.0;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int b = 0; b < B; ++b)
    for (int hq = 0; hq < Hq; ++hq) {
      const int h = hq / G;
      const uint16_t* qp = q + b * q_sb + hq * q_sh;
      const uint16_t* kb = k + b * k_sb + h * k_sh;
      const uint16_t* vb = v + b * v_sb + h * v_sh;
      const int n_items = block_idx ? block_cnt[b * Hkv + h] : nb;
      const int32_t* list = block_idx ? block_idx + (int64_t)(b * Hkv + h) * max_blocks : NULL;
      double* s = (double*)malloc(sizeof(double) * KVO_BLOCK * (size_t)(n_items > 0 ? n_items : 1));
      double qd[256];
      for (int d = 0; d < D; ++d) qd[d] = (double)bf16f(qp[d]);
      double m = -INFINITY;
      for (int i = 0; i < n_items; ++i) {
        const int blk = list ? list[i] : i;
        double bm = -INFINITY;
        for (int r = 0; r < KVO_BLOCK; ++r) {
          const int t = blk * KVO_BLOCK + r;
          double a = -INFINITY;
          if (t < T) {
            const uint16_t* kr = kb + (int64_t)t * k_st;
            a = 0.0;
            for (int d = 0; d < D; ++d) a += qd[d] * (double)bf16f(kr[d]);
            a *= scale;
          }
          s[i * KVO_BLOCK + r] = a;
          if (a > bm) bm = a;
        }
        if (bm > m) m = bm;
        if (blk_max || blk_sum) {
          double bs = 0.0;
          for (int r = 0; r < KVO_BLOCK; ++r)
            if (s[i * KVO_BLOCK + r] != -INFINITY) bs += exp(s[i * KVO_BLOCK + r] - bm);
          const int64_t o = ((int64_t)b * Hq + hq) * nb + blk;
          if (blk_max) blk_max[o] = bm;
          if (blk_sum) blk_sum[o] = bs;
        }
      }
      double l = 0.0;
      double acc[256];
      for (int d = 0; d < D; ++d) acc[d] = 0.0;
      if (m != -INFINITY) {
        for (int i = 0; i < n_items; ++i) {
          const int blk = list ? list[i] : i;
          for (int r = 0; r < KVO_BLOCK; ++r) {
            const double a = s[i * KVO_BLOCK + r];
            if (a == -INFINITY) continue;
            const double p = exp(a - m);
            l += p;
            if (out) {
              const uint16_t* vr = vb + (int64_t)(blk * KVO_BLOCK + r) * v_st;
              for (int d = 0; d < D; ++d) acc[d] += p * (double)bf16f(vr[d]);
            }
          }
        }
      }
      const int64_t o = (int64_t)b * Hq + hq;
      if (out) for (int d = 0; d < D; ++d) out[o * D + d] = l > 0.0 ? acc[d] / l : 0.0;
      if (lse) lse[o] = l > 0.0 ? m + log(l) : -INFINITY;
      free(s);
    }
}

/* ------------------------------------------------------------------------------------------
 * Single-pass V-skip, double precision (kernels/kvskip_kernel.cu:562-661).
 * Block b of a KV head contributes (to the sum and to the normaliser) iff b == 0, b >= nb-local,
 * or for some query head g of the group  lse_b(g) - lse0(g) >= log(tau), where lse0 is lse_prev
 * (given, natural log) or the log-sum-exp of block 0.  Outputs: out, lse over contributing
 * blocks, vcount [B,Hkv] = number of contributing blocks, kept [B,Hkv,nb] (u8, optional),
 * margin [B,Hkv,nb] (optional): max_g (lse_b - lse0) - log(tau), the distance of the vote from
 * its threshold (for reporting borderline votes).
 * ---------------------------------------------------------------------------------------- */
void kvo_vskip1_f64(const uint16_t* q, int64_t q_sb, int64_t q_sh,
                    const uint16_t* k, int64_t k_sb, int64_t k_sh, int64_t k_st,
                    const uint16_t* v, int64_t v_sb, int64_t v_sh, int64_t v_st,
                    int B, int Hq, int Hkv, int T, int D, double scale, double tau, int local,
                    const float* lse_prev, double* out, double* lse, int32_t* vcount,
                    uint8_t* kept, double* margin) {
  const int G = Hq / Hkv;
  const int nb = (T + KVO_BLOCK - 1) / KVO_BLOCK;
  const double log_tau = log(tau);
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < Hkv; ++h) {
      const uint16_t* kb = k + b * k_sb + h * k_sh;
      const uint16_t* vb = v + b * v_sb + h * v_sh;
      double* s = (double*)malloc(sizeof(double) * (size_t)G * nb * KVO_BLOCK);
      double* lb = (double*)malloc(sizeof(double) * (size_t)G * nb);
      for (int g = 0; g < G; ++g) {
        const uint16_t* qp = q + b * q_sb + (h * G + g) * q_sh;
        for (int blk = 0; blk < nb; ++blk) {
          double bm = -INFINITY;
          for (int r = 0; r < KVO_BLOCK; ++r) {
            const int t = blk * KVO_BLOCK + r;
            double a = -INFINITY;
            if (t < T) {
              const uint16_t* kr = kb + (int64_t)t * k_st;
              a = 0.0;
              for (int d = 0; d < D; ++d) a += (double)bf16f(qp[d]) * (double)bf16f(kr[d]);
              a *= scale;
            }
            s[((int64_t)g * nb + blk) * KVO_BLOCK + r] = a;
            if (a > bm) bm = a;
          }
          double bs = 0.0;
          for (int r = 0; r < KVO_BLOCK; ++r) {
            const double a = s[((int64_t)g * nb + blk) * KVO_BLOCK + r];
            if (a != -INFINITY) bs += exp(a - bm);
          }
          lb[g * nb + blk] = bm + log(bs);
        }
      }
      int cnt = 0;
      uint8_t* need = (uint8_t*)malloc((size_t)nb);
      for (int blk = 0; blk < nb; ++blk) {
        double best = -INFINITY;
        for (int g = 0; g < G; ++g) {
          const double l0 = lse_prev ? (double)lse_prev[(int64_t)b * Hq + h * G + g] : lb[g * nb];
          const double dlt = lb[g * nb + blk] - l0;
          if (dlt > best) best = dlt;
        }
        need[blk] = (blk == 0 || blk >= nb - local || best >= log_tau) ? 1 : 0;
        cnt += need[blk];
        if (kept) kept[((int64_t)b * Hkv + h) * nb + blk] = need[blk];
        if (margin) margin[((int64_t)b * Hkv + h) * nb + blk] = best - log_tau;
      }
      if (vcount) vcount[b * Hkv + h] = cnt;
      for (int g = 0; g < G; ++g) {
        double m = -INFINITY, l = 0.0, acc[256];
        for (int d = 0; d < D; ++d) acc[d] = 0.0;
        for (int blk = 0; blk < nb; ++blk)
          if (need[blk])
            for (int r = 0; r < KVO_BLOCK; ++r) {
              const double a = s[((int64_t)g * nb + blk) * KVO_BLOCK + r];
              if (a > m) m = a;
            }
        if (m != -INFINITY)
          for (int blk = 0; blk < nb; ++blk) {
            if (!need[blk]) continue;
            for (int r = 0; r < KVO_BLOCK; ++r) {
              const double a = s[((int64_t)g * nb + blk) * KVO_BLOCK + r];
              if (a == -INFINITY) continue;
              const double p = exp(a - m);
              l += p;
              const uint16_t* vr = vb + (int64_t)(blk * KVO_BLOCK + r) * v_st;
              for (int d = 0; d < D; ++d) acc[d] += p * (double)bf16f(vr[d]);
            }
          }
        const int64_t o = (int64_t)b * Hq + h * G + g;
        if (out) for (int d = 0; d < D; ++d) out[o * D + d] = l > 0.0 ? acc[d] / l : 0.0;
        if (lse) lse[o] = l > 0.0 ? m + log(l) : -INFINITY;
      }
      free(need);
      free(lb);
      free(s);
    }
}

/* ------------------------------------------------------------------------------------------
 * Two-pass V-skip, pass 2 (kernels/kvskip_kernel.cu:316-421): out = sum over listed blocks of
 * blk_scale[b,h,blk,g] * P[b,hq,t] * V[b,h,t,:], P given in fp16 bit patterns.
 * ---------------------------------------------------------------------------------------- */
static inline double half_bits_to_double(uint16_t hbits) {
  const int sgn = hbits >> 15, e = (hbits >> 10) & 31, f = hbits & 1023;
  double x;
  if (e == 0) x = ldexp((double)f, -24);
  else if (e == 31) x = f ? NAN : INFINITY;
  else x = ldexp((double)(f | 1024), e - 25);
  return sgn ? -x : x;
}

void kvo_pv_f64(const uint16_t* P, const uint16_t* v, int64_t v_sb, int64_t v_sh, int64_t v_st,
                const float* blk_scale, const int32_t* block_idx, const int32_t* block_cnt,
                int max_blocks, int B, int Hq, int Hkv, int T, int D, double* out) {
  const int G = Hq / Hkv;
  const int nb = (T + KVO_BLOCK - 1) / KVO_BLOCK;
  const int64_t t_pad = (int64_t)nb * KVO_BLOCK;
#pragma omp parallel for collapse(2)
  for (int b = 0; b < B; ++b)
    for (int hq = 0; hq < Hq; ++hq) {
      const int h = hq / G, g = hq % G;
      const uint16_t* vb = v + b * v_sb + h * v_sh;
      const int32_t* list = block_idx + (int64_t)(b * Hkv + h) * max_blocks;
      double acc[256];
      for (int d = 0; d < D; ++d) acc[d] = 0.0;
      for (int i = 0; i < block_cnt[b * Hkv + h]; ++i) {
        const int blk = list[i];
        const double f = (double)blk_scale[(((int64_t)b * Hkv + h) * nb + blk) * G + g];
        for (int r = 0; r < KVO_BLOCK; ++r) {
          const int t = blk * KVO_BLOCK + r;
          if (t >= T) break;
          const double p = f * half_bits_to_double(P[((int64_t)b * Hq + hq) * t_pad + t]);
          const uint16_t* vr = vb + (int64_t)t * v_st;
          for (int d = 0; d < D; ++d) acc[d] += p * (double)bf16f(vr[d]);
        }
      }
      for (int d = 0; d < D; ++d) out[((int64_t)b * Hq + hq) * D + d] = acc[d];
    }
}

/* ------------------------------------------------------------------------------------------
 * Split merge (kernels/kvskip_kernel.cu:294-314), float, kernel order: global max over splits,
 * then l and acc accumulated over s = 0..S-1 in that order; m is in log2 units.
 * part_acc [N,S,D], part_ml [N,S,2]; out [N,D] float, lse [N] natural log.
 * ---------------------------------------------------------------------------------------- */
void kvo_combine_f32(const float* part_acc, const float* part_ml, int64_t N, int S, int D,
                     float* out, float* lse) {
  for (int64_t n = 0; n < N; ++n) {
    const float* ml = part_ml + n * S * 2;
    float m = -INFINITY;
    for (int s = 0; s < S; ++s) m = fmaxf(m, ml[2 * s]);
    const float mu = (m == -INFINITY) ? 0.f : m;
    float l = 0.f;
    for (int s = 0; s < S; ++s) l = fmaf(ml[2 * s + 1], exp2f(ml[2 * s] - mu), l);
    for (int d = 0; d < D; ++d) {
      float acc = 0.f;
      for (int s = 0; s < S; ++s) acc = fmaf(part_acc[(n * S + s) * D + d], exp2f(ml[2 * s] - mu), acc);
      out[n * D + d] = l > 0.f ? acc / l : 0.f;
    }
    if (lse) lse[n] = l > 0.f ? (m + log2f(l)) * KVO_LN2 : -INFINITY;
  }
}

/* ------------------------------------------------------------------------------------------
 * Scores and block statistics in the kernels' float operation order
 * (kernels/kvskip_kernel.cu:106-118,158-218): q pre-multiplied by scale*log2(e) in float; a row's
 * dot product is eight fused-multiply-add chains (chain j covers dims 8j..8j+7 then 64+8j..64+8j+7
 * for D = 128) merged as ((p0+p4)+(p2+p6))+((p1+p5)+(p3+p7)); the block maximum is order free; the
 * block sum pairs token i with token i+32 and then folds the 32 pair sums as a butterfly
 * (distance 16, 8, 4, 2, 1).  blk_max is returned in natural-log units (max * ln 2).
 * Dense only; writes blk_max, blk_sum [B,Hq,nb] and (optional) scores2 [B,Hq,nb*64] in log2 units.
 * ---------------------------------------------------------------------------------------- */
static float butterfly32(float* x) {
  for (int o = 16; o > 0; o >>= 1) {
    float y[32];
    for (int i = 0; i < 32; ++i) y[i] = x[i] + x[i ^ o];
    memcpy(x, y, sizeof(y));
  }
  return x[0];
}

static float score_f32order(const float* qr, const uint16_t* kr, int D) {
  const int CH = D / 64;
  float p[8];
  for (int j = 0; j < 8; ++j) {
    float a = 0.f;
    for (int c = 0; c < CH; ++c)
      for (int e = 0; e < 8; ++e) a = fmaf(qr[c * 64 + 8 * j + e], bf16f(kr[c * 64 + 8 * j + e]), a);
    p[j] = a;
  }
  /* xor 4, then 2, then 1 */
  const float a0 = p[0] + p[4], a1 = p[1] + p[5], a2 = p[2] + p[6], a3 = p[3] + p[7];
  const float b0 = a0 + a2, b1 = a1 + a3;
  return b0 + b1;
}

void kvo_block_stats_f32(const uint16_t* q, int64_t q_sb, int64_t q_sh,
                         const uint16_t* k, int64_t k_sb, int64_t k_sh, int64_t k_st,
                         int B, int Hq, int Hkv, int T, int D, float scale,
                         float* blk_max, float* blk_sum, float* scores2) {
  const int G = Hq / Hkv;
  const int nb = (T + KVO_BLOCK - 1) / KVO_BLOCK;
  const float scale_log2 = (float)((double)scale * 1.4426950408889634);
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int b = 0; b < B; ++b)
    for (int hq = 0; hq < Hq; ++hq) {
      const int h = hq / G;
      const uint16_t* qp = q + b * q_sb + hq * q_sh;
      const uint16_t* kb = k + b * k_sb + h * k_sh;
      float qr[256];
      for (int d = 0; d < D; ++d) qr[d] = bf16f(qp[d]) * scale_log2;
      for (int blk = 0; blk < nb; ++blk) {
        float s[KVO_BLOCK];
        float mt = -INFINITY;
        for (int r = 0; r < KVO_BLOCK; ++r) {
          const int t = blk * KVO_BLOCK + r;
          s[r] = t < T ? score_f32order(qr, kb + (int64_t)t * k_st, D) : -INFINITY;
          mt = fmaxf(mt, s[r]);
          if (scores2) scores2[((int64_t)b * Hq + hq) * nb * KVO_BLOCK + t] = s[r];
        }
        const float mtu = (mt == -INFINITY) ? 0.f : mt;
        float e[32];
        for (int i = 0; i < 32; ++i) e[i] = exp2f(s[i] - mtu) + exp2f(s[i + 32] - mtu);
        const int64_t o = ((int64_t)b * Hq + hq) * nb + blk;
        blk_max[o] = mt * KVO_LN2;
        blk_sum[o] = butterfly32(e);
      }
    }
}

/* ------------------------------------------------------------------------------------------
 * Refresh planner, before the attention pass (kernels/kvskip_planner.cu:75-227), float,
 * kernel order.  One call handles every (b, kv head); G = 4, D = 128.
 * In place: csum (adds key T-1 when add_token), age.  Out: cs_now, est, trig, block_idx,
 * block_cnt.  Optional out dec_margin [B,Hkv]: decision value minus delta (how far the refresh
 * decision is from flipping; +inf when forced by age or flag, NaN for index-only heads).
 * ---------------------------------------------------------------------------------------- */
static inline int always_block(int blk, int nb, int local) { return blk == 0 || blk >= nb - local; }

static inline float clamped_logit(float x) {
  x = fminf(fmaxf(x, 1e-6f), 1.f - 1e-6f);
  return logf(x) - logf(1.f - x);
}

/* running log-sum-exp state (m, s): the sum is kept relative to the running maximum */
static inline void lse_fold(float* m, float* s, float e) {
  if (e == -INFINITY) return;
  if (e > *m) {
    *s = fmaf(*s, expf(*m - e), 1.f); /* the compiler fuses s*exp+1 on the GPU */
    *m = e;
  } else {
    *s += expf(e - *m);
  }
}

/* merge of 32 lane states the way a warp does it: max, then butterfly sum of rescaled sums */
static void warp_merge(const float* m, const float* s, float* M, float* S) {
  float mm = -INFINITY;
  for (int i = 0; i < 32; ++i) mm = fmaxf(mm, m[i]);
  float t[32];
  for (int i = 0; i < 32; ++i) t[i] = s[i] > 0.f ? s[i] * expf(m[i] - mm) : 0.f;
  *M = mm;
  *S = butterfly32(t);
}

void kvo_plan_f32(const uint16_t* q, int64_t q_sb, int64_t q_sh,
                  const uint16_t* k, int64_t k_sb, int64_t k_sh, int64_t k_st,
                  float* csum, const float* lse_ref, const float* cs_ref, const uint8_t* keep,
                  const float* lse_att, int32_t* age, const int32_t* flags, const uint8_t* idx,
                  const float* calib, float* est, int calib_on, int calib_kind, const uint8_t* aix,
                  float* cs_now, uint8_t* trig, int32_t* block_idx, int32_t* block_cnt,
                  int B, int Hq, int Hkv, int T, int NBC, int local, int max_age, int add_token,
                  float scale, float delta, float* dec_margin) {
  enum { PG = 4, PD = 128, PT = 128 };
  const int nb = (T + KVO_BLOCK - 1) / KVO_BLOCK;
  (void)Hq;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < Hkv; ++h) {
      const int64_t bh = (int64_t)b * Hkv + h;
      float* cs = csum + bh * NBC * PD;
      const uint8_t* kp = keep + bh * NBC;
      int32_t* bi = block_idx + bh * NBC;
      if (flags[h] & 2) { /* token-index head: index blocks + sink + newest, never refreshes */
        const uint8_t* ix = idx + (int64_t)b * NBC;
        int n = 0;
        for (int i = 0; i < nb; ++i)
          if (ix[i] || always_block(i, nb, local)) bi[n++] = i;
        block_cnt[bh] = n;
        trig[bh] = 0;
        if (dec_margin) dec_margin[bh] = NAN;
        continue;
      }
      const int uni = (flags[h] & 4) || (aix && aix[bh]);
      const uint8_t* ix = uni ? idx + (int64_t)b * NBC : NULL;
#define ATTENDED(blk) (kp[blk] || always_block((blk), nb, local) || (uni && ix[blk]))
      if (add_token) {
        const int t = T - 1;
        const uint16_t* kr = k + b * k_sb + h * k_sh + (int64_t)t * k_st;
        for (int d = 0; d < PD; ++d) cs[(int64_t)(t / KVO_BLOCK) * PD + d] += bf16f(kr[d]);
      }
      /* centroid scores: lane l owns dims 4l..4l+3; products merged left to right with fused
         multiply-adds, lanes merged by butterfly, then times 1/n */
      float* scs = (float*)malloc(sizeof(float) * PG * (size_t)nb);
      const int64_t row0 = ((int64_t)b * Hq + h * PG) * NBC;
      for (int g = 0; g < PG; ++g) {
        const uint16_t* qp = q + b * q_sb + (h * PG + g) * q_sh;
        float qv[PD];
        for (int d = 0; d < PD; ++d) qv[d] = bf16f(qp[d]) * scale;
        for (int blk = 0; blk < nb; ++blk) {
          const float* c = cs + (int64_t)blk * PD;
          const float inv_n = 1.f / (float)(blk == nb - 1 ? T - blk * KVO_BLOCK : KVO_BLOCK);
          float part[32];
          for (int l = 0; l < 32; ++l) {
            float a = qv[4 * l] * c[4 * l];
            a = fmaf(qv[4 * l + 1], c[4 * l + 1], a);
            a = fmaf(qv[4 * l + 2], c[4 * l + 2], a);
            a = fmaf(qv[4 * l + 3], c[4 * l + 3], a);
            part[l] = a;
          }
          const float val = butterfly32(part) * inv_n;
          scs[g * nb + blk] = val;
          cs_now[row0 + (int64_t)g * NBC + blk] = val;
        }
      }
      /* drift estimate: 128 virtual threads, thread t folds blocks t, t+128, ... */
      float miss = 0.f;
      for (int g = 0; g < PG; ++g) {
        float m[PT], s[PT];
        for (int t = 0; t < PT; ++t) {
          m[t] = -INFINITY;
          s[t] = 0.f;
          for (int blk = t; blk < nb; blk += PT) {
            if (ATTENDED(blk)) continue;
            const float e = lse_ref[row0 + (int64_t)g * NBC + blk] + scs[g * nb + blk] -
                            cs_ref[row0 + (int64_t)g * NBC + blk];
            lse_fold(&m[t], &s[t], e);
          }
        }
        float wM[4], wS[4];
        for (int w = 0; w < 4; ++w) warp_merge(m + 32 * w, s + 32 * w, &wM[w], &wS[w]);
        float M = -INFINITY, S = 0.f;
        for (int w = 0; w < 4; ++w)
          if (wS[w] > 0.f) M = fmaxf(M, wM[w]);
        for (int w = 0; w < 4; ++w)
          if (wS[w] > 0.f) S = fmaf(wS[w], expf(wM[w] - M), S);
        if (S > 0.f) {
          const float e = M + logf(S);
          miss = fmaxf(miss, 1.f / (1.f + expf(lse_att[(int64_t)b * Hq + h * PG + g] - e)));
        }
      }
      if (est) est[bh] = miss;
      float dec = miss;
      if (calib && calib_on)
        dec = calib_kind ? miss + calib[bh] : 1.f / (1.f + expf(-(clamped_logit(miss) + calib[bh])));
      const int a = age[bh] + 1;
      const int forced = a >= max_age || (flags[h] & 1);
      const int tr = dec > delta || forced;
      age[bh] = tr ? 0 : a;
      trig[bh] = (uint8_t)tr;
      if (dec_margin) dec_margin[bh] = forced ? INFINITY : dec - delta;
      if (tr) {
        for (int i = 0; i < nb; ++i) bi[i] = i;
        block_cnt[bh] = nb;
      } else {
        int n = 0;
        for (int i = 0; i < nb; ++i)
          if (ATTENDED(i)) bi[n++] = i;
        block_cnt[bh] = n;
      }
#undef ATTENDED
      free(scs);
    }
}

/* ------------------------------------------------------------------------------------------
 * Refresh planner, after the attention pass (kernels/kvskip_planner.cu:229-305), float, kernel
 * order: lane l of query head g owns blocks l, l+32, ...
 * In place: keep, lse_ref, cs_ref (refreshing heads), lse_att (all heads), calib, aix.
 * blk_max / blk_sum are [B,Hq,nb] (row stride nb), the state tensors [.,.,NBC].
 * Optional out topp_margin [B,Hq]: min(mass of the kept set - level, level - mass without the
 * lightest kept block): how close the top-p cut is to keeping one block more or fewer.
 * ---------------------------------------------------------------------------------------- */
void kvo_update_f32(const float* blk_max, const float* blk_sum, const uint8_t* trig,
                    const float* cs_now, uint8_t* keep, float* lse_ref, float* cs_ref,
                    float* lse_att, const int32_t* flags, const uint8_t* idx, const float* est,
                    float* calib, float calib_rate, int calib_free, int calib_kind, uint8_t* aix,
                    float aix_thr, int B, int Hq, int Hkv, int T, int NBC, int local, float level,
                    float* topp_margin) {
  enum { PG = 4 };
  const int nb = (T + KVO_BLOCK - 1) / KVO_BLOCK;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < Hkv; ++h) {
      const int64_t bh = (int64_t)b * Hkv + h;
      uint8_t* kp = keep + bh * NBC;
      const int tr = trig[bh];
      float* x = (float*)malloc(sizeof(float) * PG * (size_t)nb);
      uint8_t* skeep = (uint8_t*)calloc((size_t)nb + 1, 1);
      float real_g[PG] = {0.f, 0.f, 0.f, 0.f};
      const int uni = tr && calib && ((flags[h] & 4) || (aix && aix[bh]));
      const uint8_t* ix = uni ? idx + (int64_t)b * NBC : NULL;
      for (int g = 0; g < PG; ++g) {
        const int64_t hrow = (int64_t)b * Hq + h * PG + g;
        float* xg = x + (size_t)g * nb;
        float mx = -INFINITY;
        for (int i = 0; i < nb; ++i) {
          xg[i] = blk_max[hrow * nb + i] + logf(blk_sum[hrow * nb + i]);
          mx = fmaxf(mx, xg[i]);
        }
        if (tr && calib) { /* mass the old attended set missed: every block was read this step */
          float mi[32], si[32], mo[32], so[32];
          for (int l = 0; l < 32; ++l) {
            mi[l] = mo[l] = -INFINITY;
            si[l] = so[l] = 0.f;
            for (int i = l; i < nb; i += 32) {
              if (kp[i] || always_block(i, nb, local) || (uni && ix[i])) lse_fold(&mi[l], &si[l], xg[i]);
              else lse_fold(&mo[l], &so[l], xg[i]);
            }
          }
          float Mi, Si, Mo, So;
          warp_merge(mi, si, &Mi, &Si);
          warp_merge(mo, so, &Mo, &So);
          real_g[g] = So > 0.f ? 1.f / (1.f + expf((Mi + logf(Si)) - (Mo + logf(So)))) : 0.f;
        }
        if (tr) {
          float se[32];
          for (int l = 0; l < 32; ++l) {
            se[l] = 0.f;
            for (int i = l; i < nb; i += 32) se[l] += expf(xg[i] - mx);
          }
          const float lse = mx + logf(butterfly32(se));
          float lo = -80.f, hi = 0.f;
          for (int it = 0; it < 32; ++it) {
            const float mid = 0.5f * (lo + hi);
            float acc[32];
            for (int l = 0; l < 32; ++l) {
              acc[l] = 0.f;
              for (int i = l; i < nb; i += 32) {
                const float y = xg[i] - lse;
                if (y >= mid) acc[l] += expf(y);
              }
            }
            if (butterfly32(acc) >= level) lo = mid; else hi = mid;
          }
          /* how far the cut is from flipping: mass of the kept set above `level`, and `level` above
             the mass without the lightest kept block */
          double mass_in = 0.0, ymin = INFINITY;
          for (int i = 0; i < nb; ++i) {
            const float y = xg[i] - lse;
            if (y >= lo) {
              skeep[i] = 1;
              mass_in += exp((double)y);
              if (y < ymin) ymin = y;
            }
          }
          const float closest = (float)fmin(mass_in - (double)level, (double)level - (mass_in - exp(ymin)));
          if (topp_margin) topp_margin[hrow] = closest;
          for (int i = 0; i < NBC; ++i) {
            lse_ref[hrow * NBC + i] = i < nb ? xg[i] : -INFINITY;
            cs_ref[hrow * NBC + i] = i < nb ? cs_now[hrow * NBC + i] : 0.f;
          }
        } else if (topp_margin) {
          topp_margin[hrow] = INFINITY;
        }
      }
      if (tr && calib) {
        float real = 0.f;
        for (int g = 0; g < PG; ++g) real = fmaxf(real, real_g[g]);
        const float e = est[bh];
        const float resid = calib_kind ? real - e : clamped_logit(real) - clamped_logit(e);
        float c = calib_kind == 2 ? fmaxf((1.f - calib_rate) * calib[bh], resid)
                                  : (1.f - calib_rate) * calib[bh] + calib_rate * resid;
        if (!calib_free) c = fmaxf(c, 0.f);
        calib[bh] = c;
        if (aix && c > aix_thr) aix[bh] = 1;
      }
      if (tr)
        for (int i = 0; i < NBC; ++i) kp[i] = (uint8_t)(i < nb && (skeep[i] || always_block(i, nb, local)));
      for (int g = 0; g < PG; ++g) {
        const int64_t hrow = (int64_t)b * Hq + h * PG + g;
        const float* xg = x + (size_t)g * nb;
        float m2[32], s2[32];
        for (int l = 0; l < 32; ++l) {
          m2[l] = -INFINITY;
          s2[l] = 0.f;
          for (int i = l; i < nb; i += 32)
            if (kp[i] || always_block(i, nb, local)) lse_fold(&m2[l], &s2[l], xg[i]);
        }
        float M, S;
        warp_merge(m2, s2, &M, &S);
        lse_att[hrow] = M + logf(S);
      }
      free(skeep);
      free(x);
    }
}

/* ------------------------------------------------------------------------------------------
 * Token-index blocks of one decode step (src/lab.py:149-167 with bigram off,
 * src/run_free.py:103-112): ids [n, stride] token ids, the current token at position T-1.
 * A block is marked if it holds an earlier copy of the current token, or the position right
 * after such a copy.  out [n, out_stride] u8, entries >= ceil(T/64) are zeroed.
 * ---------------------------------------------------------------------------------------- */
void kvo_index_blocks(const int64_t* ids, int64_t stride, int n, int T, uint8_t* out, int out_stride) {
  for (int r = 0; r < n; ++r) {
    const int64_t* x = ids + r * stride;
    uint8_t* o = out + (int64_t)r * out_stride;
    memset(o, 0, (size_t)out_stride);
    const int64_t cur = x[T - 1];
    for (int t = 0; t < T - 1; ++t)
      if (x[t] == cur) {
        o[t / KVO_BLOCK] = 1;
        if (t + 1 < T) o[(t + 1) / KVO_BLOCK] = 1;
      }
  }
}

/* ------------------------------------------------------------------------------------------
 * Stored-set selection as the Python front end does it (kernels/kvskip.py:130-147, rule
 * "topp"): per query head the fewest blocks (by descending weight, stable) whose mass reaches
 * `level`, union over the group, plus sink and `local` newest blocks.  logw [B,Hq,nb] double.
 * ---------------------------------------------------------------------------------------- */
typedef struct { double w; int i; } kvo_wi;
static int cmp_desc(const void* a, const void* b) {
  const kvo_wi* x = (const kvo_wi*)a;
  const kvo_wi* y = (const kvo_wi*)b;
  if (x->w > y->w) return -1;
  if (x->w < y->w) return 1;
  return x->i - y->i;
}

void kvo_select_topp(const double* logw, int B, int Hq, int Hkv, int nb, double level, int local,
                     uint8_t* keep) {
  const int G = Hq / Hkv;
  memset(keep, 0, (size_t)B * Hkv * nb);
  for (int b = 0; b < B; ++b)
    for (int hq = 0; hq < Hq; ++hq) {
      const double* x = logw + ((int64_t)b * Hq + hq) * nb;
      uint8_t* kp = keep + ((int64_t)b * Hkv + hq / G) * nb;
      double mx = -INFINITY, z = 0.0;
      for (int i = 0; i < nb; ++i) if (x[i] > mx) mx = x[i];
      for (int i = 0; i < nb; ++i) z += exp(x[i] - mx);
      kvo_wi* w = (kvo_wi*)malloc(sizeof(kvo_wi) * (size_t)nb);
      for (int i = 0; i < nb; ++i) { w[i].w = exp(x[i] - mx) / z; w[i].i = i; }
      qsort(w, (size_t)nb, sizeof(kvo_wi), cmp_desc);
      double cum = 0.0;
      for (int j = 0; j < nb; ++j) {
        if (cum < level) kp[w[j].i] = 1;  /* mass before this block still short of level */
        cum += w[j].w;
      }
      free(w);
    }
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < Hkv; ++h) {
      uint8_t* kp = keep + ((int64_t)b * Hkv + h) * nb;
      kp[0] = 1;
      for (int i = nb - local; i < nb; ++i) if (i >= 0) kp[i] = 1;
    }
}
