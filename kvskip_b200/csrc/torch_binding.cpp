// Thin PyTorch front of libkvskip_b200: tensors in, C-ABI parameter blocks out.
//
// Exposes the same six functions, argument names and defaults as the reference's extension
// module (format37/kvskip kernels/kvskip_ext.cpp:327-352) -- decode, vskip1, pv, plan, update,
// read_bw -- so callers written against it run unchanged, plus merge / index_blocks /
// device_status for the multi-GPU merge and the device-side token index.  All work happens in the
// C library; this file only checks arguments (same conditions and wording as the reference's
// checks, kvskip_ext.cpp:12-19,29-42,212-221,276-313), allocates outputs and scratch with the
// caching allocator, and launches on the current stream of the inputs' device.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime.h>
#include <torch/extension.h>

#include <cmath>
#include <limits>

#include "../../include/kvskip_b200.h"

namespace {

void* cur_stream() { return static_cast<void*>(at::cuda::getCurrentCUDAStream().stream()); }

void raise_on(int rc) {
  TORCH_CHECK(rc == KVSKIP_OK, kvskip_last_error());
}

void need_kv(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16, name, " must be a CUDA bf16 tensor");
  TORCH_CHECK(t.dim() == 4, name, " must be [B, Hkv, T, D]");
  TORCH_CHECK(t.stride(3) == 1, name, " must have a contiguous last dim");
  TORCH_CHECK(t.stride(2) % 8 == 0 && t.stride(1) % 8 == 0 && t.stride(0) % 8 == 0, name,
              " strides must be multiples of 8 elements (16-byte rows)");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, name, " must be 16-byte aligned");
}

void need_q(const at::Tensor& q) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && q.dim() == 3, "q must be CUDA bf16 [B, Hq, D]");
  TORCH_CHECK(q.stride(2) == 1 && q.stride(1) % 8 == 0 && q.stride(0) % 8 == 0, "q rows must be 16-byte aligned");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(q.data_ptr()) % 16 == 0, "q must be 16-byte aligned");
}

void need_f32(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous(), name, " must be contiguous CUDA fp32");
}

const uint16_t* u16(const at::Tensor& t) { return reinterpret_cast<const uint16_t*>(t.data_ptr()); }
uint16_t* u16m(at::Tensor& t) { return reinterpret_cast<uint16_t*>(t.data_ptr()); }

void fill_qkv(kvskip_params& p, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v) {
  p.q = u16(q);
  p.k = u16(k);
  p.v = u16(v);
  p.q_sb = q.stride(0); p.q_sh = q.stride(1);
  p.k_sb = k.stride(0); p.k_sh = k.stride(1); p.k_st = k.stride(2);
  p.v_sb = v.stride(0); p.v_sh = v.stride(1); p.v_st = v.stride(2);
  p.B = static_cast<int32_t>(q.size(0));
  p.Hq = static_cast<int32_t>(q.size(1));
  p.Hkv = static_cast<int32_t>(k.size(1));
  p.T = static_cast<int32_t>(k.size(2));
}

// Device-resident sequence length: a one-element int32 CUDA tensor, or nothing.
const int* tdev_ptr(const c10::optional<at::Tensor>& t_dev) {
  if (!t_dev.has_value()) return nullptr;
  TORCH_CHECK(t_dev->is_cuda() && t_dev->scalar_type() == at::kInt && t_dev->numel() == 1,
              "t_dev: one-element int32 CUDA tensor");
  return t_dev->data_ptr<int32_t>();
}

// Page table of a paged cache: contiguous int32 [B, max_pages]; the pools are [pages, Hkv, 64, D].
struct Paged {
  const int32_t* table = nullptr;
  int max_pages = 0, num_pages = 0;
};
Paged paged_args(const c10::optional<at::Tensor>& page_table, const at::Tensor& k, const at::Tensor* v, int64_t B,
                 int64_t seq_len) {
  Paged pg;
  if (!page_table.has_value()) return pg;
  const at::Tensor& t = *page_table;
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.dim() == 2 && t.is_contiguous() && t.size(0) == B,
              "page_table: contiguous int32 [B, max_pages]");
  TORCH_CHECK(seq_len >= 1 && t.size(1) >= (seq_len + KVSKIP_TILE - 1) / KVSKIP_TILE,
              "page_table: one entry per 64-token block of seq_len");
  TORCH_CHECK(k.size(2) == KVSKIP_TILE && (!v || (v->size(2) == KVSKIP_TILE && v->size(0) == k.size(0))),
              "paged cache: pools are [pages, Hkv, 64, D]");
  pg.table = t.data_ptr<int32_t>();
  pg.max_pages = static_cast<int>(t.size(1));
  pg.num_pages = static_cast<int>(k.size(0));
  return pg;
}

}  // namespace

// [out bf16 [B,Hq,D] (undefined without load_v), lse [B,Hq], blk_max, blk_sum ([B,Hq,nb] or
//  undefined), out_f32 or undefined, P fp16 [B,Hq,nb*64] or undefined]
namespace {
// peers of a sequence-sharded step: device addresses of every rank's buffer and flag array
struct XchgHost {
  std::vector<int64_t> buf_ptrs, flag_ptrs;
  int64_t rank = 0, seq = 0;
};
}  // namespace

std::vector<at::Tensor> decode_common(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double scale,
                                      const c10::optional<at::Tensor>& block_idx,
                                      const c10::optional<at::Tensor>& block_cnt, bool stats, bool load_v,
                                      int64_t num_splits, int64_t stages, bool want_f32, bool write_p,
                                      const c10::optional<at::Tensor>& t_dev,
                                      const c10::optional<at::Tensor>& page_table, int64_t seq_len,
                                      const XchgHost* xh) {
  need_q(q);
  need_kv(k, "k");
  need_kv(v, "v");
  const c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), Hq = q.size(1), D = q.size(2), Hkv = k.size(1);
  const Paged pg = paged_args(page_table, k, &v, B, seq_len);
  const int64_t T = pg.table ? seq_len : k.size(2);
  TORCH_CHECK((pg.table || (k.size(0) == B && v.size(0) == B)) && k.size(3) == D && v.size(3) == D &&
                  v.size(1) == Hkv && v.size(2) == k.size(2), "shape mismatch between q, k, v");
  TORCH_CHECK(Hq % Hkv == 0, "Hq must be a multiple of Hkv");
  TORCH_CHECK(num_splits >= 1, "num_splits >= 1");
  TORCH_CHECK(load_v || stats, "load_v=false only makes sense with stats=true");
  TORCH_CHECK(!write_p || stats, "write_p needs stats=true");
  const bool masked = block_idx.has_value();
  const int64_t nb = (T + KVSKIP_TILE - 1) / KVSKIP_TILE;

  const auto f32 = q.options().dtype(at::kFloat);
  at::Tensor out, out32, bmax, bsum, pbuf, part_acc, part_ml;
  if (load_v) out = at::empty({B, Hq, D}, q.options());
  if (load_v && want_f32) out32 = at::empty({B, Hq, D}, f32);
  at::Tensor lse = at::empty({B, Hq}, f32);
  if (stats) {   // the kernels write every entry themselves (-inf / 0 on blocks a list skips)
    bmax = at::empty({B, Hq, nb}, f32);
    bsum = at::empty({B, Hq, nb}, f32);
  }
  if (write_p) pbuf = at::empty({B, Hq, nb * KVSKIP_TILE}, q.options().dtype(at::kHalf));
  if (num_splits > 1) {
    part_acc = at::empty({B, Hq, num_splits, D}, f32);
    part_ml = at::empty({B, Hq, num_splits, 2}, f32);
  }

  kvskip_params p{};
  fill_qkv(p, q, k, v);
  p.T = static_cast<int32_t>(T);
  p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
  if (masked) {
    TORCH_CHECK(block_cnt.has_value(), "block_cnt is required with block_idx");
    const at::Tensor& bi = *block_idx;
    const at::Tensor& bc = *block_cnt;
    TORCH_CHECK(bi.is_cuda() && bi.scalar_type() == at::kInt && bi.dim() == 3 && bi.is_contiguous() &&
                    bi.size(0) == B && bi.size(1) == Hkv,
                "block_idx must be contiguous int32 [B, Hkv, max_blocks]");
    TORCH_CHECK(bc.is_cuda() && bc.scalar_type() == at::kInt && bc.is_contiguous() && bc.numel() == B * Hkv,
                "block_cnt must be contiguous int32 [B, Hkv]");
    p.block_idx = bi.data_ptr<int32_t>();
    p.block_cnt = bc.data_ptr<int32_t>();
    p.max_blocks = static_cast<int32_t>(bi.size(2));
  }
  p.num_splits = static_cast<int32_t>(num_splits);
  if (num_splits > 1) {
    p.part_acc = part_acc.data_ptr<float>();
    p.part_ml = part_ml.data_ptr<float>();
  }
  if (load_v) p.out = u16m(out);
  if (out32.defined()) p.out_f32 = out32.data_ptr<float>();
  p.lse = lse.data_ptr<float>();
  if (stats) {
    p.blk_max = bmax.data_ptr<float>();
    p.blk_sum = bsum.data_ptr<float>();
  }
  p.nb = static_cast<int32_t>(nb);
  p.t_pad = nb * KVSKIP_TILE;
  if (write_p) p.p_out = u16m(pbuf);
  if (xh) {
    const int64_t R = static_cast<int64_t>(xh->buf_ptrs.size());
    TORCH_CHECK(R >= 1 && R <= 8 && xh->flag_ptrs.size() == xh->buf_ptrs.size() && !pg.table && !t_dev.has_value() &&
                    load_v, "decode_exchange arguments");
    float* bufs[8];
    unsigned int* flags[8];
    for (int64_t r = 0; r < R; ++r) {
      bufs[r] = reinterpret_cast<float*>(xh->buf_ptrs[r]);
      flags[r] = reinterpret_cast<unsigned int*>(xh->flag_ptrs[r]);
    }
    raise_on(kvskip_launch_decode_xchg(&p, static_cast<int>(D), static_cast<int>(Hq / Hkv), static_cast<int>(stages),
                                       masked, stats, bufs, flags, static_cast<int>(xh->rank), static_cast<int>(R),
                                       static_cast<unsigned int>(xh->seq), cur_stream()));
  } else if (pg.table)
    raise_on(kvskip_launch_decode_paged(&p, static_cast<int>(D), static_cast<int>(Hq / Hkv), static_cast<int>(stages),
                                        masked, stats, load_v, pg.table, pg.max_pages, pg.num_pages, tdev_ptr(t_dev),
                                        cur_stream()));
  else if (const int* td = tdev_ptr(t_dev))
    raise_on(kvskip_launch_decode_dyn(&p, static_cast<int>(D), static_cast<int>(Hq / Hkv), static_cast<int>(stages),
                                      masked, stats, load_v, td, cur_stream()));
  else
    raise_on(kvskip_launch_decode(&p, static_cast<int>(D), static_cast<int>(Hq / Hkv), static_cast<int>(stages),
                                  masked, stats, load_v, cur_stream()));
  return {out, lse, bmax, bsum, out32, pbuf};
}

std::vector<at::Tensor> decode(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double scale,
                               const c10::optional<at::Tensor>& block_idx,
                               const c10::optional<at::Tensor>& block_cnt, bool stats, bool load_v,
                               int64_t num_splits, int64_t stages, bool want_f32, bool write_p,
                               const c10::optional<at::Tensor>& t_dev, const c10::optional<at::Tensor>& page_table,
                               int64_t seq_len) {
  return decode_common(q, k, v, scale, block_idx, block_cnt, stats, load_v, num_splits, stages, want_f32, write_p, t_dev,
                       page_table, seq_len, nullptr);
}

// Sequence shards: attention over this rank's blocks, exchange with the peers and merge, one kernel.
// Returns what decode returns, for the whole sequence.
std::vector<at::Tensor> decode_exchange(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double scale,
                                        const c10::optional<at::Tensor>& block_idx,
                                        const c10::optional<at::Tensor>& block_cnt, int64_t num_splits,
                                        const std::vector<int64_t>& buf_ptrs, const std::vector<int64_t>& flag_ptrs,
                                        int64_t rank, int64_t seq) {
  XchgHost xh;
  xh.buf_ptrs = buf_ptrs;
  xh.flag_ptrs = flag_ptrs;
  xh.rank = rank;
  xh.seq = seq;
  return decode_common(q, k, v, scale, block_idx, block_cnt, false, true, num_splits, 2, true, false, c10::nullopt,
                       c10::nullopt, 0, &xh);
}

// Two-pass V-skip, second pass: [out bf16, out_f32 or undefined]
std::vector<at::Tensor> pv(const at::Tensor& P, const at::Tensor& v, const at::Tensor& blk_scale,
                           const at::Tensor& block_idx, const at::Tensor& block_cnt, int64_t num_splits,
                           bool want_f32, const c10::optional<at::Tensor>& t_dev) {
  need_kv(v, "v");
  TORCH_CHECK(P.is_cuda() && P.scalar_type() == at::kHalf && P.dim() == 3 && P.is_contiguous(), "P: fp16 [B, Hq, t_pad]");
  TORCH_CHECK(blk_scale.is_cuda() && blk_scale.scalar_type() == at::kFloat && blk_scale.dim() == 4 &&
                  blk_scale.is_contiguous(), "blk_scale: contiguous fp32 [B, Hkv, nb, G]");
  const c10::cuda::CUDAGuard guard(v.device());
  const int64_t B = v.size(0), Hkv = v.size(1), T = v.size(2), D = v.size(3);
  const int64_t Hq = P.size(1), G = Hq / Hkv;
  const int64_t nb = (T + KVSKIP_TILE - 1) / KVSKIP_TILE;
  TORCH_CHECK(num_splits >= 1, "num_splits >= 1");
  TORCH_CHECK(P.size(0) == B && P.size(2) == nb * KVSKIP_TILE, "P shape");
  TORCH_CHECK(blk_scale.size(0) == B && blk_scale.size(1) == Hkv && blk_scale.size(2) == nb && blk_scale.size(3) == G,
              "blk_scale shape");
  TORCH_CHECK(block_idx.is_cuda() && block_idx.scalar_type() == at::kInt && block_idx.is_contiguous() &&
                  block_idx.dim() == 3 && block_idx.size(0) == B && block_idx.size(1) == Hkv, "block_idx");
  TORCH_CHECK(block_cnt.is_cuda() && block_cnt.scalar_type() == at::kInt && block_cnt.is_contiguous() &&
                  block_cnt.numel() == B * Hkv, "block_cnt");
  const auto f32 = v.options().dtype(at::kFloat);
  at::Tensor out = at::empty({B, Hq, D}, v.options());
  at::Tensor out32, part_acc;
  if (want_f32) out32 = at::empty({B, Hq, D}, f32);
  if (num_splits > 1) part_acc = at::empty({B, Hq, num_splits, D}, f32);
  kvskip_params p{};
  p.v = u16(v);
  p.v_sb = v.stride(0); p.v_sh = v.stride(1); p.v_st = v.stride(2);
  p.B = static_cast<int32_t>(B); p.Hq = static_cast<int32_t>(Hq); p.Hkv = static_cast<int32_t>(Hkv);
  p.T = static_cast<int32_t>(T);
  p.block_idx = block_idx.data_ptr<int32_t>();
  p.block_cnt = block_cnt.data_ptr<int32_t>();
  p.max_blocks = static_cast<int32_t>(block_idx.size(2));
  p.num_splits = static_cast<int32_t>(num_splits);
  if (num_splits > 1) p.part_acc = part_acc.data_ptr<float>();
  p.out = u16m(out);
  if (want_f32) p.out_f32 = out32.data_ptr<float>();
  p.nb = static_cast<int32_t>(nb);
  p.t_pad = nb * KVSKIP_TILE;
  p.p_in = u16(P);
  p.blk_scale = blk_scale.data_ptr<float>();
  if (const int* td = tdev_ptr(t_dev))
    raise_on(kvskip_launch_pv_dyn(&p, static_cast<int>(D), static_cast<int>(G), td, cur_stream()));
  else
    raise_on(kvskip_launch_pv(&p, static_cast<int>(D), static_cast<int>(G), cur_stream()));
  return {out, out32};
}

// Single-pass V-skip: [out bf16, lse, out_f32 or undefined, vcount int32 [B,Hkv] or undefined]
std::vector<at::Tensor> vskip1(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double scale,
                               double tau, int64_t local, int64_t num_splits, bool want_f32, bool count,
                               const c10::optional<at::Tensor>& lse_prev,
                               const c10::optional<at::Tensor>& page_table, int64_t seq_len,
                               const c10::optional<at::Tensor>& t_dev) {
  need_q(q);
  need_kv(k, "k");
  need_kv(v, "v");
  TORCH_CHECK(!(t_dev.has_value() && page_table.has_value()), "vskip1: a device-resident length or a paged cache, not both");
  TORCH_CHECK(tau > 0.0 && local >= 0 && num_splits >= 1, "tau > 0, local >= 0, num_splits >= 1");
  const c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), Hq = q.size(1), D = q.size(2), Hkv = k.size(1);
  const Paged pg = paged_args(page_table, k, &v, B, seq_len);
  const int64_t T = pg.table ? seq_len : k.size(2);
  TORCH_CHECK((pg.table || (k.size(0) == B && v.size(0) == B)) && k.size(3) == D && v.size(3) == D &&
                  v.size(1) == Hkv && v.size(2) == k.size(2), "shape mismatch between q, k, v");
  TORCH_CHECK(Hq % Hkv == 0, "Hq must be a multiple of Hkv");
  const auto f32 = q.options().dtype(at::kFloat);
  at::Tensor out = at::empty({B, Hq, D}, q.options());
  at::Tensor lse = at::empty({B, Hq}, f32);
  at::Tensor out32, vcount, part_acc, part_ml;
  if (want_f32) out32 = at::empty({B, Hq, D}, f32);
  if (count) vcount = at::zeros({B, Hkv}, q.options().dtype(at::kInt));
  if (num_splits > 1) {
    part_acc = at::empty({B, Hq, num_splits, D}, f32);
    part_ml = at::empty({B, Hq, num_splits, 2}, f32);
  }
  kvskip_params p{};
  fill_qkv(p, q, k, v);
  p.T = static_cast<int32_t>(T);
  p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
  p.num_splits = static_cast<int32_t>(num_splits);
  if (num_splits > 1) {
    p.part_acc = part_acc.data_ptr<float>();
    p.part_ml = part_ml.data_ptr<float>();
  }
  p.out = u16m(out);
  if (want_f32) p.out_f32 = out32.data_ptr<float>();
  p.lse = lse.data_ptr<float>();
  p.nb = static_cast<int32_t>((T + KVSKIP_TILE - 1) / KVSKIP_TILE);
  p.log2_tau = static_cast<float>(std::log2(tau));
  p.local = static_cast<int32_t>(local);
  if (count) p.vcount = vcount.data_ptr<int32_t>();
  if (lse_prev.has_value()) {
    TORCH_CHECK(lse_prev->is_cuda() && lse_prev->scalar_type() == at::kFloat && lse_prev->is_contiguous() &&
                    lse_prev->numel() == B * Hq, "lse_prev: contiguous fp32 [B, Hq]");
    p.lse_prev = lse_prev->data_ptr<float>();
  }
  if (pg.table)
    raise_on(kvskip_launch_vskip1_paged(&p, static_cast<int>(D), static_cast<int>(Hq / Hkv), pg.table, pg.max_pages,
                                        pg.num_pages, cur_stream()));
  else if (const int* td = tdev_ptr(t_dev))
    raise_on(kvskip_launch_vskip1_dyn(&p, static_cast<int>(D), static_cast<int>(Hq / Hkv), td, cur_stream()));
  else
    raise_on(kvskip_launch_vskip1(&p, static_cast<int>(D), static_cast<int>(Hq / Hkv), cur_stream()));
  return {out, lse, out32, vcount};
}

void plan(const at::Tensor& q, const at::Tensor& k, at::Tensor& csum, const at::Tensor& lse_ref,
          const at::Tensor& cs_ref, const at::Tensor& keep, const at::Tensor& lse_att, at::Tensor& age,
          const at::Tensor& flags, at::Tensor& cs_now, at::Tensor& trig, at::Tensor& block_idx,
          at::Tensor& block_cnt, double scale, double delta, int64_t max_age, int64_t local, bool add_token,
          const c10::optional<at::Tensor>& idx, const c10::optional<at::Tensor>& calib,
          const c10::optional<at::Tensor>& est, bool calib_on, int64_t calib_kind,
          const c10::optional<at::Tensor>& aix, const c10::optional<at::Tensor>& t_dev,
          const c10::optional<at::Tensor>& page_table, int64_t seq_len) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && q.dim() == 3 && q.stride(2) == 1, "q: CUDA bf16 [B, Hq, D]");
  need_kv(k, "k");
  const int64_t B = q.size(0), Hq = q.size(1), D = q.size(2), Hkv = k.size(1);
  const Paged pg = paged_args(page_table, k, nullptr, B, seq_len);
  const int64_t T = pg.table ? seq_len : k.size(2);
  TORCH_CHECK(D == 128 && Hq == 4 * Hkv, "planner kernels: D = 128, G = 4");
  need_f32(csum, "csum"); need_f32(lse_ref, "lse_ref"); need_f32(cs_ref, "cs_ref");
  need_f32(lse_att, "lse_att"); need_f32(cs_now, "cs_now");
  TORCH_CHECK(keep.is_cuda() && keep.scalar_type() == at::kByte && keep.dim() == 3 && keep.is_contiguous(),
              "keep: contiguous uint8 [B, Hkv, NBC]");
  const int64_t NBC = keep.size(2);
  TORCH_CHECK((T + KVSKIP_TILE - 1) / KVSKIP_TILE <= NBC, "block capacity exceeded");
  TORCH_CHECK(csum.size(2) == NBC && lse_ref.size(2) == NBC && cs_ref.size(2) == NBC && cs_now.size(2) == NBC &&
                  block_idx.size(2) == NBC, "capacity mismatch");
  TORCH_CHECK(age.scalar_type() == at::kInt && flags.scalar_type() == at::kInt && trig.scalar_type() == at::kByte &&
                  block_idx.scalar_type() == at::kInt && block_cnt.scalar_type() == at::kInt &&
                  age.is_contiguous() && flags.is_contiguous() && trig.is_contiguous() && block_idx.is_contiguous() &&
                  block_cnt.is_contiguous(), "age / flags / block_idx / block_cnt: contiguous int32, trig: uint8");
  const c10::cuda::CUDAGuard guard(q.device());
  kvskip_plan_params p{};
  p.q = u16(q);
  p.q_sb = q.stride(0); p.q_sh = q.stride(1);
  p.k = u16(k);
  p.k_sb = k.stride(0); p.k_sh = k.stride(1); p.k_st = k.stride(2);
  p.csum = csum.data_ptr<float>();
  p.lse_ref = lse_ref.data_ptr<float>();
  p.cs_ref = cs_ref.data_ptr<float>();
  p.keep = keep.data_ptr<uint8_t>();
  p.lse_att = lse_att.data_ptr<float>();
  p.age = age.data_ptr<int32_t>();
  p.flags = flags.data_ptr<int32_t>();
  if (idx.has_value()) {
    TORCH_CHECK(idx->is_cuda() && idx->scalar_type() == at::kByte && idx->is_contiguous() && idx->size(0) == B &&
                    idx->size(1) == NBC, "idx: contiguous uint8 [B, NBC]");
    p.idx = idx->data_ptr<uint8_t>();
  }
  if (calib.has_value()) {
    need_f32(*calib, "calib");
    TORCH_CHECK(calib->numel() == B * Hkv, "calib: [B, Hkv]");
    p.calib = calib->data_ptr<float>();
  }
  if (est.has_value()) {
    need_f32(*est, "est");
    TORCH_CHECK(est->numel() == B * Hkv, "est: [B, Hkv]");
    p.est = est->data_ptr<float>();
  }
  p.calib_on = calib_on;
  p.calib_kind = static_cast<int32_t>(calib_kind);
  if (aix.has_value()) {
    TORCH_CHECK(aix->is_cuda() && aix->scalar_type() == at::kByte && aix->is_contiguous() && aix->numel() == B * Hkv,
                "aix: contiguous uint8 [B, Hkv]");
    TORCH_CHECK(idx.has_value(), "aix needs idx");
    p.aix = aix->data_ptr<uint8_t>();
  }
  p.cs_now = cs_now.data_ptr<float>();
  p.trig = trig.data_ptr<uint8_t>();
  p.block_idx = block_idx.data_ptr<int32_t>();
  p.block_cnt = block_cnt.data_ptr<int32_t>();
  p.B = static_cast<int32_t>(B); p.Hq = static_cast<int32_t>(Hq); p.Hkv = static_cast<int32_t>(Hkv);
  p.T = static_cast<int32_t>(T); p.NBC = static_cast<int32_t>(NBC);
  p.local = static_cast<int32_t>(local); p.max_age = static_cast<int32_t>(max_age); p.add_token = add_token;
  p.scale = static_cast<float>(scale); p.delta = static_cast<float>(delta);
  if (pg.table)
    raise_on(kvskip_launch_plan_paged(&p, pg.table, pg.max_pages, pg.num_pages, tdev_ptr(t_dev), cur_stream()));
  else if (const int* td = tdev_ptr(t_dev))
    raise_on(kvskip_launch_plan_dyn(&p, td, cur_stream()));
  else
    raise_on(kvskip_launch_plan(&p, cur_stream()));
}

void update(const at::Tensor& blk_max, const at::Tensor& blk_sum, const at::Tensor& trig, const at::Tensor& cs_now,
            at::Tensor& keep, at::Tensor& lse_ref, at::Tensor& cs_ref, at::Tensor& lse_att, int64_t T,
            double level, int64_t local, const c10::optional<at::Tensor>& flags,
            const c10::optional<at::Tensor>& idx, const c10::optional<at::Tensor>& est,
            const c10::optional<at::Tensor>& calib, double calib_rate, bool calib_free, int64_t calib_kind,
            const c10::optional<at::Tensor>& aix, double aix_thr, const c10::optional<at::Tensor>& t_dev) {
  need_f32(blk_max, "blk_max"); need_f32(blk_sum, "blk_sum");
  const int64_t B = keep.size(0), Hkv = keep.size(1), NBC = keep.size(2), Hq = lse_att.size(1);
  TORCH_CHECK(blk_max.size(2) == (T + KVSKIP_TILE - 1) / KVSKIP_TILE, "stats length mismatch");
  const c10::cuda::CUDAGuard guard(keep.device());
  kvskip_update_params p{};
  p.blk_max = blk_max.data_ptr<float>();
  p.blk_sum = blk_sum.data_ptr<float>();
  p.trig = trig.data_ptr<uint8_t>();
  p.cs_now = cs_now.data_ptr<float>();
  p.keep = keep.data_ptr<uint8_t>();
  p.lse_ref = lse_ref.data_ptr<float>();
  p.cs_ref = cs_ref.data_ptr<float>();
  p.lse_att = lse_att.data_ptr<float>();
  p.B = static_cast<int32_t>(B); p.Hq = static_cast<int32_t>(Hq); p.Hkv = static_cast<int32_t>(Hkv);
  p.T = static_cast<int32_t>(T); p.NBC = static_cast<int32_t>(NBC); p.local = static_cast<int32_t>(local);
  p.level = static_cast<float>(level);
  if (calib.has_value()) {
    TORCH_CHECK(flags.has_value() && est.has_value(), "calibration needs flags and est");
    TORCH_CHECK(flags->is_cuda() && flags->scalar_type() == at::kInt && flags->numel() == Hkv, "flags: int32 [Hkv]");
    need_f32(*est, "est");
    need_f32(*calib, "calib");
    TORCH_CHECK(est->numel() == B * Hkv && calib->numel() == B * Hkv, "est / calib: [B, Hkv]");
    p.flags = flags->data_ptr<int32_t>();
    p.est = est->data_ptr<float>();
    p.calib = calib->data_ptr<float>();
    p.calib_rate = static_cast<float>(calib_rate);
    p.calib_free = calib_free;
    p.calib_kind = static_cast<int32_t>(calib_kind);
    if (aix.has_value()) {
      TORCH_CHECK(aix->is_cuda() && aix->scalar_type() == at::kByte && aix->is_contiguous() && aix->numel() == B * Hkv,
                  "aix: contiguous uint8 [B, Hkv]");
      TORCH_CHECK(idx.has_value(), "aix needs idx");
      p.aix = aix->data_ptr<uint8_t>();
      p.aix_thr = static_cast<float>(aix_thr);
    }
    if (idx.has_value()) {
      TORCH_CHECK(idx->is_cuda() && idx->scalar_type() == at::kByte && idx->is_contiguous() && idx->size(0) == B &&
                      idx->size(1) == NBC, "idx: contiguous uint8 [B, NBC]");
      p.idx = idx->data_ptr<uint8_t>();
    }
  }
  if (const int* td = tdev_ptr(t_dev))
    raise_on(kvskip_launch_update_dyn(&p, td, cur_stream()));
  else
    raise_on(kvskip_launch_update(&p, cur_stream()));
}

// `update` beside the main stream.  A layer that wants its `update` off the critical path owns one of
// these: a second stream and two events.  refresh_step forks after the attention launch and records
// `done` after update; overlap_join makes the current stream wait for the latest update (before the
// layer's next step, and before anything else reads the planner state).  The caller keeps the
// statistics tensors refresh_step returned, and the index tensor it passed, alive until that join:
// nothing here tells the framework's allocator that the second stream still reads them.
struct Overlap {
  int device;
  c10::cuda::CUDAStream side;   // from the framework's pool: lives as long as the process, so memory that
                                // was marked as used on it can be released at any time
  cudaEvent_t fork, done;
  bool pending;
};

int64_t overlap_create() {
  int device = 0;
  TORCH_CHECK(cudaGetDevice(&device) == cudaSuccess, "overlap_create: no current device");
  auto* o = new Overlap{device, c10::cuda::getStreamFromPool(false, static_cast<c10::DeviceIndex>(device)), nullptr,
                        nullptr, false};
  TORCH_CHECK(cudaEventCreateWithFlags(&o->fork, cudaEventDisableTiming) == cudaSuccess &&
                  cudaEventCreateWithFlags(&o->done, cudaEventDisableTiming) == cudaSuccess,
              "overlap_create: cannot create the events");
  return reinterpret_cast<int64_t>(o);
}

void overlap_join(int64_t handle) {
  auto* o = reinterpret_cast<Overlap*>(handle);
  if (!o || !o->pending) return;
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  TORCH_CHECK(cudaStreamIsCapturing(static_cast<cudaStream_t>(cur_stream()), &st) == cudaSuccess &&
                  st == cudaStreamCaptureStatusNone,
              "overlap_join: an update of this layer is in flight on its own stream; join the layer before the capture "
              "starts (a capturing stream cannot wait for work outside the capture)");
  TORCH_CHECK(cudaStreamWaitEvent(static_cast<cudaStream_t>(cur_stream()), o->done, 0) == cudaSuccess,
              "overlap_join: cannot wait for the update stream");
  o->pending = false;
}

void overlap_destroy(int64_t handle) {
  auto* o = reinterpret_cast<Overlap*>(handle);
  if (!o) return;
  cudaEventDestroy(o->fork);    // (work already queued behind an event is not affected by its destruction)
  cudaEventDestroy(o->done);
  delete o;
}

// One layer's refresh-policy step in a single call: plan -> masked attention with block
// statistics over plan's block list -> update, three launches on the current stream and no host
// synchronisation (what the reference's caller issues as three Python calls,
// src/kvskip_attn.py:463-473).  Returns [out, lse, blk_max, blk_sum].
std::vector<at::Tensor> refresh_step(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, at::Tensor& csum,
                                     at::Tensor& lse_ref, at::Tensor& cs_ref, at::Tensor& keep, at::Tensor& lse_att,
                                     at::Tensor& age, const at::Tensor& flags, at::Tensor& cs_now, at::Tensor& trig,
                                     at::Tensor& block_idx, at::Tensor& block_cnt, double scale, double delta,
                                     int64_t max_age, int64_t local, double level, int64_t num_splits,
                                     const c10::optional<at::Tensor>& idx, const c10::optional<at::Tensor>& calib,
                                     const c10::optional<at::Tensor>& est, bool calib_on, int64_t calib_kind,
                                     double calib_rate, bool calib_free, const c10::optional<at::Tensor>& aix,
                                     double aix_thr, const c10::optional<at::Tensor>& t_dev,
                                     const c10::optional<at::Tensor>& page_table, int64_t seq_len, int64_t overlap) {
  Overlap* o = reinterpret_cast<Overlap*>(overlap);
  cudaStream_t main = static_cast<cudaStream_t>(cur_stream());
  if (o) {   // no second stream inside a stream capture: the captured step stays one chain
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(main, &st) != cudaSuccess || st != cudaStreamCaptureStatusNone) o = nullptr;
  }
  overlap_join(overlap);          // this layer's previous update wrote what plan reads
  plan(q, k, csum, lse_ref, cs_ref, keep, lse_att, age, flags, cs_now, trig, block_idx, block_cnt, scale, delta, max_age,
       local, true, idx, calib, est, calib_on, calib_kind, aix, t_dev, page_table, seq_len);
  auto r = decode(q, k, v, scale, block_idx, block_cnt, true, true, num_splits, 2, false, false, t_dev, page_table,
                  seq_len);
  const int64_t T_upd = page_table.has_value() ? seq_len : k.size(2);
  if (!o) {
    update(r[2], r[3], trig, cs_now, keep, lse_ref, cs_ref, lse_att, T_upd, level, local, flags, idx, est, calib,
           calib_rate, calib_free, calib_kind, aix, aix_thr, t_dev);
    return {r[0], r[1], r[2], r[3]};
  }
  // update on the layer's second stream: it needs the statistics of this pass and prepares the same
  // layer's next step, so whatever follows on the current stream need not wait for it
  TORCH_CHECK(cudaEventRecord(o->fork, main) == cudaSuccess && cudaStreamWaitEvent(o->side.stream(), o->fork, 0) == cudaSuccess,
              "refresh_step: cannot fork the update stream");
  {
    const c10::cuda::CUDAStream side = o->side;
    const c10::cuda::CUDAStreamGuard on_side(side);
    update(r[2], r[3], trig, cs_now, keep, lse_ref, cs_ref, lse_att, T_upd, level, local, flags, idx, est, calib,
           calib_rate, calib_free, calib_kind, aix, aix_thr, t_dev);
  }
  TORCH_CHECK(cudaEventRecord(o->done, o->side.stream()) == cudaSuccess, "refresh_step: cannot record the end of update");
  o->pending = true;
  return {r[0], r[1], r[2], r[3]};
}

void read_bw(const at::Tensor& x, at::Tensor& out, int64_t blocks, bool bulk) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.nbytes() % 16 == 0, "x: contiguous CUDA, 16-byte multiple");
  const c10::cuda::CUDAGuard guard(x.device());
  if (bulk) {
    raise_on(kvskip_launch_read_bulk(x.data_ptr(), static_cast<int64_t>(x.nbytes()),
                                     reinterpret_cast<uint32_t*>(out.data_ptr()), static_cast<int>(blocks), cur_stream()));
    return;
  }
  raise_on(kvskip_launch_read(x.data_ptr(), static_cast<int64_t>(x.nbytes()), reinterpret_cast<uint32_t*>(out.data_ptr()),
                              static_cast<int>(blocks), cur_stream()));
}

// part_acc [R,N,D] fp32, part_ml [R,N,2] fp32 -> [out bf16 [N,D], out_f32 [N,D], lse [N]]
std::vector<at::Tensor> merge(const at::Tensor& part_acc, const at::Tensor& part_ml) {
  need_f32(part_acc, "part_acc"); need_f32(part_ml, "part_ml");
  TORCH_CHECK(part_acc.dim() == 3 && part_ml.dim() == 3 && part_ml.size(2) == 2 && part_ml.size(0) == part_acc.size(0) &&
                  part_ml.size(1) == part_acc.size(1), "part_acc [R,N,D], part_ml [R,N,2]");
  const c10::cuda::CUDAGuard guard(part_acc.device());
  const int64_t R = part_acc.size(0), N = part_acc.size(1), D = part_acc.size(2);
  at::Tensor out = at::empty({N, D}, part_acc.options().dtype(at::kBFloat16));
  at::Tensor out32 = at::empty({N, D}, part_acc.options());
  at::Tensor lse = at::empty({N}, part_acc.options());
  raise_on(kvskip_launch_merge(part_acc.data_ptr<float>(), part_ml.data_ptr<float>(), static_cast<int>(R), N,
                               static_cast<int>(D), u16m(out), out32.data_ptr<float>(), lse.data_ptr<float>(),
                               cur_stream()));
  return {out, out32, lse};
}

// out_f32 [.., D] fp32, lse [..] fp32 -> packed [N, D+2] fp32 (rows [out | lse/ln2 | 1])
at::Tensor pack_partial(const at::Tensor& out_f32, const at::Tensor& lse) {
  need_f32(out_f32, "out_f32"); need_f32(lse, "lse");
  const int64_t D = out_f32.size(-1), N = out_f32.numel() / D;
  TORCH_CHECK(lse.numel() == N, "lse: one value per row of out_f32");
  const c10::cuda::CUDAGuard guard(out_f32.device());
  at::Tensor packed = at::empty({N, D + 2}, out_f32.options());
  raise_on(kvskip_launch_pack_partial(out_f32.data_ptr<float>(), lse.data_ptr<float>(), packed.data_ptr<float>(), N,
                                      static_cast<int>(D), cur_stream()));
  return packed;
}

// parts [R,N,D+2] fp32 -> [out bf16 [N,D], out_f32 [N,D], lse [N]]
std::vector<at::Tensor> merge_packed(const at::Tensor& parts) {
  need_f32(parts, "parts");
  TORCH_CHECK(parts.dim() == 3 && parts.size(2) > 2, "parts [R,N,D+2]");
  const c10::cuda::CUDAGuard guard(parts.device());
  const int64_t R = parts.size(0), N = parts.size(1), D = parts.size(2) - 2;
  at::Tensor out = at::empty({N, D}, parts.options().dtype(at::kBFloat16));
  at::Tensor out32 = at::empty({N, D}, parts.options());
  at::Tensor lse = at::empty({N}, parts.options());
  raise_on(kvskip_launch_merge_packed(parts.data_ptr<float>(), static_cast<int>(R), N, static_cast<int>(D), u16m(out),
                                      out32.data_ptr<float>(), lse.data_ptr<float>(), cur_stream()));
  return {out, out32, lse};
}

// Fused exchange + merge over peer memory; buf_ptrs / flag_ptrs are the peers' device addresses.
std::vector<at::Tensor> exchange_merge(const at::Tensor& out_f32, const at::Tensor& lse,
                                       const std::vector<int64_t>& buf_ptrs, const std::vector<int64_t>& flag_ptrs,
                                       int64_t rank, int64_t seq) {
  need_f32(out_f32, "out_f32"); need_f32(lse, "lse");
  const int64_t D = out_f32.size(-1), N = out_f32.numel() / D, R = static_cast<int64_t>(buf_ptrs.size());
  TORCH_CHECK(lse.numel() == N && flag_ptrs.size() == buf_ptrs.size() && R >= 1 && R <= 8, "exchange_merge arguments");
  const c10::cuda::CUDAGuard guard(out_f32.device());
  float* bufs[8];
  unsigned int* flags[8];
  for (int64_t r = 0; r < R; ++r) {
    bufs[r] = reinterpret_cast<float*>(buf_ptrs[r]);
    flags[r] = reinterpret_cast<unsigned int*>(flag_ptrs[r]);   // unused by the library
  }
  at::Tensor out = at::empty({N, D}, out_f32.options().dtype(at::kBFloat16));
  at::Tensor out32 = at::empty({N, D}, out_f32.options());
  at::Tensor res_lse = at::empty({N}, out_f32.options());
  raise_on(kvskip_launch_exchange_merge(out_f32.data_ptr<float>(), lse.data_ptr<float>(), bufs, flags,
                                        static_cast<int>(rank), static_cast<int>(R), N, static_cast<int>(D),
                                        static_cast<unsigned int>(seq), u16m(out), out32.data_ptr<float>(),
                                        res_lse.data_ptr<float>(), cur_stream()));
  return {out, out32, res_lse};
}

void index_blocks(const at::Tensor& ids, int64_t T, at::Tensor& out, const c10::optional<at::Tensor>& t_dev) {
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.dim() == 2 && ids.stride(1) == 1, "ids: CUDA int64 [n, >= T]");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kByte && out.dim() == 2 && out.is_contiguous() &&
                  out.size(0) == ids.size(0), "out: contiguous uint8 [n, NBC]");
  TORCH_CHECK(T >= 1 && T <= ids.size(1), "T within ids");
  const c10::cuda::CUDAGuard guard(ids.device());
  if (const int* td = tdev_ptr(t_dev))
    raise_on(kvskip_launch_index_blocks_dyn(ids.data_ptr<int64_t>(), ids.stride(0), static_cast<int>(ids.size(0)),
                                            static_cast<int>(T), td, out.data_ptr<uint8_t>(),
                                            static_cast<int>(out.size(1)), cur_stream()));
  else
    raise_on(kvskip_launch_index_blocks(ids.data_ptr<int64_t>(), ids.stride(0), static_cast<int>(ids.size(0)),
                                        static_cast<int>(T), out.data_ptr<uint8_t>(), static_cast<int>(out.size(1)),
                                        cur_stream()));
}

// The newest token's K and V rows (k_new, v_new [B,Hkv,D]) into row T-1 of a contiguous cache
// [B,Hkv,cap,D] or, with a page table, of a page pool [pages,Hkv,64,D]; T is the length after the
// append (read from t_dev if given, T then bounds it).
void append(at::Tensor& k, at::Tensor& v, const at::Tensor& k_new, const at::Tensor& v_new, int64_t T,
            const c10::optional<at::Tensor>& t_dev, const c10::optional<at::Tensor>& page_table) {
  need_kv(k, "k"); need_kv(v, "v");
  const int64_t B = k_new.size(0), Hkv = k.size(1), D = k.size(3);
  TORCH_CHECK(k_new.is_cuda() && v_new.is_cuda() && k_new.scalar_type() == at::kBFloat16 &&
                  v_new.scalar_type() == at::kBFloat16 && k_new.is_contiguous() && v_new.is_contiguous() &&
                  k_new.dim() == 3 && k_new.sizes() == v_new.sizes() && k_new.size(1) == Hkv && k_new.size(2) == D,
              "k_new, v_new: contiguous CUDA bf16 [B, Hkv, D]");
  TORCH_CHECK(k.sizes() == v.sizes() && k.strides() == v.strides(), "k and v must share shape and strides");
  const Paged pg = paged_args(page_table, k, &v, B, T);
  TORCH_CHECK(pg.table || (k.size(0) == B && T >= 1 && T <= k.size(2)), "append: T within the cache");
  const c10::cuda::CUDAGuard guard(k.device());
  raise_on(kvskip_launch_append(u16m(k), u16m(v), k.stride(0), k.stride(1), k.stride(2), u16(k_new), u16(v_new),
                                static_cast<int>(B), static_cast<int>(Hkv), static_cast<int>(D), static_cast<int>(T),
                                tdev_ptr(t_dev), pg.table, pg.max_pages, pg.num_pages, cur_stream()));
}

// Block selection of the two-pass V-skip on the device: [keep u8 [B,Hkv,nb], block_idx, block_cnt, weight [B,Hkv,nb,4]]
std::vector<at::Tensor> select_dev(const at::Tensor& blk_max, const at::Tensor& blk_sum, int64_t rule, double value,
                               int64_t local, const c10::optional<at::Tensor>& t_dev, int64_t T_bound) {
  need_f32(blk_max, "blk_max"); need_f32(blk_sum, "blk_sum");
  TORCH_CHECK(blk_max.dim() == 3 && blk_max.sizes() == blk_sum.sizes() && blk_max.size(1) % 4 == 0,
              "blk_max, blk_sum: fp32 [B, 4*Hkv, nb]");
  const int64_t B = blk_max.size(0), Hkv = blk_max.size(1) / 4, nb = blk_max.size(2);
  const c10::cuda::CUDAGuard guard(blk_max.device());
  at::Tensor keep = at::empty({B, Hkv, nb}, blk_max.options().dtype(at::kByte));
  at::Tensor bi = at::empty({B, Hkv, nb}, blk_max.options().dtype(at::kInt));
  at::Tensor bc = at::empty({B, Hkv}, blk_max.options().dtype(at::kInt));
  at::Tensor w = at::empty({B, Hkv, nb, 4}, blk_max.options());
  if (const int* td = tdev_ptr(t_dev)) {
    TORCH_CHECK((T_bound + KVSKIP_TILE - 1) / KVSKIP_TILE == nb, "select: T_bound must match the rows of blk_max");
    raise_on(kvskip_launch_select_dyn(blk_max.data_ptr<float>(), blk_sum.data_ptr<float>(), static_cast<int>(B),
                                      static_cast<int>(Hkv), static_cast<int>(T_bound), td, static_cast<int>(rule),
                                      static_cast<float>(value), static_cast<int>(local), keep.data_ptr<uint8_t>(),
                                      bi.data_ptr<int32_t>(), bc.data_ptr<int32_t>(), w.data_ptr<float>(), cur_stream()));
    return {keep, bi, bc, w};
  }
  raise_on(kvskip_launch_select(blk_max.data_ptr<float>(), blk_sum.data_ptr<float>(), static_cast<int>(B),
                                static_cast<int>(Hkv), static_cast<int>(nb), static_cast<int>(rule),
                                static_cast<float>(value), static_cast<int>(local), keep.data_ptr<uint8_t>(),
                                bi.data_ptr<int32_t>(), bc.data_ptr<int32_t>(), w.data_ptr<float>(), cur_stream()));
  return {keep, bi, bc, w};
}

// *t_dev += delta in stream order
void advance(at::Tensor& t_dev, int64_t delta) {
  TORCH_CHECK(t_dev.is_cuda() && t_dev.scalar_type() == at::kInt && t_dev.numel() == 1,
              "t_dev: one-element int32 CUDA tensor");
  const c10::cuda::CUDAGuard guard(t_dev.device());
  raise_on(kvskip_launch_advance(t_dev.data_ptr<int32_t>(), static_cast<int>(delta), cur_stream()));
}

void set_option(const std::string& name, int64_t value) {
  raise_on(kvskip_set_option(name.c_str(), static_cast<int>(value)));
}

int64_t get_option(const std::string& name) {
  const int v = kvskip_get_option(name.c_str());
  TORCH_CHECK(v >= 0, kvskip_last_error());
  return v;
}

int64_t device_status() {
  unsigned int st = 0;
  raise_on(kvskip_device_status(cur_stream(), &st));
  return static_cast<int64_t>(st);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("read_bw", &read_bw, "streaming read of x (bandwidth ceiling); bulk: through the copy engine",
        py::arg("x"), py::arg("out"), py::arg("blocks"), py::arg("bulk") = false);
  m.def("plan", &plan, "refresh planner: decision and block lists (before the pass)",
        py::arg("q"), py::arg("k"), py::arg("csum"), py::arg("lse_ref"), py::arg("cs_ref"), py::arg("keep"),
        py::arg("lse_att"), py::arg("age"), py::arg("flags"), py::arg("cs_now"), py::arg("trig"),
        py::arg("block_idx"), py::arg("block_cnt"), py::arg("scale"), py::arg("delta"), py::arg("max_age"),
        py::arg("local"), py::arg("add_token"), py::arg("idx") = py::none(), py::arg("calib") = py::none(),
        py::arg("est") = py::none(), py::arg("calib_on") = false, py::arg("calib_kind") = 0,
        py::arg("aix") = py::none(), py::arg("t_dev") = py::none(), py::arg("page_table") = py::none(),
        py::arg("seq_len") = 0);
  m.def("update", &update, "refresh planner: stored set and references (after the pass)",
        py::arg("blk_max"), py::arg("blk_sum"), py::arg("trig"), py::arg("cs_now"), py::arg("keep"),
        py::arg("lse_ref"), py::arg("cs_ref"), py::arg("lse_att"), py::arg("T"), py::arg("level"), py::arg("local"),
        py::arg("flags") = py::none(), py::arg("idx") = py::none(), py::arg("est") = py::none(),
        py::arg("calib") = py::none(), py::arg("calib_rate") = 0.0, py::arg("calib_free") = false,
        py::arg("calib_kind") = 0, py::arg("aix") = py::none(), py::arg("aix_thr") = 0.0,
        py::arg("t_dev") = py::none());
  m.def("vskip1", &vskip1, "single-pass V-skip", py::arg("q"), py::arg("k"), py::arg("v"), py::arg("scale"),
        py::arg("tau"), py::arg("local") = 2, py::arg("num_splits") = 1, py::arg("want_f32") = false,
        py::arg("count") = false, py::arg("lse_prev") = py::none(), py::arg("page_table") = py::none(),
        py::arg("seq_len") = 0, py::arg("t_dev") = py::none());
  m.def("decode", &decode, "split-K decode attention", py::arg("q"), py::arg("k"), py::arg("v"), py::arg("scale"),
        py::arg("block_idx") = py::none(), py::arg("block_cnt") = py::none(), py::arg("stats") = false,
        py::arg("load_v") = true, py::arg("num_splits") = 1, py::arg("stages") = 2, py::arg("want_f32") = false,
        py::arg("write_p") = false, py::arg("t_dev") = py::none(), py::arg("page_table") = py::none(),
        py::arg("seq_len") = 0);
  m.def("pv", &pv, "two-pass V-skip, pass 2", py::arg("P"), py::arg("v"), py::arg("blk_scale"), py::arg("block_idx"),
        py::arg("block_cnt"), py::arg("num_splits") = 1, py::arg("want_f32") = false, py::arg("t_dev") = py::none());
  m.def("refresh_step", &refresh_step, "plan -> masked+stats attention -> update for one layer, one call",
        py::arg("q"), py::arg("k"), py::arg("v"), py::arg("csum"), py::arg("lse_ref"), py::arg("cs_ref"),
        py::arg("keep"), py::arg("lse_att"), py::arg("age"), py::arg("flags"), py::arg("cs_now"), py::arg("trig"),
        py::arg("block_idx"), py::arg("block_cnt"), py::arg("scale"), py::arg("delta"), py::arg("max_age"),
        py::arg("local"), py::arg("level"), py::arg("num_splits"), py::arg("idx") = py::none(),
        py::arg("calib") = py::none(), py::arg("est") = py::none(), py::arg("calib_on") = false,
        py::arg("calib_kind") = 0, py::arg("calib_rate") = 0.0, py::arg("calib_free") = false,
        py::arg("aix") = py::none(), py::arg("aix_thr") = 0.0, py::arg("t_dev") = py::none(),
        py::arg("page_table") = py::none(), py::arg("seq_len") = 0, py::arg("overlap") = 0);
  m.def("overlap_create", &overlap_create, "a second stream + events for a layer's `update` (handle for refresh_step)");
  m.def("overlap_join", &overlap_join, "the current stream waits for the layer's latest `update`", py::arg("handle"));
  m.def("overlap_destroy", &overlap_destroy, py::arg("handle"));
  m.def("merge", &merge, "merge of R partial (max, sum, acc) rows", py::arg("part_acc"), py::arg("part_ml"));
  m.def("pack_partial", &pack_partial, "rank-local (out_f32, lse) -> packed (acc, m, l) rows", py::arg("out_f32"),
        py::arg("lse"));
  m.def("merge_packed", &merge_packed, "merge of R packed partial buffers [R,N,D+2]", py::arg("parts"));
  m.def("decode_exchange", &decode_exchange,
        "sequence shards: local attention, peer-memory exchange and merge in one kernel", py::arg("q"), py::arg("k"),
        py::arg("v"), py::arg("scale"), py::arg("block_idx") = py::none(), py::arg("block_cnt") = py::none(),
        py::arg("num_splits") = 2, py::arg("buf_ptrs"), py::arg("flag_ptrs"), py::arg("rank"), py::arg("seq"));
  m.def("exchange_merge", &exchange_merge, "sequence shards: peer-memory exchange and merge in one kernel",
        py::arg("out_f32"), py::arg("lse"), py::arg("buf_ptrs"), py::arg("flag_ptrs"), py::arg("rank"), py::arg("seq"));
  m.def("index_blocks", &index_blocks, "token-index blocks of one step", py::arg("ids"), py::arg("T"), py::arg("out"),
        py::arg("t_dev") = py::none());
  m.def("append", &append, "the newest token's K and V rows into the cache (contiguous or paged)", py::arg("k"),
        py::arg("v"), py::arg("k_new"), py::arg("v_new"), py::arg("T"), py::arg("t_dev") = py::none(),
        py::arg("page_table") = py::none());
  m.def("select", &select_dev, "two-pass V-skip: block selection, list and second-pass weights in one launch",
        py::arg("blk_max"), py::arg("blk_sum"), py::arg("rule"), py::arg("value"), py::arg("local") = 2,
        py::arg("t_dev") = py::none(), py::arg("T_bound") = 0);
  m.def("advance", &advance, "device-resident sequence length += delta, in stream order", py::arg("t_dev"),
        py::arg("delta") = 1);
  m.def("set_option", &set_option, "process-wide option, e.g. (\"decode_path\", 1) for the exact-order kernels",
        py::arg("name"), py::arg("value"));
  m.def("get_option", &get_option, py::arg("name"));
  m.def("device_status", &device_status, "synchronise and return the kernels' status word (0 = fine)");
}
