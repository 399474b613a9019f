"""ctypes binding of the C ABI (include/kvskip_b200.h): the stub a host that cannot use the
pybind module would write.  Functions take CUDA torch tensors only to borrow their device
pointers and strides; every launch goes through `kvskip_launch_*` of libkvskip_b200.so.

`CAbi(path, prefix)` can also be pointed at another library exporting the same entry points under
a different prefix; the tests use that to drive the reference's kernels with identical arguments.
"""

import ctypes as C
import math
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
TILE = 64

_vp, _i64, _i32, _f32 = C.c_void_p, C.c_int64, C.c_int32, C.c_float


class Params(C.Structure):
    _fields_ = [("q", _vp), ("k", _vp), ("v", _vp),
                ("q_sb", _i64), ("q_sh", _i64),
                ("k_sb", _i64), ("k_sh", _i64), ("k_st", _i64),
                ("v_sb", _i64), ("v_sh", _i64), ("v_st", _i64),
                ("B", _i32), ("Hq", _i32), ("Hkv", _i32), ("T", _i32),
                ("scale_log2", _f32),
                ("block_idx", _vp), ("block_cnt", _vp), ("max_blocks", _i32),
                ("num_splits", _i32), ("part_acc", _vp), ("part_ml", _vp),
                ("out", _vp), ("out_f32", _vp), ("lse", _vp),
                ("blk_max", _vp), ("blk_sum", _vp), ("nb", _i32),
                ("p_out", _vp), ("p_in", _vp), ("blk_scale", _vp), ("t_pad", _i64),
                ("log2_tau", _f32), ("local", _i32), ("vcount", _vp), ("lse_prev", _vp)]


class PlanParams(C.Structure):
    _fields_ = [("q", _vp), ("q_sb", _i64), ("q_sh", _i64),
                ("k", _vp), ("k_sb", _i64), ("k_sh", _i64), ("k_st", _i64),
                ("csum", _vp), ("lse_ref", _vp), ("cs_ref", _vp), ("keep", _vp), ("lse_att", _vp),
                ("age", _vp), ("flags", _vp), ("idx", _vp), ("calib", _vp), ("est", _vp),
                ("calib_on", _i32), ("calib_kind", _i32), ("aix", _vp),
                ("cs_now", _vp), ("trig", _vp), ("block_idx", _vp), ("block_cnt", _vp),
                ("B", _i32), ("Hq", _i32), ("Hkv", _i32), ("T", _i32), ("NBC", _i32), ("local", _i32),
                ("max_age", _i32), ("add_token", _i32), ("scale", _f32), ("delta", _f32)]


class UpdateParams(C.Structure):
    _fields_ = [("blk_max", _vp), ("blk_sum", _vp), ("trig", _vp), ("cs_now", _vp), ("keep", _vp),
                ("lse_ref", _vp), ("cs_ref", _vp), ("lse_att", _vp), ("flags", _vp), ("idx", _vp),
                ("est", _vp), ("calib", _vp), ("calib_rate", _f32), ("calib_free", _i32),
                ("calib_kind", _i32), ("aix", _vp), ("aix_thr", _f32),
                ("B", _i32), ("Hq", _i32), ("Hkv", _i32), ("T", _i32), ("NBC", _i32), ("local", _i32),
                ("level", _f32)]


def _ptr(t):
    return None if t is None else t.data_ptr()


def _default_lib():
    from . import build
    return build.LIB


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class CAbi:
    def __init__(self, path=None, prefix="kvskip"):
        self.path = Path(path) if path else _default_lib()
        if not self.path.exists():
            raise RuntimeError(f"{self.path} is missing: build it with `python -m kvskip_b200.build`")
        self.lib = C.CDLL(str(self.path))
        self.prefix = prefix
        getattr(self.lib, f"{prefix}_last_error").restype = C.c_char_p

    def _call(self, name, *args):
        rc = getattr(self.lib, f"{self.prefix}_launch_{name}")(*args)
        if rc != 0:
            raise RuntimeError(getattr(self.lib, f"{self.prefix}_last_error")().decode())

    @staticmethod
    def _qkv(p, q, k, v):
        p.q, p.k, p.v = _ptr(q), _ptr(k), _ptr(v)
        p.q_sb, p.q_sh = q.stride(0), q.stride(1)
        p.k_sb, p.k_sh, p.k_st = k.stride(0), k.stride(1), k.stride(2)
        p.v_sb, p.v_sh, p.v_st = v.stride(0), v.stride(1), v.stride(2)
        p.B, p.Hq, p.Hkv, p.T = q.shape[0], q.shape[1], k.shape[1], k.shape[2]

    def decode_noalloc(self, q, k, v, scale, out, lse, block_idx=None, block_cnt=None, num_splits=1, out_f32=None):
        """kvskip_launch_decode_noalloc: the caller passes every buffer (out bf16 [B,Hq,D], lse fp32
        [B,Hq], optional out_f32); nothing is allocated here or in the library, the split
        partials live in the library's built-in array."""
        B, Hq, D = q.shape
        Hkv, T = k.shape[1], k.shape[2]
        p = Params()
        self._qkv(p, q, k, v)
        p.scale_log2 = scale * 1.4426950408889634
        if block_idx is not None:
            p.block_idx, p.block_cnt, p.max_blocks = _ptr(block_idx), _ptr(block_cnt), block_idx.shape[2]
        p.num_splits = num_splits
        p.out, p.out_f32, p.lse = _ptr(out), _ptr(out_f32), _ptr(lse)
        p.nb, p.t_pad = math.ceil(T / TILE), math.ceil(T / TILE) * TILE
        self._call("decode_noalloc", C.byref(p), D, Hq // Hkv, 2, int(block_idx is not None), 0, 1, _stream())

    def decode(self, q, k, v, scale, block_idx=None, block_cnt=None, stats=False, load_v=True, num_splits=1,
               stages=2, want_f32=False, write_p=False, t_dev=None, page_table=None, seq_len=None):
        """Same arguments and return list as the extension's decode().  t_dev (int32 CUDA scalar):
        kvskip_launch_decode_dyn; page_table (int32 [B, max_pages]) with seq_len:
        kvskip_launch_decode_paged over page pools k, v [pages,Hkv,64,D]."""
        B, Hq, D = q.shape
        Hkv, T = k.shape[1], (k.shape[2] if page_table is None else int(seq_len))
        nb = math.ceil(T / TILE)
        dev = q.device
        f32 = dict(dtype=torch.float32, device=dev)
        out = torch.empty(B, Hq, D, dtype=torch.bfloat16, device=dev) if load_v else None
        o32 = torch.empty(B, Hq, D, **f32) if load_v and want_f32 else None
        lse = torch.empty(B, Hq, **f32)
        bmax = torch.full((B, Hq, nb), float("-inf"), **f32) if stats else None
        bsum = torch.zeros(B, Hq, nb, **f32) if stats else None
        pbuf = torch.empty(B, Hq, nb * TILE, dtype=torch.float16, device=dev) if write_p else None
        pacc = torch.empty(B, Hq, num_splits, D, **f32) if num_splits > 1 else None
        pml = torch.empty(B, Hq, num_splits, 2, **f32) if num_splits > 1 else None
        p = Params()
        self._qkv(p, q, k, v)
        p.scale_log2 = scale * 1.4426950408889634
        if block_idx is not None:
            assert block_idx.dtype == torch.int32 and block_idx.is_contiguous() and block_cnt.dtype == torch.int32
            p.block_idx, p.block_cnt, p.max_blocks = _ptr(block_idx), _ptr(block_cnt), block_idx.shape[2]
        p.num_splits, p.part_acc, p.part_ml = num_splits, _ptr(pacc), _ptr(pml)
        p.out, p.out_f32, p.lse = _ptr(out), _ptr(o32), _ptr(lse)
        p.blk_max, p.blk_sum, p.nb = _ptr(bmax), _ptr(bsum), nb
        p.t_pad, p.p_out = nb * TILE, _ptr(pbuf)
        p.T = T
        flags = (C.byref(p), D, Hq // Hkv, stages, int(block_idx is not None), int(stats), int(load_v))
        if page_table is not None:
            assert page_table.dtype == torch.int32 and page_table.is_contiguous() and page_table.shape[0] == B
            self._call("decode_paged", *flags, C.c_void_p(_ptr(page_table)), page_table.shape[1], k.shape[0],
                       C.c_void_p(_ptr(t_dev)), _stream())
        elif t_dev is not None:
            self._call("decode_dyn", *flags, C.c_void_p(_ptr(t_dev)), _stream())
        else:
            self._call("decode", *flags, _stream())
        self._keep = (pacc, pml)   # scratch must outlive the asynchronous launch
        return [out, lse, bmax, bsum, o32, pbuf]

    def vskip1(self, q, k, v, scale, tau, local=2, num_splits=1, want_f32=False, count=False, lse_prev=None):
        B, Hq, D = q.shape
        Hkv, T = k.shape[1], k.shape[2]
        dev = q.device
        f32 = dict(dtype=torch.float32, device=dev)
        out = torch.empty(B, Hq, D, dtype=torch.bfloat16, device=dev)
        o32 = torch.empty(B, Hq, D, **f32) if want_f32 else None
        lse = torch.empty(B, Hq, **f32)
        vcount = torch.zeros(B, Hkv, dtype=torch.int32, device=dev) if count else None
        pacc = torch.empty(B, Hq, num_splits, D, **f32) if num_splits > 1 else None
        pml = torch.empty(B, Hq, num_splits, 2, **f32) if num_splits > 1 else None
        p = Params()
        self._qkv(p, q, k, v)
        p.scale_log2 = scale * 1.4426950408889634
        p.num_splits, p.part_acc, p.part_ml = num_splits, _ptr(pacc), _ptr(pml)
        p.out, p.out_f32, p.lse = _ptr(out), _ptr(o32), _ptr(lse)
        p.nb = math.ceil(T / TILE)
        p.log2_tau, p.local, p.vcount, p.lse_prev = math.log2(tau), local, _ptr(vcount), _ptr(lse_prev)
        self._call("vskip1", C.byref(p), D, Hq // Hkv, _stream())
        self._keep = (pacc, pml)
        return [out, lse, o32, vcount]

    def pv(self, P, v, blk_scale, block_idx, block_cnt, num_splits=1, want_f32=False):
        B, Hkv, T, D = v.shape
        Hq = P.shape[1]
        nb = math.ceil(T / TILE)
        dev = v.device
        out = torch.empty(B, Hq, D, dtype=torch.bfloat16, device=dev)
        o32 = torch.empty(B, Hq, D, dtype=torch.float32, device=dev) if want_f32 else None
        pacc = torch.empty(B, Hq, num_splits, D, dtype=torch.float32, device=dev) if num_splits > 1 else None
        p = Params()
        p.v, p.v_sb, p.v_sh, p.v_st = _ptr(v), v.stride(0), v.stride(1), v.stride(2)
        p.B, p.Hq, p.Hkv, p.T = B, Hq, Hkv, T
        p.block_idx, p.block_cnt, p.max_blocks = _ptr(block_idx), _ptr(block_cnt), block_idx.shape[2]
        p.num_splits, p.part_acc = num_splits, _ptr(pacc)
        p.out, p.out_f32 = _ptr(out), _ptr(o32)
        p.nb, p.t_pad, p.p_in, p.blk_scale = nb, nb * TILE, _ptr(P), _ptr(blk_scale)
        self._call("pv", C.byref(p), D, Hq // Hkv, _stream())
        self._keep = (pacc,)
        return [out, o32]

    def plan(self, q, k, csum, lse_ref, cs_ref, keep, lse_att, age, flags, cs_now, trig, block_idx, block_cnt,
             scale, delta, max_age, local, add_token, idx=None, calib=None, est=None, calib_on=False,
             calib_kind=0, aix=None):
        p = PlanParams()
        p.q, p.q_sb, p.q_sh = _ptr(q), q.stride(0), q.stride(1)
        p.k, p.k_sb, p.k_sh, p.k_st = _ptr(k), k.stride(0), k.stride(1), k.stride(2)
        p.csum, p.lse_ref, p.cs_ref, p.keep, p.lse_att = map(_ptr, (csum, lse_ref, cs_ref, keep, lse_att))
        p.age, p.flags, p.idx, p.calib, p.est = map(_ptr, (age, flags, idx, calib, est))
        p.calib_on, p.calib_kind, p.aix = int(calib_on), calib_kind, _ptr(aix)
        p.cs_now, p.trig, p.block_idx, p.block_cnt = map(_ptr, (cs_now, trig, block_idx, block_cnt))
        p.B, p.Hq, p.Hkv, p.T, p.NBC = q.shape[0], q.shape[1], k.shape[1], k.shape[2], keep.shape[2]
        p.local, p.max_age, p.add_token, p.scale, p.delta = local, max_age, int(add_token), scale, delta
        self._call("plan", C.byref(p), _stream())

    def update(self, blk_max, blk_sum, trig, cs_now, keep, lse_ref, cs_ref, lse_att, T, level, local, flags=None,
               idx=None, est=None, calib=None, calib_rate=0.0, calib_free=False, calib_kind=0, aix=None,
               aix_thr=0.0):
        p = UpdateParams()
        p.blk_max, p.blk_sum, p.trig, p.cs_now = map(_ptr, (blk_max, blk_sum, trig, cs_now))
        p.keep, p.lse_ref, p.cs_ref, p.lse_att = map(_ptr, (keep, lse_ref, cs_ref, lse_att))
        if calib is not None:
            p.flags, p.idx, p.est, p.calib, p.aix = map(_ptr, (flags, idx, est, calib, aix))
            p.calib_rate, p.calib_free, p.calib_kind, p.aix_thr = calib_rate, int(calib_free), calib_kind, aix_thr
        p.B, p.Hkv, p.NBC, p.Hq = keep.shape[0], keep.shape[1], keep.shape[2], lse_att.shape[1]
        p.T, p.local, p.level = T, local, level
        self._call("update", C.byref(p), _stream())

    def append(self, k, v, k_new, v_new, T, t_dev=None, page_table=None):
        """kvskip_launch_append: rows of the newest token into a contiguous cache or a page pool."""
        B, Hkv, D = k_new.shape
        pt = page_table
        self._call("append", C.c_void_p(_ptr(k)), C.c_void_p(_ptr(v)), C.c_int64(k.stride(0)), C.c_int64(k.stride(1)),
                   C.c_int64(k.stride(2)), C.c_void_p(_ptr(k_new)), C.c_void_p(_ptr(v_new)), B, Hkv, D, int(T),
                   C.c_void_p(_ptr(t_dev)), C.c_void_p(_ptr(pt)), 0 if pt is None else pt.shape[1],
                   0 if pt is None else k.shape[0], _stream())

    def advance(self, t_dev, delta=1):
        self._call("advance", C.c_void_p(_ptr(t_dev)), int(delta), _stream())

    def read_bw(self, x, out, blocks):
        self._call("read", C.c_void_p(x.data_ptr()), C.c_int64(x.numel() * x.element_size()),
                   C.c_void_p(out.data_ptr()), int(blocks), _stream())
