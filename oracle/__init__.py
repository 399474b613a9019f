"""ctypes front end of the CPU oracle (oracle/kvskip_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline leg of
bench.py.  Nothing under kvskip_b200/ imports this package.

All functions take CPU torch tensors (bf16 tensors are passed as their bit patterns, any strides
with the last dim contiguous) and mirror the argument order of the reference's extension functions
(kernels/kvskip_ext.cpp:327-352) so a test can run the same call against either side.
"""

import ctypes
import math
import subprocess
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
_LIB = None
BLOCK = 64


def build(force: bool = False) -> Path:
    so = HERE / "libkvskip_oracle.so"
    src = HERE / "kvskip_oracle.c"
    if force or not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "libkvskip_oracle.so"], check=True, capture_output=True)
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(str(build()))
        _LIB.kvo_version.restype = ctypes.c_int
        _LIB.kvo_num_threads.restype = ctypes.c_int
    return _LIB


def num_threads() -> int:
    return int(lib().kvo_num_threads())


def use_all_cores() -> int:
    """All cores this process may run on, whatever OMP_NUM_THREADS says (torchrun exports 1)."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().kvo_set_num_threads(int(n))
    return num_threads()


def _p(t):
    if t is None:
        return ctypes.c_void_p(0)
    assert t.device.type == "cpu"
    return ctypes.c_void_p(t.data_ptr())


def _i64(x):
    return ctypes.c_int64(int(x))


def _i(x):
    return ctypes.c_int(int(x))


def _f(x):
    return ctypes.c_float(float(x))


def _d(x):
    return ctypes.c_double(float(x))


def _qkv_args(q, k, v=None):
    assert q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and k.stride(-1) == 1
    a = [_p(q), _i64(q.stride(0)), _i64(q.stride(1)), _p(k), _i64(k.stride(0)), _i64(k.stride(1)), _i64(k.stride(2))]
    if v is not None:
        assert v.dtype == torch.bfloat16 and v.stride(-1) == 1
        a += [_p(v), _i64(v.stride(0)), _i64(v.stride(1)), _i64(v.stride(2))]
    return a


def decode_f64(q, k, v, scale, block_idx=None, block_cnt=None, stats=False, load_v=True):
    """Double-precision attention of one decode step; dict(out, lse[, blk_max, blk_sum])."""
    if q.dim() == 4:
        q = q.squeeze(2)
    B, Hq, D = q.shape
    Hkv, T = k.shape[1], k.shape[2]
    nb = math.ceil(T / BLOCK)
    out = torch.empty(B, Hq, D, dtype=torch.float64) if load_v else None
    lse = torch.empty(B, Hq, dtype=torch.float64)
    bmax = torch.empty(B, Hq, nb, dtype=torch.float64) if stats else None
    bsum = torch.empty(B, Hq, nb, dtype=torch.float64) if stats else None
    if block_idx is not None:
        block_idx = block_idx.to(torch.int32).contiguous()
        block_cnt = block_cnt.to(torch.int32).contiguous()
    lib().kvo_decode_f64(*_qkv_args(q, k, v), _i(B), _i(Hq), _i(Hkv), _i(T), _i(D), _d(scale),
                         _p(block_idx), _p(block_cnt), _i(0 if block_idx is None else block_idx.shape[-1]),
                         _p(out), _p(lse), _p(bmax), _p(bsum))
    d = {"out": out, "lse": lse}
    if stats:
        d["blk_max"], d["blk_sum"] = bmax, bsum
    return d


def vskip1_f64(q, k, v, scale, tau=1e-4, local=2, lse_prev=None):
    if q.dim() == 4:
        q = q.squeeze(2)
    B, Hq, D = q.shape
    Hkv, T = k.shape[1], k.shape[2]
    nb = math.ceil(T / BLOCK)
    out = torch.empty(B, Hq, D, dtype=torch.float64)
    lse = torch.empty(B, Hq, dtype=torch.float64)
    vcount = torch.empty(B, Hkv, dtype=torch.int32)
    kept = torch.empty(B, Hkv, nb, dtype=torch.uint8)
    margin = torch.empty(B, Hkv, nb, dtype=torch.float64)
    if lse_prev is not None:
        lse_prev = lse_prev.float().contiguous()
    lib().kvo_vskip1_f64(*_qkv_args(q, k, v), _i(B), _i(Hq), _i(Hkv), _i(T), _i(D), _d(scale), _d(tau),
                         _i(local), _p(lse_prev), _p(out), _p(lse), _p(vcount), _p(kept), _p(margin))
    return {"out": out, "lse": lse, "v_tiles": vcount, "kept": kept.bool(), "margin": margin}


def pv_f64(P, v, blk_scale, block_idx, block_cnt):
    B, Hkv, T, D = v.shape
    Hq = P.shape[1]
    assert P.dtype == torch.float16 and P.is_contiguous() and v.stride(-1) == 1
    out = torch.empty(B, Hq, D, dtype=torch.float64)
    block_idx = block_idx.to(torch.int32).contiguous()
    block_cnt = block_cnt.to(torch.int32).contiguous()
    blk_scale = blk_scale.float().contiguous()
    lib().kvo_pv_f64(_p(P), _p(v), _i64(v.stride(0)), _i64(v.stride(1)), _i64(v.stride(2)), _p(blk_scale),
                     _p(block_idx), _p(block_cnt), _i(block_idx.shape[-1]), _i(B), _i(Hq), _i(Hkv), _i(T), _i(D),
                     _p(out))
    return out


def combine_f32(part_acc, part_ml):
    """part_acc [..., S, D], part_ml [..., S, 2] (m in log2 units, l) -> out [..., D], lse [...]."""
    part_acc = part_acc.float().contiguous()
    part_ml = part_ml.float().contiguous()
    S, D = part_acc.shape[-2], part_acc.shape[-1]
    N = part_acc.numel() // (S * D)
    out = torch.empty(*part_acc.shape[:-2], D, dtype=torch.float32)
    lse = torch.empty(part_acc.shape[:-2], dtype=torch.float32)
    lib().kvo_combine_f32(_p(part_acc), _p(part_ml), _i64(N), _i(S), _i(D), _p(out), _p(lse))
    return out, lse


def block_stats_f32(q, k, scale, want_scores=False):
    """Dense block statistics in the kernels' float operation order."""
    if q.dim() == 4:
        q = q.squeeze(2)
    B, Hq, D = q.shape
    Hkv, T = k.shape[1], k.shape[2]
    nb = math.ceil(T / BLOCK)
    bmax = torch.empty(B, Hq, nb, dtype=torch.float32)
    bsum = torch.empty(B, Hq, nb, dtype=torch.float32)
    sc = torch.full((B, Hq, nb * BLOCK), float("-inf"), dtype=torch.float32) if want_scores else None
    lib().kvo_block_stats_f32(*_qkv_args(q, k), _i(B), _i(Hq), _i(Hkv), _i(T), _i(D), _f(scale),
                              _p(bmax), _p(bsum), _p(sc))
    return (bmax, bsum, sc) if want_scores else (bmax, bsum)


def _chk(t, dtype, name):
    assert t.dtype == dtype and t.is_contiguous() and t.device.type == "cpu", name


def plan(q, k, csum, lse_ref, cs_ref, keep, lse_att, age, flags, cs_now, trig, block_idx, block_cnt,
         scale, delta, max_age, local, add_token, idx=None, calib=None, est=None, calib_on=False,
         calib_kind=0, aix=None, dec_margin=None):
    """Same arguments as the extension's plan(); state tensors are modified in place."""
    B, Hq, D = q.shape
    Hkv, T = k.shape[1], k.shape[2]
    assert D == 128 and Hq == 4 * Hkv
    NBC = keep.shape[2]
    assert math.ceil(T / BLOCK) <= NBC
    for t, dt, n in ((csum, torch.float32, "csum"), (lse_ref, torch.float32, "lse_ref"),
                     (cs_ref, torch.float32, "cs_ref"), (keep, torch.uint8, "keep"),
                     (lse_att, torch.float32, "lse_att"), (age, torch.int32, "age"),
                     (flags, torch.int32, "flags"), (cs_now, torch.float32, "cs_now"),
                     (trig, torch.uint8, "trig"), (block_idx, torch.int32, "block_idx"),
                     (block_cnt, torch.int32, "block_cnt")):
        _chk(t, dt, n)
    if aix is not None:
        assert idx is not None
    lib().kvo_plan_f32(*_qkv_args(q, k), _p(csum), _p(lse_ref), _p(cs_ref), _p(keep), _p(lse_att), _p(age),
                       _p(flags), _p(idx), _p(calib), _p(est), _i(bool(calib_on)), _i(calib_kind), _p(aix),
                       _p(cs_now), _p(trig), _p(block_idx), _p(block_cnt), _i(B), _i(Hq), _i(Hkv), _i(T),
                       _i(NBC), _i(local), _i(max_age), _i(bool(add_token)), _f(scale), _f(delta),
                       _p(dec_margin))


def update(blk_max, blk_sum, trig, cs_now, keep, lse_ref, cs_ref, lse_att, T, level, local, flags=None,
           idx=None, est=None, calib=None, calib_rate=0.0, calib_free=False, calib_kind=0, aix=None,
           aix_thr=0.0, topp_margin=None):
    """Same arguments as the extension's update(); state tensors are modified in place."""
    B, Hkv, NBC = keep.shape
    Hq = lse_att.shape[1]
    assert blk_max.shape[2] == math.ceil(T / BLOCK)
    _chk(blk_max, torch.float32, "blk_max")
    _chk(blk_sum, torch.float32, "blk_sum")
    if calib is not None:
        assert flags is not None and est is not None
    else:
        flags = idx = est = aix = None          # the extension ignores them without calibration
    lib().kvo_update_f32(_p(blk_max), _p(blk_sum), _p(trig), _p(cs_now), _p(keep), _p(lse_ref), _p(cs_ref),
                         _p(lse_att), _p(flags), _p(idx), _p(est), _p(calib), _f(calib_rate),
                         _i(bool(calib_free)), _i(calib_kind), _p(aix), _f(aix_thr), _i(B), _i(Hq), _i(Hkv),
                         _i(T), _i(NBC), _i(local), _f(level), _p(topp_margin))


def index_blocks(ids, T, n_out):
    """ids int64 [n, >= T]; returns uint8 [n, n_out] token-index blocks of the step whose current
    token sits at T - 1."""
    ids = ids.to(torch.int64)
    assert ids.stride(1) == 1
    out = torch.empty(ids.shape[0], n_out, dtype=torch.uint8)
    lib().kvo_index_blocks(_p(ids), _i64(ids.stride(0)), _i(ids.shape[0]), _i(T), _p(out), _i(n_out))
    return out


def select_topp(logw, G, level, local=2):
    logw = logw.double().contiguous()
    B, Hq, nb = logw.shape
    keep = torch.empty(B, Hq // G, nb, dtype=torch.uint8)
    lib().kvo_select_topp(_p(logw), _i(B), _i(Hq), _i(Hq // G), _i(nb), _d(level), _i(local), _p(keep))
    return keep.bool()
