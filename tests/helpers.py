"""Shared by the CPU and GPU tests: oracle-backed stand-ins and comparison helpers."""
import math

import numpy as np
import torch

import oracle
from kvskip_b200 import kvskip as K


def rel_err(x, ref) -> float:
    """Norm-wise relative error, the reference's own criterion (bench/harness.py:134-135)."""
    x = x.double().cpu()
    ref = ref.double().cpu()
    return float((x - ref).norm() / ref.norm())


def unpack_masks(packed, nb_max):
    return np.unpackbits(packed, axis=-1)[..., :nb_max].astype(bool)


class OracleOps:
    """CPU stand-in for the extension inside kvskip_b200.refresh.RefreshLayer: attention in
    double precision, block statistics and planner in the kernels' float operation order."""

    def decode(self, q, k, v, scale, plan=None, stats=False):
        bi, bc = (None, None) if plan is None else (plan.block_idx, plan.block_cnt)
        r = oracle.decode_f64(q, k, v, scale, bi, bc, stats=False)
        d = {"out": r["out"].to(torch.bfloat16), "lse": r["lse"].float(), "out_f64": r["out"]}
        if stats:
            bmax, bsum = oracle.block_stats_f32(q, k, scale)
            if plan is not None:
                B, Hq, nb = bmax.shape
                G = Hq // k.shape[1]
                n = bi.shape[-1]
                valid = torch.arange(n)[None, None, :] < bc[..., None]
                m = torch.zeros(B, k.shape[1], n + 1, dtype=torch.bool)
                m.scatter_(-1, torch.where(valid, bi.long(), n), True)
                read = m[..., :nb].repeat_interleave(G, dim=1)
                bmax = bmax.masked_fill(~read, float("-inf"))
                bsum = bsum.masked_fill(~read, 0.0)
            d["blk_max"], d["blk_sum"] = bmax, bsum
        return d

    def plan(self, *a):
        return oracle.plan(*a)

    def update(self, *a):
        return oracle.update(*a)
