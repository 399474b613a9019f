"""kvskip_b200: decode attention of format37/kvskip (split-K flash-decoding in dense, masked
block-list, block-statistics and V-skip variants, split merge, device-side refresh planner)
written for NVIDIA B200 (sm_100a).

    from kvskip_b200 import kvskip      # same surface as the reference's kernels/kvskip.py
    kvskip.decode(q, k, v, scale)

The C ABI lives in include/kvskip_b200.h / libkvskip_b200.so; `kvskip.ext()` is the PyTorch front
of it.  There is no CPU implementation in this package.
"""
from . import kvskip  # noqa: F401

__version__ = "0.1.0"
