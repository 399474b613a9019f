"""`kernels.kvskip` of the reference layout: re-exports kvskip_b200.kvskip (same names)."""
from kvskip_b200.kvskip import *  # noqa: F401,F403
from kvskip_b200.kvskip import (TILE, Plan, always_keep, block_weights, decode, ext, make_plan,  # noqa: F401
                                num_sms, num_splits_for, pv, select_blocks, vskip_one_pass, vskip_two_pass)
