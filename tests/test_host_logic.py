"""Host-side logic that needs no GPU: split heuristic, plans, selectors, the alias package."""
import numpy as np
import torch

from kvskip_b200 import kvskip as K


def test_split_heuristic_matches_reference_table(golden_dir):
    g = np.load(golden_dir / "decode_golden.npz")
    for i, bh in enumerate(g["splits_bh"]):
        for j, nt in enumerate(g["splits_tiles"]):
            assert K.num_splits_for(int(bh), int(nt), sms=148) == int(g["splits_148"][i, j]), (bh, nt)
    assert K.num_splits_for(8, 1024, sms=148) == 18      # batch 1, 64k context on a B200
    assert K.num_splits_for(8, 3, sms=148) == 1          # never fewer than 4 blocks per split


def test_selectors_and_plan_match_reference(golden_dir):
    g = np.load(golden_dir / "decode_golden.npz")
    logw = torch.from_numpy(g["c1_blk_max"] + np.log(g["c1_blk_sum"])).float()
    assert np.array_equal(K.select_blocks(logw, 4, "topp", 0.99, 2).numpy(), g["c1_topp099"])
    assert np.array_equal(K.select_blocks(logw, 4, "topp", 0.90, 2).numpy(), g["c1_topp090"])
    assert np.array_equal(K.select_blocks(logw, 4, "tau", 1e-3, 2).numpy(), g["c1_tau1e3"])
    plan = K.make_plan(torch.from_numpy(g["c1_keep"]))
    assert np.array_equal(plan.block_idx.numpy(), g["c1_plan_idx"])
    assert np.array_equal(plan.block_cnt.numpy(), g["c1_plan_cnt"])
    assert plan.max_cnt == int(g["c1_plan_max"]) and plan.nb == 64
    assert K.make_plan(torch.from_numpy(g["c1_keep"]), sync=False).max_cnt == 64
    a = K.always_keep(10, 2, "cpu")
    assert a.tolist() == [True] + [False] * 7 + [True, True]


def test_reference_import_path_resolves_here():
    from kernels import kvskip as alias
    assert alias.decode is K.decode and alias.Plan is K.Plan and alias.TILE == 64
    for name in ("ext", "num_sms", "num_splits_for", "make_plan", "block_weights", "always_keep", "select_blocks",
                 "pv", "vskip_two_pass", "vskip_one_pass"):
        assert hasattr(alias, name)
