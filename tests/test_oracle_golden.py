"""Pins the CPU oracle to golden vectors produced by the reference's own Python code
(tests/golden/make_golden.py).  No GPU needed."""
import math

import numpy as np
import pytest
import torch

import oracle
from kvskip_b200 import synth
from kvskip_b200.refresh import RefreshConfig, RefreshLayer
from helpers import OracleOps, rel_err, unpack_masks


@pytest.fixture(scope="module")
def dg(golden_dir):
    return np.load(golden_dir / "decode_golden.npz")


def test_decode_f64_config1_dense_and_masked(dg):
    q, k, v, scale, keep = synth.sink_body_case(int(dg["c1_seed"]), int(dg["c1_T"]))
    assert np.array_equal(keep.numpy(), dg["c1_keep"])
    r = oracle.decode_f64(q, k, v, scale, stats=True)
    assert rel_err(r["out"], torch.from_numpy(dg["c1_dense_out"])) < 1e-12
    assert np.allclose(r["blk_max"].numpy(), dg["c1_blk_max"], rtol=0, atol=1e-12)
    assert np.allclose(r["blk_sum"].numpy(), dg["c1_blk_sum"], rtol=1e-12)
    bi, bc = synth.keep_to_plan(keep)
    assert np.array_equal(bi.numpy(), dg["c1_plan_idx"]) and np.array_equal(bc.numpy(), dg["c1_plan_cnt"])
    m = oracle.decode_f64(q, k, v, scale, bi, bc, stats=True)
    assert rel_err(m["out"], torch.from_numpy(dg["c1_masked_out"])) < 1e-12
    kq = keep.repeat_interleave(4, dim=1)
    assert torch.isinf(m["blk_max"][~kq]).all() and (m["blk_sum"][~kq] == 0).all()
    assert torch.equal(m["blk_max"][kq], r["blk_max"][kq])
    # lse is the log-sum-exp of the block log-weights over the blocks read
    logw = (r["blk_max"] + torch.log(r["blk_sum"])).masked_fill(~kq, float("-inf"))
    assert torch.allclose(m["lse"], torch.logsumexp(logw, -1), rtol=0, atol=1e-10)


@pytest.mark.parametrize("i", range(5))
def test_decode_f64_edge_cases(dg, i):
    D, T, seed = int(dg[f"edge{i}_D"]), int(dg[f"edge{i}_T"]), int(dg[f"edge{i}_seed"])
    q, k, v, scale = synth.sink_case(seed, 2, T, D)
    r = oracle.decode_f64(q, k, v, scale, stats=True)
    assert rel_err(r["out"], torch.from_numpy(dg[f"edge{i}_out"])) < 1e-12
    assert np.allclose(r["blk_max"].numpy(), dg[f"edge{i}_blk_max"], rtol=0, atol=1e-11)
    assert np.allclose(r["blk_sum"].numpy(), dg[f"edge{i}_blk_sum"], rtol=1e-11)


def test_block_stats_f32_order_close_to_f64(dg):
    q, k, v, scale, _ = synth.sink_body_case(int(dg["c1_seed"]), int(dg["c1_T"]))
    bmax, bsum = oracle.block_stats_f32(q, k, scale)
    assert np.abs(bmax.double().numpy() - dg["c1_blk_max"]).max() < 2e-5
    assert np.abs(bsum.double().numpy() / dg["c1_blk_sum"] - 1).max() < 2e-5


def test_select_topp_matches_reference(dg):
    logw = torch.from_numpy(dg["c1_blk_max"] + np.log(dg["c1_blk_sum"])).float()
    assert np.array_equal(oracle.select_topp(logw, 4, 0.99, 2).numpy(), dg["c1_topp099"])
    assert np.array_equal(oracle.select_topp(logw, 4, 0.90, 2).numpy(), dg["c1_topp090"])


def test_combine_f32_equals_unsplit():
    torch.manual_seed(0)
    N, S, D = 6, 5, 128
    m = torch.randn(N, S) * 3
    l = torch.rand(N, S) + 0.1
    acc = torch.randn(N, S, D)
    m[0, 2] = float("-inf"); l[0, 2] = 0; acc[0, 2] = 0          # an empty split
    out, lse = oracle.combine_f32(acc, torch.stack([m, l], -1))
    M = m.double().amax(-1, keepdim=True)
    w = torch.exp2(m.double() - M)
    L = (l.double() * w).sum(-1)
    ref = (acc.double() * w[..., None]).sum(1) / L[:, None]
    assert rel_err(out, ref) < 1e-6
    assert torch.allclose(lse.double(), (M[:, 0] + torch.log2(L)) * math.log(2), atol=1e-5)


def test_vskip1_rule_matches_reference_fp64(golden_dir):
    g = np.load(golden_dir / "vskip_golden.npz")
    q, k, v, scale, _ = synth.body_union_case(int(g["seed"]), int(g["T"]))
    for tau in (1e-4, 1e-3):
        r = oracle.vskip1_f64(q, k, v, scale, tau=tau, local=2)
        assert np.array_equal(r["kept"].numpy(), g[f"sink_keep_{tau:g}"])
        assert rel_err(r["out"], torch.from_numpy(g[f"sink_out_{tau:g}"])) < 1e-12
        assert np.array_equal(r["v_tiles"].numpy(), g[f"sink_keep_{tau:g}"].sum(-1))
        r2 = oracle.vskip1_f64(q, k, v, scale, tau=tau, local=2, lse_prev=torch.from_numpy(g["lse_exact"]))
        assert np.array_equal(r2["kept"].numpy(), g[f"prev_keep_{tau:g}"])
        assert rel_err(r2["out"], torch.from_numpy(g[f"prev_out_{tau:g}"])) < 1e-12
        # the planted background must actually be skipped, or the case tests nothing
        assert 0.3 < r2["kept"].float().mean() < 0.8


def test_index_blocks_matches_reference(golden_dir):
    g = np.load(golden_dir / "index_golden.npz")
    P, S = int(g["P"]), int(g["S"])
    ids = synth.token_ids_with_repeats(int(g["seed"]), 3, P + S, vocab=int(g["vocab"]), repeat_p=float(g["repeat_p"]))
    nbm = g["blocks"].shape[-1]
    for t in range(S):
        T = P + t + 1
        got = oracle.index_blocks(ids, T, nbm).numpy().astype(bool)
        assert np.array_equal(got, g["blocks"][t]), t
        assert np.array_equal(synth.index_blocks(ids, T, nbm).numpy().astype(bool), g["blocks"][t]), t


VARIANTS = {
    "plain": dict(dense_heads=(6,)),
    "union": dict(dense_heads=(6,), index_heads=(2,), index_union=True),
    "only": dict(dense_heads=(6,), index_heads=(2,), index_union=False),
    "peak_auto": dict(calib=0.05, calib_warm=(32, 8), calib_kind="peak", calib_auto_ix=0.001),
    "logit": dict(calib=0.3, calib_warm=(32, 8), calib_kind="logit"),
    "add_union": dict(calib=0.3, calib_warm=(32, 8), calib_kind="add", index_heads=(2,), index_union=True),
}


@pytest.mark.parametrize("name", list(VARIANTS))
def test_planner_loop_matches_python_planner(golden_dir, name):
    """The float restatement of plan/update, driven by the host-side refresh driver, reads the same
    blocks on every head-step as the reference's Python planner, and ends in the same state."""
    g = np.load(golden_dir / "planner_golden.npz")
    T0, steps, B, nbm = int(g["T0"]), int(g["steps"]), int(g["B"]), int(g["nb_max"])
    walk = synth.planner_walk(int(g["seed"]), T0, steps, B=B)
    ids = synth.token_ids_with_repeats(int(g["seed"]) + 1, B, T0 + steps)
    masks = unpack_masks(g[f"{name}_masks"], nbm)
    layer = RefreshLayer(RefreshConfig(**VARIANTS[name]), ops=OracleOps())
    agree = total = 0
    for t in range(steps):
        Tt = T0 + t + 1
        nb = math.ceil(Tt / 64)
        idx = synth.index_blocks(ids, Tt, nb) if layer.uses_index() else None
        out = layer.step(walk.q[t], walk.k[:, :, :Tt], walk.v[:, :, :Tt], walk.scale, idx)
        got = np.ones((B, 8, nb), bool) if t == 0 else layer.read_mask(nb).numpy()
        same = (got == masks[t, :, :, :nb]).all(-1)
        agree += int(same.sum())
        total += same.size
        if same.all():
            n = out.float().norm(dim=-1).numpy()
            assert np.allclose(n, g[f"{name}_out_norms"][t], rtol=2e-2), t
    assert agree == total, f"{name}: identical read sets on {agree}/{total} head-steps"
    s = layer.state
    nb = math.ceil((T0 + steps) / 64)
    assert np.array_equal(s["keep"][..., :nb].numpy().astype(bool), g[f"{name}_keep"][..., :nb])
    # an index-only head leaves `plan` before its age is touched (the device kernel keeps it stale by
    # design, kernels/kvskip_planner.cu:87-107) while the Python planner keeps counting
    live = [h for h in range(8) if not (VARIANTS[name].get("index_heads") == (h,) and not VARIANTS[name].get("index_union"))]
    assert np.array_equal(s["age"].numpy()[:, live], g[f"{name}_age"][:, live])
    assert np.array_equal(s["aix"].numpy().astype(bool), g[f"{name}_aix"])
    assert np.allclose(s["calib"].numpy(), g[f"{name}_calib"][-1], rtol=0, atol=1e-5)
    assert np.allclose(s["lse_att"].numpy(), g[f"{name}_lse_att"], rtol=0, atol=1e-5)
