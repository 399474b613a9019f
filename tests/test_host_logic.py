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


def test_graph_scalars_follow_the_step_counter():
    """The scalars a captured step freezes are those the next step would pass to the kernels: the
    maximum age of the warm-up period and whether the correction is applied yet."""
    from kvskip_b200.refresh import RefreshConfig, RefreshLayer
    layer = RefreshLayer(RefreshConfig(calib=0.05, calib_warm=(4, 8), calib_hold=6, max_age=32), ops=object())
    seen = []
    for _ in range(8):
        seen.append(layer.graph_scalars())
        layer.note_replayed()
        assert layer.max_age_now() == seen[-1][0]
        assert (layer.t >= 6) == seen[-1][1]
    assert seen[0] == (8, False) and seen[2] == (8, False) and seen[3] == (32, False) and seen[5] == (32, True)
    assert RefreshLayer(RefreshConfig(), ops=object()).graph_scalars() == (32, False)


def test_step_graph_runs_eager_steps_before_capturing(monkeypatch):
    """StepGraph's bookkeeping with the CUDA graph replaced by a recorder: eager steps first, one
    capture per distinct set of host-decided scalars, the layers' counters advanced on replays."""
    import torch
    from kvskip_b200 import graph as G

    class FakeGraph:
        def __init__(self):
            self.fn = None

        def replay(self):
            calls.append("replay")

    class FakeCapture:
        def __init__(self, g, **kw):
            pass

        def __enter__(self):
            calls.append("capture")

        def __exit__(self, *a):
            return False

    class Layer:
        t = 0

        def graph_scalars(self):
            return (8 if self.t + 1 < 4 else 32,)

        def note_replayed(self):
            self.t += 1

    calls, layer = [], Layer()

    def launch():
        layer.t += 1
        calls.append("launch")
        return layer.t

    monkeypatch.setattr(torch.cuda, "CUDAGraph", FakeGraph)
    monkeypatch.setattr(torch.cuda, "graph", FakeCapture)
    g = G.StepGraph(launch, [layer], eager=2)
    assert not g.will_capture()
    for _ in range(7):
        g.step()
    assert layer.t == 7 and g.captures == 2 and g.replays == 5
    assert calls == ["launch", "launch", "capture", "launch", "replay", "capture", "launch", "replay", "replay", "replay",
                     "replay"]


def test_paged_cache_bookkeeping_on_cpu():
    """Page hand-out, prefill scatter and gather of PagedKV need no GPU (the append kernel does)."""
    import torch
    from kvskip_b200.cache import PagedKV
    B, H, D, T = 3, 2, 16, 150
    g = torch.Generator().manual_seed(0)
    k = torch.randn(B, H, T, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, H, T, D, generator=g).to(torch.bfloat16)
    pg = PagedKV(B * 4 + 2, B, H, D, 256, "cpu", order="shuffled", seed=1)
    pg.write(k, v)
    used = pg.table_host[:, :3].reshape(-1).tolist()
    assert len(set(used)) == B * 3 and (pg.table_host[:, 3:] == -1).all()       # distinct pages, none beyond
    gk, gv = pg.gather()
    assert torch.equal(gk, k) and torch.equal(gv, v)
    pg.reserve(256)
    assert (pg.table_host >= 0).all() and len(set(pg.table_host.reshape(-1).tolist())) == B * 4
    for _ in range(256 - T):
        pg.note_replayed()
    assert pg.get_seq_length() == 256
    import pytest
    with pytest.raises(RuntimeError, match="reserved"):
        pg.note_replayed()
    with pytest.raises(RuntimeError, match="exceed"):
        pg.reserve(257)
    small = PagedKV(2, B, H, D, 256, "cpu")
    with pytest.raises(RuntimeError, match="exhausted"):
        small.reserve(64)


def test_pv_splits_is_one_wave_of_pieces_of_at_least_16_blocks():
    """Split rule of the two-pass V-skip's second pass: as many pieces per (batch, kv head) as keep
    the grid within the SM count, none shorter than 16 blocks, at least one."""
    from kvskip_b200 import kvskip as K
    assert K.pv_splits(8, 1024, sms=148) == 18
    assert K.pv_splits(32, 1024, sms=148) == 4
    assert K.pv_splits(64, 1024, sms=148) == 2
    assert K.pv_splits(128, 512, sms=148) == 1
    assert K.pv_splits(1000, 512, sms=148) == 1
    assert K.pv_splits(8, 20, sms=148) == 2
    assert K.pv_splits(8, 1, sms=148) == 1
    for bh in (1, 7, 8, 33, 148, 149):
        for cnt in (1, 15, 16, 17, 500, 4096):
            s_ = K.pv_splits(bh, cnt, sms=148)
            assert s_ >= 1 and (s_ == 1 or (bh * s_ <= 148 and (s_ - 1) * 16 < cnt))

