"""Caches either side of the kernels: the growing contiguous cache and the paged one.

A paged launch must give bit for bit what the contiguous launch gives on the same tokens (same
kernel, same arithmetic, only the addresses differ), with the pool's pages handed out in shuffled
order and stale NaN in every page row that holds no token."""
import math

import pytest
import torch

import oracle
from kvskip_b200 import kvskip as K
from kvskip_b200 import synth
from kvskip_b200.cache import GrowingKV, PagedKV
from kvskip_b200.graph import StepGraph
from kvskip_b200.refresh import RefreshConfig, RefreshLayer

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _paged_from(k, v, T, max_tokens, seed=0, spare=7):
    B, H, _, D = k.shape
    pg = PagedKV(B * math.ceil(max_tokens / 64) + spare, B, H, D, max_tokens, DEV, order="shuffled", seed=seed)
    pg.k.fill_(float("nan"))
    pg.v.fill_(float("nan"))
    pg.write(k[:, :, :T], v[:, :, :T])
    nb, r = math.ceil(T / 64), T % 64
    if r:                                            # rows past T in the last pages: back to NaN
        last = pg.table[:, nb - 1].long()
        pg.k[last, :, r:] = float("nan")
        pg.v[last, :, r:] = float("nan")
    return pg


def test_growing_cache_matches_reference_behaviour():
    B, H, D = 2, 8, 128
    g = torch.Generator().manual_seed(0)
    c = GrowingKV(capacity=256)
    k0 = torch.randn(B, H, 100, D, generator=g).to(torch.bfloat16).to(DEV)
    v0 = torch.randn(B, H, 100, D, generator=g).to(torch.bfloat16).to(DEV)
    ks, vs = c.update(k0, v0)
    assert ks.shape[2] == 100 and c.full()[0].shape[2] == 640 and torch.equal(ks, k0)      # ceil((100+512)/64)*64
    rows_k, rows_v = [k0], [v0]
    for _ in range(600):                               # crosses one re-allocation (doubling)
        kn = torch.randn(B, H, 1, D, generator=g).to(torch.bfloat16).to(DEV)
        vn = torch.randn(B, H, 1, D, generator=g).to(torch.bfloat16).to(DEV)
        ks, vs = c.update(kn, vn)
        rows_k.append(kn)
        rows_v.append(vn)
    assert c.get_seq_length() == 700 and c.full()[0].shape[2] == 1280
    assert torch.equal(ks, torch.cat(rows_k, 2)) and torch.equal(vs, torch.cat(rows_v, 2))
    c.crop(-50)
    assert c.get_seq_length() == 650 and c.views()[0].shape[2] == 650
    c.crop(600)
    assert c.get_seq_length() == 600


@pytest.mark.parametrize("T", [1, 64, 65, 1000, 1471])
def test_paged_dense_and_masked_match_contiguous(T):
    cap, B, Hkv = 1536, 2, 8
    q, k, v, scale = synth.dense_case(900 + T, B, cap)
    q, k, v = q.to(DEV), k.to(DEV), v.to(DEV)
    pg = _paged_from(k, v, T, cap, seed=T)
    gk, gv = pg.gather()
    assert torch.equal(gk, k[:, :, :T]) and torch.equal(gv, v[:, :, :T])
    nb = math.ceil(T / 64)
    for splits in (1, 3):
        a = K.decode(q, k[:, :, :T], v[:, :, :T], scale, stats=True, out_f32=True, num_splits=splits)
        b = K.decode(q, pg.k, pg.v, scale, stats=True, out_f32=True, num_splits=splits, page_table=pg.table, seq_len=T)
        assert torch.equal(a["out_f32"], b["out_f32"]) and torch.equal(a["lse"], b["lse"])
        assert torch.equal(a["blk_max"], b["blk_max"]) and torch.equal(a["blk_sum"], b["blk_sum"])
        assert torch.isfinite(b["out_f32"]).all()
    if nb >= 3:
        keep = torch.rand(B, Hkv, nb, generator=torch.Generator().manual_seed(T)) < 0.4
        keep[..., 0] = True
        keep[..., -1] = True
        plan = K.make_plan(keep.to(DEV))
        a = K.decode(q, k[:, :, :T], v[:, :, :T], scale, plan=plan, stats=True, out_f32=True)
        b = K.decode(q, pg.k, pg.v, scale, plan=plan, stats=True, out_f32=True, page_table=pg.table, seq_len=T)
        assert torch.equal(a["out_f32"], b["out_f32"]) and torch.equal(a["lse"], b["lse"])
        assert torch.equal(a["blk_max"], b["blk_max"]) and torch.equal(a["blk_sum"], b["blk_sum"])
        # the paged launch against the CPU oracle on the gathered sequence
        bi, bc = synth.keep_to_plan(keep)
        ref = oracle.decode_f64(q.cpu(), gk.cpu(), gv.cpu(), scale, bi, bc)
        assert float((b["out_f32"].double().cpu() - ref["out"]).norm() / ref["out"].norm()) < 5e-5
        assert torch.allclose(b["lse"].double().cpu(), ref["lse"], rtol=0, atol=2e-4)
    ref = oracle.decode_f64(q.cpu(), gk.cpu(), gv.cpu(), scale)
    paged = K.decode(q, pg.k, pg.v, scale, out_f32=True, page_table=pg.table, seq_len=T)
    assert float((paged["out_f32"].double().cpu() - ref["out"]).norm() / ref["out"].norm()) < 5e-5
    assert float((paged["out"].double().cpu() - ref["out"]).norm() / ref["out"].norm()) < 2e-3
    # with the length on the device as well
    t_dev = torch.tensor([T], dtype=torch.int32, device=DEV)
    c = K.decode(q, pg.k, pg.v, scale, out_f32=True, num_splits=3, page_table=pg.table, seq_len=cap, t_dev=t_dev)
    d = K.decode(q, k[:, :, :T], v[:, :, :T], scale, out_f32=True, num_splits=3)
    assert torch.equal(c["out_f32"], d["out_f32"]) and torch.equal(c["lse"], d["lse"])


def test_paged_refuses_what_it_does_not_support():
    q, k, v, scale = synth.dense_case(1, 1, 256)
    pg = _paged_from(k.to(DEV), v.to(DEV), 200, 256)
    with pytest.raises(ValueError, match="seq_len"):
        K.decode(q.to(DEV), pg.k, pg.v, scale, page_table=pg.table)
    with pytest.raises(RuntimeError, match="one entry per 64-token block"):
        K.decode(q.to(DEV), pg.k, pg.v, scale, page_table=pg.table[:, :2], seq_len=200)
    K.ext().set_option("decode_path", 1)
    try:
        with pytest.raises(RuntimeError, match="tensor-core path"):
            K.decode(q.to(DEV), pg.k, pg.v, scale, page_table=pg.table, seq_len=200)
    finally:
        K.ext().set_option("decode_path", 0)


@pytest.mark.parametrize("graph", [False, True], ids=["launches", "captured"])
def test_planner_loop_on_a_paged_cache_matches_contiguous(graph):
    """30 decode steps: tokens appended to a growing contiguous cache and to a shuffled page pool,
    the refresh policy on both; outputs and planner state identical after every step.  In the
    captured form the append, the token index and the three kernels replay from one graph."""
    T0, steps, B = 2048 - 10, 30, 2
    walk = synth.planner_walk(31, T0, steps, B=B)
    ids = synth.token_ids_with_repeats(12, B, T0 + steps).to(DEV)
    kc, vc, qc = walk.k.to(DEV), walk.v.to(DEV), walk.q.to(DEV)
    cap = T0 + steps
    cfg = RefreshConfig(calib=0.05, calib_kind="peak", calib_auto_ix=0.001, max_age=8)
    la, lb = RefreshLayer(cfg), RefreshLayer(cfg)
    cont = GrowingKV()
    cont.update(kc[:, :, :T0], vc[:, :, :T0])
    pg = _paged_from(kc, vc, T0, cap, seed=3)
    pg.reserve(cap)
    nbc = math.ceil((T0 + 1) / 64) + cfg.margin
    idx = torch.zeros(B, nbc, dtype=torch.uint8, device=DEV)
    idx_g = torch.zeros(B, nbc, dtype=torch.uint8, device=DEV)
    t_dev = torch.tensor([T0], dtype=torch.int32, device=DEV)
    q_buf = torch.zeros_like(qc[0])
    kn_buf = torch.zeros(B, 8, 128, dtype=torch.bfloat16, device=DEV)
    vn_buf = torch.zeros_like(kn_buf)

    def launch():
        K.ext().advance(t_dev, 1)
        pg.append(kn_buf, vn_buf, t_dev=t_dev)
        K.ext().index_blocks(ids, cap, idx_g, t_dev)
        return lb.step(q_buf, pg.k, pg.v, walk.scale, idx_g, t_dev=t_dev, page_table=pg.table, seq_len=cap)

    g = StepGraph(launch, [lb, pg], eager=1)
    for t in range(steps):
        T = T0 + t + 1
        kn, vn = kc[:, :, T - 1].contiguous(), vc[:, :, T - 1].contiguous()
        ks, vs = cont.update(kn.unsqueeze(2), vn.unsqueeze(2))
        K.ext().index_blocks(ids, T, idx)
        oa = la.step(qc[t], ks, vs, walk.scale, idx)
        if t == 0:          # state is built on the host from contiguous views
            pg.append(kn, vn)
            K.ext().advance(t_dev, 1)
            ob = lb.step(qc[t], ks, vs, walk.scale, idx)
        elif graph:
            q_buf.copy_(qc[t]); kn_buf.copy_(kn); vn_buf.copy_(vn)
            ob = g.step()
        else:
            pg.append(kn, vn)
            K.ext().advance(t_dev, 1)
            ob = lb.step(qc[t], pg.k, pg.v, walk.scale, idx, page_table=pg.table, seq_len=T)
        assert pg.get_seq_length() == T and int(t_dev) == T
        assert torch.equal(oa, ob), f"output differs at step {t}"
        for key in ("trig", "block_cnt", "age", "keep", "aix", "calib", "est", "lse_att", "cs_now", "lse_ref", "cs_ref",
                    "csum"):
            assert torch.equal(la.state[key], lb.state[key]), f"{key} differs at step {t}"
    gk, gv = pg.gather()
    assert torch.equal(gk, kc[:, :, :T0 + steps]) and torch.equal(gv, vc[:, :, :T0 + steps])
    assert K.ext().device_status() == 0


def test_dyn_and_paged_entry_points_through_ctypes():
    """The C ABI itself (no PyTorch binding in between): kvskip_launch_decode_dyn / _decode_paged /
    _append / _advance give what the by-value launch gives."""
    from kvskip_b200.cabi import CAbi
    abi = CAbi()
    cap, B, T = 1024, 2, 700
    q, k, v, scale = synth.dense_case(77, B, cap)
    q, k, v = q.to(DEV), k.to(DEV), v.to(DEV)
    ref = abi.decode(q, k[:, :, :T], v[:, :, :T], scale, stats=True, num_splits=4, want_f32=True)
    t_dev = torch.tensor([T - 1], dtype=torch.int32, device=DEV)
    abi.advance(t_dev, 1)
    dyn = abi.decode(q, k, v, scale, stats=True, num_splits=4, want_f32=True, t_dev=t_dev)
    nb = math.ceil(T / 64)
    assert torch.equal(ref[4], dyn[4]) and torch.equal(ref[1], dyn[1]) and torch.equal(ref[2], dyn[2][..., :nb])
    pg = _paged_from(k, v, T - 1, cap, seed=5)
    pg.reserve(T)
    abi.append(pg.k, pg.v, k[:, :, T - 1].contiguous(), v[:, :, T - 1].contiguous(), cap, t_dev=t_dev, page_table=pg.table)
    paged = abi.decode(q, pg.k, pg.v, scale, stats=True, num_splits=4, want_f32=True, page_table=pg.table, seq_len=T)
    assert torch.equal(ref[4], paged[4]) and torch.equal(ref[1], paged[1]) and torch.equal(ref[2], paged[2])
    kc, vc = k.clone(), v.clone()
    kc[:, :, T - 1] = 0
    abi.append(kc, vc, k[:, :, T - 1].contiguous(), v[:, :, T - 1].contiguous(), T)
    assert torch.equal(kc, k) and torch.equal(vc, v)


@pytest.mark.parametrize("T", [4096, 4000])
def test_paged_single_pass_vskip_matches_contiguous(T):
    """The single-pass V-skip over a shuffled page pool with NaN in every unused page row: same
    votes, same outputs as over the contiguous cache."""
    q, k, v, scale, _ = synth.body_union_case(5, 4096)
    q, k, v = q.to(DEV), k.to(DEV), v.to(DEV)
    pg = _paged_from(k, v, T, 4096, seed=T)
    lse = K.decode(q, k[:, :, :T], v[:, :, :T], scale)["lse"]
    for prev in (None, lse):
        for splits in (1, 5):
            a = K.vskip_one_pass(q, k[:, :, :T], v[:, :, :T], scale, tau=1e-4, lse_prev=prev, num_splits=splits,
                                 out_f32=True, count=True)
            b = K.vskip_one_pass(q, pg.k, pg.v, scale, tau=1e-4, lse_prev=prev, num_splits=splits, out_f32=True,
                                 count=True, page_table=pg.table, seq_len=T)
            assert torch.equal(a["v_tiles"], b["v_tiles"]) and 0 < a["kept_frac"] < 1
            assert torch.equal(a["out_f32"], b["out_f32"]) and torch.equal(a["lse"], b["lse"])
            assert torch.isfinite(b["out_f32"]).all()
