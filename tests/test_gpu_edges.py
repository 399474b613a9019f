"""More shapes for the GPU kernels: tiny and ragged contexts, other head counts, strided views with
block lists, very long contexts (planner beyond the reference's 3072-block limit), both paths."""
import math

import pytest
import torch

import oracle
from kvskip_b200 import kvskip as K
from kvskip_b200 import synth
from kvskip_b200.refresh import RefreshConfig, RefreshLayer
from helpers import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL_BF16, TOL_F32 = 2e-3, 5e-5


@pytest.fixture(params=["auto", "exact"], autouse=True)
def path(request):
    K.ext().set_option("decode_path", 1 if request.param == "exact" else 0)
    yield request.param
    K.ext().set_option("decode_path", 0)


@pytest.mark.parametrize("T", [1, 2, 63, 64, 65, 127, 129, 6 * 64, 6 * 64 + 1, 13 * 64 - 1])
@pytest.mark.parametrize("splits", [1, 3])
def test_tiny_and_ragged_contexts(T, splits):
    q, k, v, scale = synth.dense_case(200 + T, 3, T)
    ref = oracle.decode_f64(q, k, v, scale, stats=True)
    r = K.decode(q.to(DEV), k.to(DEV), v.to(DEV), scale, num_splits=splits, stats=True, out_f32=True)
    assert rel_err(r["out_f32"], ref["out"]) < TOL_F32 and rel_err(r["out"], ref["out"]) < TOL_BF16
    assert torch.allclose(r["lse"].double().cpu(), ref["lse"], rtol=0, atol=2e-4)
    assert (r["blk_max"].double().cpu() - ref["blk_max"]).abs().max() < 2e-5
    assert ((r["blk_sum"].double().cpu() - ref["blk_sum"]) / ref["blk_sum"]).abs().max() < 2e-5


@pytest.mark.parametrize("Hkv", [1, 2, 5])
def test_other_head_counts_and_strided_views_with_lists(Hkv):
    """Hq = 4*Hkv for a few Hkv; K/V as views into a larger cache in token-major memory layout;
    a block list on top."""
    B, T, cap = 2, 1500, 2048
    q, k, v, scale = synth.dense_case(300 + Hkv, B, cap, Hq=4 * Hkv, Hkv=Hkv)
    kc = k.to(DEV).transpose(1, 2).contiguous().transpose(1, 2)[:, :, :T]     # [B,T,Hkv,D] memory, view of length T
    vc = v.to(DEV).transpose(1, 2).contiguous().transpose(1, 2)[:, :, :T]
    nb = math.ceil(T / 64)
    keep = torch.rand(B, Hkv, nb, generator=torch.Generator().manual_seed(Hkv)) < 0.5
    keep[..., -1] = True
    bi, bc = synth.keep_to_plan(keep)
    ref = oracle.decode_f64(q, k[:, :, :T], v[:, :, :T], scale, bi, bc, stats=True)
    for splits in (None, 1, 4):
        r = K.decode(q.to(DEV), kc, vc, scale, plan=K.make_plan(keep.to(DEV)), stats=True, out_f32=True,
                     num_splits=splits)
        assert rel_err(r["out_f32"], ref["out"]) < TOL_F32
        fin = torch.isfinite(ref["blk_max"])
        assert torch.equal(torch.isfinite(r["blk_max"]).cpu(), fin)
        assert (r["blk_max"].double().cpu()[fin] - ref["blk_max"][fin]).abs().max() < 2e-5
        assert (r["blk_sum"].cpu()[~fin] == 0).all()
    rv = K.vskip_one_pass(q.to(DEV), kc, vc, scale, tau=1e-3, out_f32=True, count=True)
    refv = oracle.vskip1_f64(q, k[:, :, :T], v[:, :, :T], scale, tau=1e-3)
    border = (refv["margin"].abs() < 1e-3).sum(-1)
    assert ((rv["v_tiles"].cpu() - refv["v_tiles"]).abs() <= border).all()
    if int(border.sum()) == 0:
        assert rel_err(rv["out_f32"], refv["out"]) < TOL_F32


def test_unsynced_plan_with_one_full_head():
    """Lists of very different lengths under one split count sized for every block (what the fused
    planner step produces): a head that reads everything next to heads that read a tenth."""
    q, k, v, scale = synth.dense_case(17, 2, 16384)
    nb = 256
    keep = torch.rand(2, 8, nb, generator=torch.Generator().manual_seed(3)) < 0.1
    keep[:, 0] = True
    keep[1, 5] = False                                        # and an empty one
    bi, bc = synth.keep_to_plan(keep)
    ref = oracle.decode_f64(q, k, v, scale, bi, bc, stats=True)
    plan = K.make_plan(keep.to(DEV), sync=False)
    for splits in (None, 16, 64):
        r = K.decode(q.to(DEV), k.to(DEV), v.to(DEV), scale, plan=plan, stats=True, out_f32=True, num_splits=splits)
        assert rel_err(r["out_f32"], ref["out"]) < TOL_F32
        assert torch.isinf(r["lse"][1, 20:24]).all() and (r["out_f32"][1, 20:24] == 0).all()
        assert torch.allclose(r["lse"].double().cpu()[0], ref["lse"][0], rtol=0, atol=2e-4)
        fin = torch.isfinite(ref["blk_max"])
        assert torch.equal(torch.isfinite(r["blk_max"]).cpu(), fin)


def test_long_context_planner_beyond_3072_blocks(path):
    """256k tokens = 4096 blocks (beyond the reference's 3072-block limit): three planner steps, the
    attention pass over plan's list against the oracle, and the third step's plan and update against
    the CPU restatement run from a snapshot of the state before that step: refresh decision, list
    length and list equal wherever the decision does not sit on its threshold, the new stored set
    equal wherever the kept mass does not sit on the level (rows this long take the shared-memory
    form of the top-p bisection)."""
    if path == "exact":
        pytest.skip("the planner kernels do not depend on the attention path")
    T0 = 4096 * 64 - 40
    walk = synth.planner_walk_device(77, T0, 3, DEV)
    cfg = RefreshConfig(dense_heads=(6,))             # one head refreshes on every step: update's heavy part runs
    layer = RefreshLayer(cfg)
    names = ("csum", "lse_ref", "cs_ref", "keep", "lse_att", "age", "flags", "cs_now", "trig", "block_idx",
             "block_cnt", "est")
    for t in range(3):
        Tt = T0 + t + 1
        if t == 2:
            snap = {n: layer.state[n].cpu().clone() for n in names}
        out = layer.step(walk.q[t], walk.k[:, :, :Tt], walk.v[:, :, :Tt], walk.scale)
    nb = math.ceil(Tt / 64)
    s = layer.state
    assert int(s["block_cnt"].max()) <= nb and int(s["block_cnt"].min()) >= 3
    mask = layer.read_mask(nb).cpu()
    assert mask[..., 0].all() and mask[..., -2:].all()
    bi, bc = synth.keep_to_plan(mask)
    qh, kh, vh = walk.q[2].cpu(), walk.k[:, :, :Tt].cpu(), walk.v[:, :, :Tt].cpu()
    ref = oracle.decode_f64(qh, kh, vh, walk.scale, bi, bc)
    assert rel_err(out, ref["out"]) < TOL_BF16
    # plan on the CPU restatement from the same pre-step state reproduces the decision and the list
    margin = torch.zeros(1, 8)
    c = snap
    oracle.plan(qh, kh, c["csum"], c["lse_ref"], c["cs_ref"], c["keep"], c["lse_att"], c["age"], c["flags"],
                c["cs_now"], c["trig"], c["block_idx"], c["block_cnt"], walk.scale, cfg.delta, cfg.max_age, cfg.local,
                True, None, None, c["est"], False, 0, None, dec_margin=margin)
    safe = ~(margin.abs() < 1e-4)
    assert safe.float().mean() >= 0.75
    assert bool(c["trig"][0, 6]) and int(c["block_cnt"][0, 6]) == nb
    assert torch.equal(s["trig"].cpu()[safe], c["trig"][safe])
    assert torch.equal(s["block_cnt"].cpu()[safe], c["block_cnt"][safe])
    for h in range(8):
        if safe[0, h]:
            n = int(c["block_cnt"][0, h])
            assert torch.equal(s["block_idx"][0, h, :n].cpu(), c["block_idx"][0, h, :n]), h
    assert torch.allclose(s["cs_now"].cpu()[..., :nb], c["cs_now"][..., :nb], rtol=1e-5, atol=1e-6)
    assert torch.allclose(s["est"].cpu(), c["est"], rtol=1e-4, atol=1e-6)
    # update on the CPU restatement from the GPU's statistics of that pass: the new stored set
    for n in ("trig", "cs_now", "est"):
        c[n] = s[n].cpu().clone()
    tm = torch.zeros(1, 32)
    oracle.update(layer.last["blk_max"].cpu(), layer.last["blk_sum"].cpu(), c["trig"], c["cs_now"], c["keep"],
                  c["lse_ref"], c["cs_ref"], c["lse_att"], Tt, cfg.level, cfg.local, c["flags"], None, c["est"], None,
                  0.0, False, 0, None, 0.0, topp_margin=tm)
    ok = ~(tm < 2e-6).view(1, 8, 4).any(-1)
    assert ok.float().mean() >= 0.75 and bool(c["trig"][0, 6])
    assert torch.equal(s["keep"].cpu()[ok], c["keep"][ok])
    okq = ok.repeat_interleave(4, dim=1)
    assert torch.allclose(s["lse_att"].cpu()[okq], c["lse_att"][okq], rtol=1e-5, atol=1e-5)
    assert K.ext().device_status() == 0


@pytest.mark.parametrize("T,B,splits", [(1000, 2, None), (33, 2, 3), (4096 + 17, 1, 7), (65, 3, 1), (20000, 4, None)])
def test_head_dim_64_on_the_tensor_core_path(T, B, splits, path):
    """D = 64 (half-size stages, two per consumer warp): dense, statistics, statistics only, block
    lists, device-resident length and paged cache against the CPU oracle."""
    if path == "exact":
        pytest.skip("this test is about the tensor-core instantiation")
    from kvskip_b200.cache import PagedKV
    q, k, v, scale = synth.sink_case(60 + T, B, T, D=64)
    qc, kc, vc = q.to(DEV), k.to(DEV), v.to(DEV)
    nb = math.ceil(T / 64)
    ref = oracle.decode_f64(q, k, v, scale, stats=True)
    r = K.decode(qc, kc, vc, scale, stats=True, out_f32=True, num_splits=splits)
    assert rel_err(r["out"], ref["out"]) < TOL_BF16 and rel_err(r["out_f32"], ref["out"]) < TOL_F32
    assert torch.allclose(r["lse"].double().cpu(), ref["lse"], rtol=0, atol=2e-4)
    assert torch.allclose(r["blk_max"].double().cpu(), ref["blk_max"], rtol=0, atol=1e-4)      # nats; scores reach +-30
    assert torch.allclose(r["blk_sum"].double().cpu(), ref["blk_sum"], rtol=2e-4, atol=1e-6)
    so = K.decode(qc, kc, vc, scale, stats=True, load_v=False, num_splits=splits)
    assert torch.equal(so["blk_max"], r["blk_max"]) and torch.equal(so["blk_sum"], r["blk_sum"])
    d = K.decode(qc, kc, vc, scale, out_f32=True, num_splits=splits)
    assert rel_err(d["out_f32"], ref["out"]) < TOL_F32
    # block lists (one empty)
    keep = torch.rand(B, 8, nb, generator=torch.Generator().manual_seed(T)) < 0.5
    keep[..., 0] = True
    keep[..., -1] = True
    keep[B - 1, 5] = False
    bi, bc = synth.keep_to_plan(keep)
    refm = oracle.decode_f64(q, k, v, scale, bi, bc)
    m = K.decode(qc, kc, vc, scale, plan=K.make_plan(keep.to(DEV)), stats=True, out_f32=True, num_splits=splits)
    live = bc.repeat_interleave(4, dim=1) > 0
    assert float((m["out_f32"].double().cpu() - refm["out"])[live].norm() / refm["out"][live].norm()) < TOL_F32
    assert torch.isinf(m["lse"].cpu()[~live]).all()
    assert torch.equal(torch.isfinite(m["blk_max"]).cpu(), keep.repeat_interleave(4, dim=1))
    # device-resident length (cache tail poisoned) and paged cache: same bits as the plain launch
    cap = nb * 64 + 128
    kbig = torch.full((B, 8, cap, 64), float("nan"), dtype=torch.bfloat16, device=DEV)
    vbig = torch.full((B, 8, cap, 64), float("nan"), dtype=torch.bfloat16, device=DEV)
    kbig[:, :, :T], vbig[:, :, :T] = kc, vc
    t_dev = torch.tensor([T], dtype=torch.int32, device=DEV)
    ns = d["num_splits"]
    dd = K.decode(qc, kbig, vbig, scale, out_f32=True, num_splits=ns, t_dev=t_dev)
    assert torch.equal(dd["out_f32"], d["out_f32"]) and torch.equal(dd["lse"], d["lse"])
    pg = PagedKV(B * (cap // 64) + 3, B, 8, 64, cap, DEV, order="shuffled", seed=T)
    pg.k.fill_(float("nan"))
    pg.v.fill_(float("nan"))
    pg.write(kc, vc)
    if T % 64:
        last = pg.table[:, nb - 1].long()
        pg.k[last, :, T % 64:] = float("nan")
        pg.v[last, :, T % 64:] = float("nan")
    dp = K.decode(qc, pg.k, pg.v, scale, out_f32=True, num_splits=ns, page_table=pg.table, seq_len=T)
    assert torch.equal(dp["out_f32"], d["out_f32"]) and torch.equal(dp["lse"], d["lse"])
    assert K.ext().device_status() == 0
