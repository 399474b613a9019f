"""Device-resident sequence length and captured decode steps.

The kernels that read the length from device memory must give bit for bit what the by-value
launches give on views of that length, whatever the cache holds beyond it; a planner loop replayed
from one CUDA graph must leave every state tensor identical to the same loop issued launch by
launch."""
import math

import pytest
import torch

import oracle
from kvskip_b200 import kvskip as K
from kvskip_b200 import synth
from kvskip_b200.graph import StepGraph
from kvskip_b200.refresh import RefreshConfig, RefreshLayer

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _poison_tail(x, T):
    """NaN in every row past T: nothing there may reach a result."""
    x[:, :, T:] = float("nan")
    return x


@pytest.mark.parametrize("T", [1, 63, 64, 65, 1000, 1024, 1500])
@pytest.mark.parametrize("splits", [1, 4])
def test_dense_with_device_length_matches_by_value(T, splits):
    cap = 1536
    q, k, v, scale = synth.dense_case(700 + T, 2, cap)
    q, k, v = q.to(DEV), _poison_tail(k.to(DEV), T), _poison_tail(v.to(DEV), T)
    t_dev = torch.tensor([T], dtype=torch.int32, device=DEV)
    a = K.decode(q, k[:, :, :T], v[:, :, :T], scale, stats=True, out_f32=True, num_splits=splits)
    b = K.decode(q, k, v, scale, stats=True, out_f32=True, num_splits=splits, t_dev=t_dev)
    nb = math.ceil(T / 64)
    assert torch.equal(a["out_f32"], b["out_f32"]) and torch.equal(a["out"], b["out"]) and torch.equal(a["lse"], b["lse"])
    assert torch.equal(a["blk_max"], b["blk_max"][..., :nb]) and torch.equal(a["blk_sum"], b["blk_sum"][..., :nb])
    assert (b["blk_max"][..., nb:] == float("-inf")).all() and (b["blk_sum"][..., nb:] == 0).all()
    assert torch.isfinite(b["out_f32"]).all()
    if splits == 4 and T in (65, 1000, 1500):
        # and against the CPU oracle directly (double precision, the first T tokens only)
        ref = oracle.decode_f64(q.cpu(), k[:, :, :T].cpu(), v[:, :, :T].cpu(), scale, stats=True)
        err = float((b["out_f32"].double().cpu() - ref["out"]).norm() / ref["out"].norm())
        assert err < 5e-5, err
        assert float((b["out"].double().cpu() - ref["out"]).norm() / ref["out"].norm()) < 2e-3
        assert torch.allclose(b["lse"].double().cpu(), ref["lse"], rtol=0, atol=2e-4)
        assert torch.allclose(b["blk_max"][..., :nb].double().cpu(), ref["blk_max"], rtol=0, atol=2e-5)
    # the plain dense kernel (no statistics) too
    c = K.decode(q, k, v, scale, out_f32=True, num_splits=splits, t_dev=t_dev)
    d = K.decode(q, k[:, :, :T], v[:, :, :T], scale, out_f32=True, num_splits=splits)
    assert torch.equal(c["out_f32"], d["out_f32"]) and torch.equal(c["lse"], d["lse"])


@pytest.mark.parametrize("T", [130, 1000, 1471])
def test_masked_with_device_length_matches_by_value(T):
    cap, B, Hkv = 1536, 2, 8
    q, k, v, scale = synth.dense_case(800 + T, B, cap)
    q, k, v = q.to(DEV), _poison_tail(k.to(DEV), T), _poison_tail(v.to(DEV), T)
    nb, nbc = math.ceil(T / 64), cap // 64
    keep = torch.rand(B, Hkv, nb, generator=torch.Generator().manual_seed(T)) < 0.4
    keep[..., 0] = True
    keep[..., -1] = True                                   # the ragged newest block is read
    keep[1, 3] = False                                     # one empty list
    plan = K.make_plan(keep.to(DEV))
    wide = torch.zeros(B, Hkv, nbc, dtype=torch.int32, device=DEV)
    wide[..., :nb] = plan.block_idx
    t_dev = torch.tensor([T], dtype=torch.int32, device=DEV)
    for splits in (1, 3):
        a = K.decode(q, k[:, :, :T], v[:, :, :T], scale, plan=plan, stats=True, out_f32=True, num_splits=splits)
        b = K.decode(q, k, v, scale, plan=K.Plan(wide, plan.block_cnt, plan.max_cnt, nbc), stats=True, out_f32=True,
                     num_splits=splits, t_dev=t_dev)
        assert torch.equal(a["out_f32"], b["out_f32"]) and torch.equal(a["lse"], b["lse"])
        assert torch.equal(a["blk_max"], b["blk_max"][..., :nb]) and torch.equal(a["blk_sum"], b["blk_sum"][..., :nb])
        assert (b["blk_max"][..., nb:] == float("-inf")).all() and (b["blk_sum"][..., nb:] == 0).all()
    # the device-length launch against the CPU oracle over the same block lists
    bi, bc = synth.keep_to_plan(keep)
    ref = oracle.decode_f64(q.cpu(), k[:, :, :T].cpu(), v[:, :, :T].cpu(), scale, bi, bc)
    live = bc.repeat_interleave(4, dim=1) > 0
    err = float((b["out_f32"].double().cpu() - ref["out"])[live].norm() / ref["out"][live].norm())
    assert err < 5e-5, err
    assert torch.allclose(b["lse"].double().cpu()[live], ref["lse"][live], rtol=0, atol=2e-4)


def test_exact_path_refuses_device_length():
    q, k, v, scale = synth.dense_case(1, 1, 256)
    t_dev = torch.tensor([200], dtype=torch.int32, device=DEV)
    K.ext().set_option("decode_path", 1)
    try:
        with pytest.raises(RuntimeError, match="tensor-core path"):
            K.decode(q.to(DEV), k.to(DEV), v.to(DEV), scale, t_dev=t_dev)
    finally:
        K.ext().set_option("decode_path", 0)


def test_advance_and_index_blocks_with_device_length():
    B, T, cap = 3, 700, 1024
    ids = synth.token_ids_with_repeats(5, B, cap).to(DEV)
    nbc = cap // 64 + 4
    t_dev = torch.tensor([T - 2], dtype=torch.int32, device=DEV)
    K.ext().advance(t_dev, 2)
    assert int(t_dev) == T
    a = torch.zeros(B, nbc, dtype=torch.uint8, device=DEV)
    b = torch.ones(B, nbc, dtype=torch.uint8, device=DEV)      # the launch clears it
    K.ext().index_blocks(ids, T, a)
    K.ext().index_blocks(ids, cap, b, t_dev)
    assert torch.equal(a, b) and int(a.sum()) > 0


VARIANTS = {
    "plain": dict(dense_heads=(6,)),
    "peak_auto_warm": dict(calib=0.05, calib_warm=(12, 8), calib_kind="peak", calib_auto_ix=0.001),
    "logit_union": dict(calib=0.3, calib_hold=6, calib_kind="logit", index_heads=(2,), index_union=True),
}


@pytest.mark.parametrize("overlap", [False, True], ids=["serial", "update_on_side_stream"])
@pytest.mark.parametrize("name", list(VARIANTS))
def test_planner_loop_replayed_from_a_graph_matches_launches(name, overlap):
    """40 steps of two layers: launch by launch on views of the current length, and as one captured
    step replayed with the length on the device.  Outputs and every planner state tensor are equal
    after every step; the host-decided scalars change during the loop, so the step is captured
    more than once in the variants that have a warm-up or a hold period.  With `overlap` the
    update kernels run on a second stream inside the graph, joined at the end of the step."""
    T0, steps, B, L = 4096 - 20, 40, 2, 2
    walks = [synth.planner_walk(20 + l, T0, steps, B=B) for l in range(L)]
    ids = synth.token_ids_with_repeats(11, B, T0 + steps).to(DEV)
    ks = [_poison_tail(w.k.to(DEV).clone(), T0 + 1) for w in walks]     # rows of later steps filled in as we go
    vs = [_poison_tail(w.v.to(DEV).clone(), T0 + 1) for w in walks]
    qs = [w.q.to(DEV) for w in walks]
    cap = T0 + steps
    cfg = RefreshConfig(**VARIANTS[name])
    eager = [RefreshLayer(cfg) for _ in range(L)]
    graphed = [RefreshLayer(cfg) for _ in range(L)]
    nbc = math.ceil((T0 + 1) / 64) + cfg.margin
    idx_a = torch.zeros(B, nbc, dtype=torch.uint8, device=DEV)
    idx_b = torch.zeros(B, nbc, dtype=torch.uint8, device=DEV)
    q_buf = torch.zeros(L, *qs[0][0].shape, dtype=qs[0].dtype, device=DEV)
    t_dev = torch.tensor([T0], dtype=torch.int32, device=DEV)

    side = torch.cuda.Stream() if overlap else None

    def launch():
        K.ext().advance(t_dev, 1)
        K.ext().index_blocks(ids, cap, idx_b, t_dev)
        outs = [graphed[l].step(q_buf[l], ks[l], vs[l], walks[l].scale, idx_b, t_dev=t_dev, update_stream=side)
                for l in range(L)]
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
        return outs

    g = StepGraph(launch, graphed, eager=1)
    for t in range(steps):
        T = T0 + t + 1
        for l in range(L):                                   # the token of this step enters the cache
            ks[l][:, :, T - 1] = walks[l].k[:, :, T - 1].to(DEV)
            vs[l][:, :, T - 1] = walks[l].v[:, :, T - 1].to(DEV)
            q_buf[l].copy_(qs[l][t])
        K.ext().index_blocks(ids, T, idx_a)
        out_a = [eager[l].step(qs[l][t], ks[l][:, :, :T], vs[l][:, :, :T], walks[l].scale, idx_a) for l in range(L)]
        if t == 0:      # the first step builds the state on the host, from views of the current length
            out_b = [graphed[l].step(qs[l][t], ks[l][:, :, :T], vs[l][:, :, :T], walks[l].scale, idx_a) for l in range(L)]
            K.ext().advance(t_dev, 1)
        else:
            out_b = g.step()
        assert int(t_dev) == T
        for l in range(L):
            assert torch.equal(out_a[l], out_b[l]), f"output of layer {l} differs at step {t}"
            assert torch.isfinite(out_b[l].float()).all()
            for key in ("trig", "block_cnt", "age", "keep", "aix", "calib", "est", "lse_att", "cs_now", "lse_ref",
                        "cs_ref", "csum"):
                assert torch.equal(eager[l].state[key], graphed[l].state[key]), f"{key} of layer {l} differs at step {t}"
            nb = math.ceil(T / 64)
            assert torch.equal(eager[l].read_mask(nb), graphed[l].read_mask(nb))
            assert eager[l].t == graphed[l].t
    assert g.replays == steps - 2                        # first step on the host, one eager step
    assert g.captures == (1 if name == "plain" else 2)
    assert K.ext().device_status() == 0


@pytest.mark.parametrize("T", [65, 1000, 1471])
def test_vskip_variants_with_device_length_match_by_value(T):
    """Single-pass V-skip (both normaliser rules) and the two-pass form (statistics + P pass,
    selection, P.V pass) with the length read on the device from views of the whole cache, whose
    tail holds NaN: same bits as the by-value launches on views of the current length."""
    cap = 1536
    q, k, v, scale, _ = synth.body_union_case(900 + T, cap)
    q, k, v = q.to(DEV), _poison_tail(k.to(DEV), T), _poison_tail(v.to(DEV), T)
    t_dev = torch.tensor([T], dtype=torch.int32, device=DEV)
    nb = math.ceil(T / 64)
    kv, vv = k[:, :, :T], v[:, :, :T]
    lse = K.decode(q, kv, vv, scale)["lse"]
    for prev in (None, lse):
        a = K.vskip_one_pass(q, kv, vv, scale, tau=1e-3, out_f32=True, count=True, lse_prev=prev, num_splits=3)
        b = K.vskip_one_pass(q, k, v, scale, tau=1e-3, out_f32=True, count=True, lse_prev=prev, num_splits=3,
                             sync=False, t_dev=t_dev)
        assert torch.equal(a["out_f32"], b["out_f32"]) and torch.equal(a["lse"], b["lse"])
        assert torch.equal(a["v_tiles"], b["v_tiles"]) and torch.isfinite(b["out_f32"]).all()
    for rule, value in (("topp", 0.95), ("tau", 1e-3)):
        a = K.vskip_two_pass(q, kv, vv, scale, rule, value, sync=False, out_f32=True)
        b = K.vskip_two_pass(q, k, v, scale, rule, value, sync=False, out_f32=True, t_dev=t_dev)
        # the split counts are sized from the bound here and from the length there: same sums in another order
        assert torch.isfinite(b["out_f32"]).all()
        assert float((a["out_f32"] - b["out_f32"]).norm() / a["out_f32"].norm()) < 2e-6
        assert torch.equal(a["keep"], b["keep"][..., :nb]) and not b["keep"][..., nb:].any()
    ref = oracle.vskip1_f64(q.cpu(), kv.cpu(), vv.cpu(), scale, tau=1e-3, lse_prev=lse.cpu())
    border = (ref["margin"].abs() < 1e-3).sum(-1)
    got = K.vskip_one_pass(q, k, v, scale, tau=1e-3, out_f32=True, count=True, lse_prev=lse, sync=False, t_dev=t_dev)
    assert ((got["v_tiles"].cpu() - ref["v_tiles"]).abs() <= border).all()
    if int(border.sum()) == 0:
        assert float((got["out_f32"].double().cpu() - ref["out"]).norm() / ref["out"].norm()) < 5e-5


def test_single_pass_vskip_replayed_from_a_graph():
    """The vskip1 decode mode as a captured step: append, advance, V-skip with the previous step's
    normaliser, replayed while the cache grows; equal to the same steps issued one by one."""
    T0, steps, cap = 700, 12, 1024
    q, k, v, scale, _ = synth.body_union_case(77, cap)
    q, k, v = q.to(DEV), k.to(DEV), v.to(DEV)
    eager, prev = [], None
    for t in range(steps):
        T = T0 + t + 1
        r = K.vskip_one_pass(q, k[:, :, :T], v[:, :, :T], scale, tau=1e-4, lse_prev=prev, num_splits=4)
        prev = r["lse"]
        eager.append((r["out"].clone(), r["lse"].clone()))
    t_dev = torch.tensor([T0], dtype=torch.int32, device=DEV)
    prev_buf = torch.empty_like(prev)
    prev_buf.copy_(K.vskip_one_pass(q, k[:, :, :T0 + 1], v[:, :, :T0 + 1], scale, tau=1e-4, num_splits=4)["lse"])
    K.ext().advance(t_dev, 1)                                  # step 0 done eagerly (no previous normaliser)

    def launch():
        K.ext().advance(t_dev, 1)
        r = K.vskip_one_pass(q, k, v, scale, tau=1e-4, lse_prev=prev_buf, num_splits=4, sync=False, t_dev=t_dev)
        prev_buf.copy_(r["lse"])
        return r["out"], r["lse"]

    g = StepGraph(launch, eager=1)
    for t in range(1, steps):
        out, lse = g.step()
        assert torch.equal(out, eager[t][0]) and torch.equal(lse, eager[t][1]), t
    assert g.captures == 1 and g.replays >= steps - 2
    assert K.ext().device_status() == 0


def test_update_on_the_layers_own_stream_changes_nothing():
    """RefreshLayer runs `update` on a second stream by default (it prepares the layer's next step;
    the attention output does not wait for it).  Two layers walk the same 24 steps, one with the
    overlap and one without, with other work of the model in between on the main stream: outputs
    and every state tensor are bit-equal after every step, and reading `state` joins the streams."""
    import math
    from kvskip_b200.refresh import RefreshConfig, RefreshLayer
    cfg = RefreshConfig(calib=0.05, calib_warm=(16, 4), calib_kind="peak", calib_auto_ix=0.001)
    steps, T0, B = 24, 4096 + 11, 2
    walk = synth.planner_walk_device(61, T0, steps, torch.device(DEV), B=B)
    ids = synth.token_ids_with_repeats(7, B, T0 + steps).to(DEV)
    a, b = RefreshLayer(cfg), RefreshLayer(cfg, overlap_update=False)
    a.OVERLAP_MIN_WORK = 0          # (by default only steps long enough to pay for the fork and join)
    filler = torch.randn(2048, 2048, device=DEV)
    for t in range(steps):
        T = T0 + t + 1
        idx = synth.index_blocks(ids, T, math.ceil(T / 64))
        oa = a.step(walk.q[t], walk.k[:, :, :T], walk.v[:, :, :T], walk.scale, idx)
        filler = torch.tanh(filler @ filler * 1e-3)          # the rest of a model's layer, on the main stream
        ob = b.step(walk.q[t], walk.k[:, :, :T], walk.v[:, :, :T], walk.scale, idx)
        assert torch.equal(oa, ob), t
        for key in ("keep", "lse_ref", "cs_ref", "csum", "lse_att", "age", "calib", "est", "aix", "cs_now", "trig",
                    "block_cnt"):
            assert torch.equal(a.state[key], b.state[key]), (t, key)
    assert a._ov != 0 and b._ov == 0
    assert K.ext().device_status() == 0
