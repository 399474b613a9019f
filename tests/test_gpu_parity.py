"""GPU parity: the CUDA library against the CPU oracle and the reference-generated goldens.

Every test here needs a B200 and drives the kernels through the compiled extension (pybind front
of the C ABI) or through ctypes on libkvskip_b200.so directly.  Tolerances: integer outputs
(block lists, decisions, stored sets, V-block counts) exact; attention outputs and block
log-sum-exps within 2e-3 relative (bf16 in/out, fp32 accumulation), as the reference's own
criterion (bench/test_decode.py:192-196).
"""
import math

import numpy as np
import pytest
import torch

import oracle
from kvskip_b200 import kvskip as K
from kvskip_b200 import synth
from kvskip_b200.cabi import CAbi
from kvskip_b200.refresh import RefreshConfig, RefreshLayer
from helpers import rel_err, unpack_masks

pytestmark = pytest.mark.gpu

TOL_BF16 = 2e-3      # bf16 outputs, norm-wise relative
TOL_F32 = 5e-5       # fp32 outputs of the exact-order path
DEV = "cuda"


def cuda(*ts):
    return [t.to(DEV) for t in ts]


@pytest.fixture(params=["auto", "exact"], autouse=True)
def path(request):
    """Every test runs on both attention paths: the default (tensor-core kernel for D = 128) and the
    exact-order CUDA-core kernel.  Bit-level assertions apply to the exact-order path only."""
    K.ext().set_option("decode_path", 1 if request.param == "exact" else 0)
    yield request.param
    K.ext().set_option("decode_path", 0)


@pytest.fixture(scope="module")
def dg(golden_dir):
    return np.load(golden_dir / "decode_golden.npz")


@pytest.fixture(scope="module")
def c1(dg):
    q, k, v, scale, keep = synth.sink_body_case(int(dg["c1_seed"]), int(dg["c1_T"]))
    return dict(q=q, k=k, v=v, scale=scale, keep=keep, ref=oracle.decode_f64(q, k, v, scale, stats=True))


def test_extension_is_native():
    ext = K.ext()
    assert ext.__file__.endswith("_kvskip_ext.so")
    assert torch.cuda.get_device_capability()[0] >= 10


@pytest.mark.parametrize("splits", [None, 1, 7])
def test_dense_config1(c1, dg, splits):
    q, k, v = cuda(c1["q"], c1["k"], c1["v"])
    r = K.decode(q, k, v, c1["scale"], num_splits=splits, out_f32=True)
    gold = torch.from_numpy(dg["c1_dense_out"])
    assert rel_err(r["out"], gold) < TOL_BF16
    assert rel_err(r["out_f32"], gold) < TOL_F32
    assert torch.allclose(r["lse"].double().cpu(), c1["ref"]["lse"], rtol=0, atol=2e-4)


def test_dense_fa2_layout(c1, dg):
    q, k, v = cuda(c1["q"], c1["k"], c1["v"])
    ks = k.transpose(1, 2).contiguous().transpose(1, 2)     # memory [B,T,Hkv,D] seen as [B,Hkv,T,D]
    vs = v.transpose(1, 2).contiguous().transpose(1, 2)
    r = K.decode(q, ks, vs, c1["scale"], out_f32=True)
    assert rel_err(r["out_f32"], torch.from_numpy(dg["c1_dense_out"])) < TOL_F32
    r4 = K.decode(q[:, :, None], ks, vs, c1["scale"])          # q as [B,Hq,1,D]
    assert torch.equal(r4["out"], r["out"])


def test_block_stats_config1(c1, dg, path):
    q, k, v = cuda(c1["q"], c1["k"], c1["v"])
    r = K.decode(q, k, v, c1["scale"], stats=True, out_f32=True)
    assert rel_err(r["out_f32"], torch.from_numpy(dg["c1_dense_out"])) < TOL_F32
    M, S = torch.from_numpy(dg["c1_blk_max"]), torch.from_numpy(dg["c1_blk_sum"])
    assert (r["blk_max"].double().cpu() - M).abs().max() < 2e-5
    assert ((r["blk_sum"].double().cpu() - S) / S).abs().max() < 2e-5
    lse_b = r["blk_max"].double().cpu() + torch.log(r["blk_sum"].double().cpu())
    assert ((lse_b - (M + torch.log(S))).abs() / (M + torch.log(S)).abs().clamp_min(1)).max() < TOL_BF16
    # the exact-order path reproduces the float operation order of the scores: block maxima are
    # bit-identical to the CPU restatement of that order, block sums differ only by ex2.approx
    bmax32, bsum32 = oracle.block_stats_f32(c1["q"], c1["k"], c1["scale"])
    if path == "exact":
        assert torch.equal(r["blk_max"].cpu(), bmax32)
        assert torch.allclose(r["blk_sum"].cpu(), bsum32, rtol=3e-6, atol=0)
    else:
        assert torch.allclose(r["blk_max"].cpu(), bmax32, rtol=0, atol=1e-5)
        assert torch.allclose(r["blk_sum"].cpu(), bsum32, rtol=2e-5, atol=0)
    # statistics only (V never read) gives the same bits, at any split count
    r2 = K.decode(q, k, v, c1["scale"], stats=True, load_v=False)
    assert r2["out"] is None
    assert torch.equal(r2["blk_max"], r["blk_max"]) and torch.equal(r2["blk_sum"], r["blk_sum"])
    r3 = K.decode(q, k, v, c1["scale"], stats=True, num_splits=5)
    assert torch.equal(r3["blk_max"], r["blk_max"]) and torch.equal(r3["blk_sum"], r["blk_sum"])
    w = K.block_weights(r["blk_max"], r["blk_sum"]).double().cpu()
    assert (w - torch.softmax(M + torch.log(S), -1)).abs().max() < 1e-6


@pytest.mark.parametrize("splits", [None, 1, 5])
def test_masked_config1(c1, dg, splits):
    q, k, v = cuda(c1["q"], c1["k"], c1["v"])
    keep = c1["keep"].to(DEV)
    plan = K.make_plan(keep)
    assert np.array_equal(plan.block_idx.cpu().numpy(), dg["c1_plan_idx"])
    r = K.decode(q, k, v, c1["scale"], plan=plan, num_splits=splits, out_f32=True, stats=True)
    gold = torch.from_numpy(dg["c1_masked_out"])
    assert rel_err(r["out"], gold) < TOL_BF16
    assert rel_err(r["out_f32"], gold) < TOL_F32
    vis = keep.repeat_interleave(4, 1)
    dense = K.decode(q, k, v, c1["scale"], stats=True)
    assert torch.isinf(r["blk_max"][~vis]).all() and (r["blk_sum"][~vis] == 0).all()
    assert torch.equal(r["blk_max"][vis], dense["blk_max"][vis])
    assert torch.equal(r["blk_sum"][vis], dense["blk_sum"][vis])
    bi, bc = synth.keep_to_plan(c1["keep"])
    ref = oracle.decode_f64(c1["q"], c1["k"], c1["v"], c1["scale"], bi, bc)
    assert torch.allclose(r["lse"].double().cpu(), ref["lse"], rtol=0, atol=2e-4)
    # unsynchronised plan: split count sized for every block, list longer than the count
    r_ns = K.decode(q, k, v, c1["scale"], plan=K.make_plan(keep, sync=False), out_f32=True)
    assert rel_err(r_ns["out_f32"], gold) < TOL_F32


def test_empty_and_single_block_lists(c1):
    q, k, v = cuda(c1["q"], c1["k"], c1["v"])
    nb = c1["keep"].shape[-1]
    keep = torch.zeros(1, 8, nb, dtype=torch.bool, device=DEV)
    keep[0, 1, 5] = True                                     # head 1 reads one block, the others none
    r = K.decode(q, k, v, c1["scale"], plan=K.make_plan(keep), stats=True, out_f32=True, num_splits=3)
    assert torch.isinf(r["lse"][0, :4]).all() and (r["lse"][0, :4] < 0).all()
    assert (r["out_f32"][0, :4] == 0).all() and (r["out_f32"][0, 8:] == 0).all()
    bi, bc = synth.keep_to_plan(keep.cpu())
    ref = oracle.decode_f64(c1["q"], c1["k"], c1["v"], c1["scale"], bi, bc)
    assert rel_err(r["out_f32"][0, 4:8], ref["out"][0, 4:8]) < TOL_F32


@pytest.mark.parametrize("i,splits", [(0, None), (1, 3), (2, 4), (3, 9), (4, 64)])
def test_edge_cases(dg, i, splits):
    """D 64, T 33/64/65/1000/3000, more splits than blocks, a sink tens of nats above the rest."""
    D, T, seed = int(dg[f"edge{i}_D"]), int(dg[f"edge{i}_T"]), int(dg[f"edge{i}_seed"])
    q, k, v, scale = synth.sink_case(seed, 2, T, D)
    qc, kc, vc = cuda(q, k, v)
    r = K.decode(qc, kc, vc, scale, num_splits=splits, out_f32=True, stats=True)
    gold = torch.from_numpy(dg[f"edge{i}_out"])
    assert rel_err(r["out"], gold) < TOL_BF16
    assert rel_err(r["out_f32"], gold) < TOL_F32
    M = torch.from_numpy(dg[f"edge{i}_blk_max"])
    assert (r["blk_max"].double().cpu() - M).abs().max() < 1e-4
    S = torch.from_numpy(dg[f"edge{i}_blk_sum"])
    assert ((r["blk_sum"].double().cpu() - S) / S).abs().max() < 2e-5
    for _ in range(2):   # same launch twice gives the same bits (no shared-memory race)
        r2 = K.decode(qc, kc, vc, scale, num_splits=splits, out_f32=True, stats=True)
        assert torch.equal(r2["out_f32"], r["out_f32"]) and torch.equal(r2["blk_sum"], r["blk_sum"])


def test_batch_and_cabi_ctypes(dg):
    """Batch 12 at a ragged length, once through pybind and once through ctypes on the C ABI."""
    q, k, v, scale = synth.dense_case(7, 12, 2000)
    ref = oracle.decode_f64(q, k, v, scale)
    qc, kc, vc = cuda(q, k, v)
    r = K.decode(qc, kc, vc, scale, out_f32=True)
    assert rel_err(r["out"], ref["out"]) < TOL_BF16 and rel_err(r["out_f32"], ref["out"]) < TOL_F32
    abi = CAbi()
    assert abi.lib.kvskip_get_option(b"decode_path") == K.ext().get_option("decode_path")   # one library, one state
    out, lse, _, _, o32, _ = abi.decode(qc, kc, vc, scale, num_splits=r["num_splits"], want_f32=True)
    assert torch.equal(out, r["out"]) and torch.equal(o32, r["out_f32"]) and torch.equal(lse, r["lse"])
    with pytest.raises(RuntimeError):
        abi.decode(qc, kc, vc, scale, stages=5)
    with pytest.raises(RuntimeError):
        K.ext().decode(qc, kc, vc, scale, None, None, False, False, 1, 2, False, False)   # load_v=False without stats


def test_vskip1_matches_oracle(golden_dir):
    g = np.load(golden_dir / "vskip_golden.npz")
    q, k, v, scale, _ = synth.body_union_case(int(g["seed"]), int(g["T"]))
    qc, kc, vc = cuda(q, k, v)
    for tau in (1e-4, 1e-3):
        r = K.vskip_one_pass(qc, kc, vc, scale, tau=tau, out_f32=True, count=True)
        ref = oracle.vskip1_f64(q, k, v, scale, tau=tau)
        border = (ref["margin"].abs() < 1e-3).sum(-1)                 # votes within 1e-3 nats of log(tau)
        diff = (r["v_tiles"].cpu() - ref["v_tiles"]).abs()
        assert (diff <= border).all(), (diff, border)
        if int(border.sum()) == 0:
            assert np.array_equal(r["v_tiles"].cpu().numpy(), g[f"sink_keep_{tau:g}"].sum(-1))
            assert rel_err(r["out_f32"], torch.from_numpy(g[f"sink_out_{tau:g}"])) < TOL_F32
        assert rel_err(r["out"], ref["out"]) < TOL_BF16
        lse_exact = torch.from_numpy(g["lse_exact"]).to(DEV)
        for splits in (None, 1, 6):
            r2 = K.vskip_one_pass(qc, kc, vc, scale, tau=tau, out_f32=True, count=True, lse_prev=lse_exact,
                                  num_splits=splits)
            ref2 = oracle.vskip1_f64(q, k, v, scale, tau=tau, lse_prev=torch.from_numpy(g["lse_exact"]))
            border2 = (ref2["margin"].abs() < 1e-3).sum(-1)
            assert ((r2["v_tiles"].cpu() - ref2["v_tiles"]).abs() <= border2).all()
            if int(border2.sum()) == 0:
                assert rel_err(r2["out_f32"], torch.from_numpy(g[f"prev_out_{tau:g}"])) < TOL_F32
                assert torch.allclose(r2["lse"].double().cpu(), ref2["lse"], rtol=0, atol=2e-4)
            assert 0.3 < r2["kept_frac"] < 0.8


def test_vskip_two_pass(c1):
    q, k, v = cuda(c1["q"], c1["k"], c1["v"])
    for rule, val in (("topp", 0.99), ("tau", 1e-4)):
        r = K.vskip_two_pass(q, k, v, c1["scale"], rule=rule, value=val, out_f32=True)
        bi, bc = synth.keep_to_plan(r["keep"].cpu())
        ref = oracle.decode_f64(c1["q"], c1["k"], c1["v"], c1["scale"], bi, bc)
        assert rel_err(r["out"], ref["out"]) < TOL_BF16
        assert rel_err(r["out_f32"], ref["out"]) < 2e-4          # P travels in fp16
    # pass 2 alone against the CPU restatement, several split counts
    first = K.decode(q, k, v, c1["scale"], stats=True, load_v=False, write_p=True)
    logw = first["blk_max"] + torch.log(first["blk_sum"])
    keep = K.select_blocks(logw, 4, "topp", 0.9, 2)
    kq = keep.repeat_interleave(4, dim=1)
    lk = logw.masked_fill(~kq, float("-inf")).logsumexp(-1, keepdim=True)
    w = torch.exp(first["blk_max"] - lk).masked_fill(~kq, 0.0).view(1, 8, 4, -1).transpose(2, 3).contiguous()
    plan = K.make_plan(keep)
    ref = oracle.pv_f64(first["p"].cpu(), c1["v"], w.cpu(), plan.block_idx.cpu(), plan.block_cnt.cpu())
    for splits in (1, 4, None):
        out, o32 = K.pv(first["p"], v, w, plan, num_splits=splits, out_f32=True)
        assert rel_err(o32, ref) < 1e-5


def _planner_state(seed, B, T, NBC, device):
    """Random but well-formed planner state around a dense pass at length T."""
    q, k, v, scale = synth.dense_case(seed, B, T)
    g = torch.Generator().manual_seed(seed)
    nb = math.ceil(T / 64)
    from kvskip_b200.refresh import centroid_sums
    csum = torch.zeros(B, 8, NBC, 128)
    before = centroid_sums(k[:, :, :T - 1])                 # the step's own token is added by plan
    csum[:, :, :before.shape[2]] = before
    st = dict(
        csum=csum,
        lse_ref=torch.full((B, 32, NBC), float("-inf")),
        cs_ref=torch.zeros(B, 32, NBC),
        keep=torch.zeros(B, 8, NBC, dtype=torch.uint8),
        lse_att=torch.randn(B, 32, generator=g) * 0.3 + 6.0,
        age=torch.randint(0, 30, (B, 8), generator=g, dtype=torch.int32),
        flags=torch.tensor([0, 0, 4, 0, 2, 0, 1, 0], dtype=torch.int32),
        cs_now=torch.zeros(B, 32, NBC),
        trig=torch.zeros(B, 8, dtype=torch.uint8),
        block_idx=torch.zeros(B, 8, NBC, dtype=torch.int32),
        block_cnt=torch.zeros(B, 8, dtype=torch.int32),
        idx=(torch.rand(B, NBC, generator=g) < 0.05).to(torch.uint8),
        calib=torch.rand(B, 8, generator=g) * 0.02,
        est=torch.zeros(B, 8),
        aix=(torch.rand(B, 8, generator=g) < 0.3).to(torch.uint8))
    st["lse_ref"][:, :, :nb] = torch.randn(B, 32, nb, generator=g) * 1.5
    st["cs_ref"][:, :, :nb] = torch.randn(B, 32, nb, generator=g) * 0.05
    st["keep"][:, :, :nb] = (torch.rand(B, 8, nb, generator=g) < 0.4).to(torch.uint8)
    st["idx"][:, nb:] = 0
    return q, k, v, scale, st


PLAN_OUT = ("csum", "age", "cs_now", "trig", "block_idx", "block_cnt", "est")
UPD_OUT = ("keep", "lse_ref", "cs_ref", "lse_att", "calib", "aix")


@pytest.mark.parametrize("T,kind,calib_on,B", [(4096, 2, True, 2), (4137, 0, True, 2), (8192 + 3, 1, False, 2),
                                               (199, 2, True, 2), (32768 + 70, 2, True, 1), (64000 + 9, 1, True, 1),
                                               (80000, 2, True, 1), (96000 + 5, 0, True, 1), (128000 - 3, 2, True, 1)])
def test_plan_update_single_step_vs_oracle(T, kind, calib_on, B, path):
    """One plan and one update call on random state: integer outputs identical to the CPU
    restatement, float outputs equal up to the GPU's approximate exp/log.  The longer rows (514 to
    2000 blocks) go through every register width of update's top-p bisection."""
    if T > 10000 and path == "exact":
        pytest.skip("the planner kernels do not depend on the attention path: long rows once")
    NBC = math.ceil(T / 64) + 64
    nb = math.ceil(T / 64)
    q, k, v, scale, st = _planner_state(40 + kind, B, T, NBC, DEV)
    cpu = {n: t.clone() for n, t in st.items()}
    gpu = {n: t.to(DEV) for n, t in st.items()}
    margin = torch.zeros(B, 8)
    oracle.plan(q, k, cpu["csum"], cpu["lse_ref"], cpu["cs_ref"], cpu["keep"], cpu["lse_att"], cpu["age"], cpu["flags"],
                cpu["cs_now"], cpu["trig"], cpu["block_idx"], cpu["block_cnt"], scale, 0.05, 32, 2, True, cpu["idx"],
                cpu["calib"], cpu["est"], calib_on, kind, cpu["aix"], dec_margin=margin)
    qc, kc, vc = cuda(q, k, v)
    K.ext().plan(qc, kc, gpu["csum"], gpu["lse_ref"], gpu["cs_ref"], gpu["keep"], gpu["lse_att"], gpu["age"],
                 gpu["flags"], gpu["cs_now"], gpu["trig"], gpu["block_idx"], gpu["block_cnt"], scale, 0.05, 32, 2,
                 True, gpu["idx"], gpu["calib"], gpu["est"], calib_on, kind, gpu["aix"])
    safe = ~(margin.abs() < 1e-4)                                  # decisions not sitting on the threshold
    assert safe.float().mean() > 0.8
    assert torch.equal(gpu["trig"].cpu()[safe], cpu["trig"][safe])
    assert torch.equal(gpu["age"].cpu()[safe], cpu["age"][safe])
    assert torch.equal(gpu["block_cnt"].cpu()[safe], cpu["block_cnt"][safe])
    for b in range(B):
        for h in range(8):
            if safe[b, h]:
                n = int(cpu["block_cnt"][b, h])
                assert torch.equal(gpu["block_idx"][b, h, :n].cpu(), cpu["block_idx"][b, h, :n])
    assert torch.allclose(gpu["csum"].cpu(), cpu["csum"], rtol=0, atol=0)
    assert torch.allclose(gpu["cs_now"].cpu()[:, :, :nb], cpu["cs_now"][:, :, :nb], rtol=1e-5, atol=1e-6)
    assert torch.allclose(gpu["est"].cpu(), cpu["est"], rtol=1e-4, atol=1e-6)
    # the pass itself, then update on both sides from the same statistics
    plan = K.Plan(gpu["block_idx"], gpu["block_cnt"], nb, nb)
    r = K.decode(qc, kc, vc, scale, plan=plan, stats=True)
    bmax, bsum = r["blk_max"].cpu(), r["blk_sum"].cpu()
    for n in PLAN_OUT:                                           # continue from identical state
        cpu[n] = gpu[n].cpu().clone()
    tm = torch.zeros(B, 32)
    oracle.update(bmax, bsum, cpu["trig"], cpu["cs_now"], cpu["keep"], cpu["lse_ref"], cpu["cs_ref"], cpu["lse_att"],
                  T, 0.99, 2, cpu["flags"], cpu["idx"], cpu["est"], cpu["calib"], 0.05, False, kind, cpu["aix"],
                  0.01, topp_margin=tm)
    K.ext().update(r["blk_max"], r["blk_sum"], gpu["trig"], gpu["cs_now"], gpu["keep"], gpu["lse_ref"], gpu["cs_ref"],
                   gpu["lse_att"], T, 0.99, 2, gpu["flags"], gpu["idx"], gpu["est"], gpu["calib"], 0.05, False, kind,
                   gpu["aix"], 0.01)
    tie = (tm < 2e-6).view(B, 8, 4).any(-1)                        # kept mass within float error of the level
    ok = ~tie
    assert ok.float().mean() > 0.6
    assert torch.equal(gpu["keep"].cpu()[ok], cpu["keep"][ok])
    assert torch.equal(gpu["aix"].cpu(), cpu["aix"])
    assert torch.allclose(gpu["calib"].cpu(), cpu["calib"], rtol=1e-4, atol=1e-6)
    assert torch.equal(torch.isinf(gpu["lse_ref"].cpu()), torch.isinf(cpu["lse_ref"]))
    fin = torch.isfinite(cpu["lse_ref"])
    assert torch.allclose(gpu["lse_ref"].cpu()[fin], cpu["lse_ref"][fin], rtol=1e-5, atol=1e-5)
    assert torch.equal(gpu["cs_ref"].cpu(), cpu["cs_ref"])
    okq = ok.repeat_interleave(4, dim=1)
    assert torch.allclose(gpu["lse_att"].cpu()[okq], cpu["lse_att"][okq], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("T,B", [(8192 + 3, 2), (199, 3), (40, 1), (65536 + 1, 1)])
def test_plan_work_layouts_give_the_same_bits(T, B):
    """`plan` spreads a head's centroid scores over several CTAs in two ways: a thread-block cluster
    whose CTAs hand their results to the first one through its shared memory (1, 2, 4 or 8 CTAs per
    head), and independent CTAs of 32-block rounds counted in global memory (1, 2, 4 or 8 rounds
    each).  Every layout must leave every output bit-identical: same state in, one call each."""
    NBC = math.ceil(T / 64) + 64
    q, k, v, scale, st = _planner_state(77, B, T, NBC, DEV)
    qc, kc = q.to(DEV), k.to(DEV)
    ext = K.ext()
    outs = {}
    layouts = [("plan_cluster", -1), ("plan_cluster", 1), ("plan_cluster", 2), ("plan_cluster", 4), ("plan_cluster", 8),
               ("plan_rounds", 0), ("plan_rounds", 1), ("plan_rounds", 2), ("plan_rounds", 4), ("plan_rounds", 8)]
    try:
        for name, value in layouts:
            ext.set_option("plan_cluster", value if name == "plan_cluster" else 0)
            ext.set_option("plan_rounds", value if name == "plan_rounds" else 0)
            gpu = {n: t.to(DEV) for n, t in st.items()}
            ext.plan(qc, kc, gpu["csum"], gpu["lse_ref"], gpu["cs_ref"], gpu["keep"], gpu["lse_att"], gpu["age"],
                     gpu["flags"], gpu["cs_now"], gpu["trig"], gpu["block_idx"], gpu["block_cnt"], scale, 0.05, 32, 2,
                     True, gpu["idx"], gpu["calib"], gpu["est"], True, 2, gpu["aix"])
            cnt = gpu["block_cnt"]
            valid = torch.arange(NBC, device=DEV)[None, None, :] < cnt[..., None]
            gpu["block_idx"] = torch.where(valid, gpu["block_idx"], 0)
            outs[(name, value)] = gpu
    finally:
        ext.set_option("plan_cluster", -1)
        ext.set_option("plan_rounds", 0)
    assert ext.device_status() == 0
    first = outs[layouts[0]]
    assert int(first["block_cnt"].sum()) > 0
    for key, got in outs.items():
        for n in ("csum", "cs_now", "trig", "age", "est", "block_cnt", "block_idx"):
            assert torch.equal(got[n], first[n]), (key, n)


VARIANTS = {
    "plain": dict(dense_heads=(6,)),
    "union": dict(dense_heads=(6,), index_heads=(2,), index_union=True),
    "only": dict(dense_heads=(6,), index_heads=(2,), index_union=False),
    "peak_auto": dict(calib=0.05, calib_warm=(32, 8), calib_kind="peak", calib_auto_ix=0.001),
    "logit": dict(calib=0.3, calib_warm=(32, 8), calib_kind="logit"),
    "add_union": dict(calib=0.3, calib_warm=(32, 8), calib_kind="add", index_heads=(2,), index_union=True),
}


@pytest.mark.parametrize("name", list(VARIANTS))
def test_planner_loop_vs_python_planner_golden(golden_dir, name):
    """plan -> masked+stats attention -> update for 48 steps with no host sync inside a step; the
    blocks read on every head-step must equal the reference's Python planner's (golden)."""
    g = np.load(golden_dir / "planner_golden.npz")
    T0, steps, B, nbm = int(g["T0"]), int(g["steps"]), int(g["B"]), int(g["nb_max"])
    walk = synth.planner_walk(int(g["seed"]), T0, steps, B=B)
    ids = synth.token_ids_with_repeats(int(g["seed"]) + 1, B, T0 + steps).to(DEV)
    masks = unpack_masks(g[f"{name}_masks"], nbm)
    kc, vc, qc = cuda(walk.k, walk.v, walk.q)
    layer = RefreshLayer(RefreshConfig(**VARIANTS[name]))
    got, outs = [], []
    for t in range(steps):
        Tt = T0 + t + 1
        nb = math.ceil(Tt / 64)
        idx = None
        if layer.uses_index():
            idx = torch.empty(B, nbm, dtype=torch.uint8, device=DEV)
            K.ext().index_blocks(ids, Tt, idx)
        out = layer.step(qc[t], kc[:, :, :Tt], vc[:, :, :Tt], walk.scale, idx)
        got.append(torch.ones(B, 8, nb, dtype=torch.bool, device=DEV) if t == 0 else layer.read_mask(nb))
        outs.append(out)
    agree = total = 0
    for t in range(steps):
        nb = got[t].shape[-1]
        same = (got[t].cpu().numpy() == masks[t, :, :, :nb]).all(-1)
        agree += int(same.sum())
        total += same.size
    assert agree == total, f"{name}: identical read sets on {agree}/{total} head-steps"
    s = layer.state
    nb = math.ceil((T0 + steps) / 64)
    assert np.array_equal(s["keep"][..., :nb].cpu().numpy().astype(bool), g[f"{name}_keep"][..., :nb])
    assert np.array_equal(s["aix"].cpu().numpy().astype(bool), g[f"{name}_aix"])
    # corrections and attended log-sum-exps of the last step against the Python planner's: 1e-5 absolute
    # (measured on both attention paths: <= 1.6e-6 and <= 1.9e-6)
    assert np.allclose(s["calib"].cpu().numpy(), g[f"{name}_calib"][-1], rtol=0, atol=1e-5)
    assert np.allclose(s["lse_att"].cpu().numpy(), g[f"{name}_lse_att"], rtol=0, atol=1e-5)
    assert rel_err(outs[-1].float(), torch.from_numpy(g[f"{name}_out_last"])) < 2 * TOL_BF16


def test_index_blocks_kernel(golden_dir):
    g = np.load(golden_dir / "index_golden.npz")
    P, S = int(g["P"]), int(g["S"])
    ids = synth.token_ids_with_repeats(int(g["seed"]), 3, P + S, vocab=int(g["vocab"]), repeat_p=float(g["repeat_p"]))
    idc = ids.to(DEV)
    nbm = g["blocks"].shape[-1]
    out = torch.empty(3, nbm, dtype=torch.uint8, device=DEV)
    for t in range(S):
        K.ext().index_blocks(idc, P + t + 1, out)
        assert np.array_equal(out.cpu().numpy().astype(bool), g["blocks"][t]), t


def test_merge_entry_point():
    torch.manual_seed(3)
    R, N, D = 4, 64, 128
    m = torch.randn(R, N) * 4
    l = torch.rand(R, N) + 0.5
    acc = torch.randn(R, N, D)
    m[1, :5] = float("-inf"); l[1, :5] = 0; acc[1, :5] = 0
    ml = torch.stack([m, l], -1).contiguous()
    out, o32, lse = K.ext().merge(acc.to(DEV), ml.to(DEV))
    ref_out, ref_lse = oracle.combine_f32(acc.transpose(0, 1).contiguous(), ml.transpose(0, 1).contiguous())
    assert torch.allclose(o32.cpu(), ref_out, rtol=2e-6, atol=1e-6)
    assert torch.allclose(lse.cpu(), ref_lse, rtol=0, atol=1e-5)
    assert torch.equal(out.cpu(), o32.cpu().to(torch.bfloat16))


def test_full_size_64k_dense_and_masked():
    """Benchmark size (batch 1, 64k context, 1024 blocks): full comparison with the CPU oracle plus
    the size-independent identities: statistics reproduce the output's normaliser, the masked pass
    over every block equals the dense pass bit for bit, split counts agree within tolerance."""
    q, k, v, scale, keep = synth.body_union_case(3, 65536)
    qc, kc, vc = cuda(q, k, v)
    r = K.decode(qc, kc, vc, scale, stats=True, out_f32=True)
    ref = oracle.decode_f64(q, k, v, scale, stats=True)
    assert rel_err(r["out"], ref["out"]) < TOL_BF16 and rel_err(r["out_f32"], ref["out"]) < TOL_F32
    logw = r["blk_max"].double() + torch.log(r["blk_sum"].double())
    assert torch.allclose(torch.logsumexp(logw, -1).cpu(), r["lse"].double().cpu(), rtol=0, atol=1e-4)
    assert torch.allclose(r["lse"].double().cpu(), ref["lse"], rtol=0, atol=2e-4)
    full = torch.ones(1, 8, 1024, dtype=torch.bool, device=DEV)
    rf = K.decode(qc, kc, vc, scale, plan=K.make_plan(full), stats=True, out_f32=True, num_splits=r["num_splits"])
    assert torch.equal(rf["out_f32"], r["out_f32"]) and torch.equal(rf["blk_sum"], r["blk_sum"])
    kp = keep.to(DEV)
    assert 0.5 < keep.float().mean() < 0.62
    rm = K.decode(qc, kc, vc, scale, plan=K.make_plan(kp), stats=True, out_f32=True)
    bi, bc = synth.keep_to_plan(keep)
    refm = oracle.decode_f64(q, k, v, scale, bi, bc)
    assert rel_err(rm["out"], refm["out"]) < TOL_BF16 and rel_err(rm["out_f32"], refm["out"]) < TOL_F32
    lse_prev = r["lse"]
    rv = K.vskip_one_pass(qc, kc, vc, scale, tau=1e-4, lse_prev=lse_prev, count=True, out_f32=True)
    refv = oracle.vskip1_f64(q, k, v, scale, tau=1e-4, lse_prev=lse_prev.cpu())
    border = (refv["margin"].abs() < 1e-3).sum(-1)
    assert ((rv["v_tiles"].cpu() - refv["v_tiles"]).abs() <= border).all()
    assert rel_err(rv["out"], refv["out"]) < TOL_BF16


def test_no_wait_timed_out():
    assert K.ext().device_status() == 0


@pytest.mark.parametrize("R", [2, 8])
def test_sequence_shards_emulated_on_one_gpu(R):
    """The sequence-sharded path with the ranks emulated on one GPU: every shard's local pass, the
    (acc, m, l) triples stacked as an all-gather would deliver them, one merge.  Against the CPU
    oracle on the whole sequence and against the unsharded kernel."""
    from kvskip_b200 import shard
    q, k, v, scale, keep = synth.sink_body_case(13, T=8192 + 100, B=2)
    qc, kc, vc = cuda(q, k, v)
    nb = keep.shape[-1]
    parts, partsm = [], []
    for r in range(R):
        lo, hi = shard.block_range(nb, r, R)
        kl, vl = kc[:, :, lo * 64:hi * 64], vc[:, :, lo * 64:hi * 64]
        parts.append(shard.local_partial(qc, kl, vl, scale))
        lk = shard.shard_plan(keep, r, R).to(DEV)
        partsm.append(shard.local_partial(qc, kl, vl, scale, plan=K.make_plan(lk)))
    got = shard.merge_partials(torch.stack(parts), 2, 32)
    gotm = shard.merge_partials(torch.stack(partsm), 2, 32)
    ref = oracle.decode_f64(q, k, v, scale)
    bi, bc = synth.keep_to_plan(keep)
    refm = oracle.decode_f64(q, k, v, scale, bi, bc)
    assert rel_err(got["out"], ref["out"]) < TOL_BF16 and rel_err(got["out_f32"], ref["out"]) < TOL_F32
    assert rel_err(gotm["out"], refm["out"]) < TOL_BF16 and rel_err(gotm["out_f32"], refm["out"]) < TOL_F32
    assert torch.allclose(got["lse"].double().cpu(), ref["lse"], rtol=0, atol=2e-4)
    assert torch.allclose(gotm["lse"].double().cpu(), refm["lse"], rtol=0, atol=2e-4)
    one = K.decode(qc, kc, vc, scale, out_f32=True)
    assert rel_err(got["out_f32"], one["out_f32"].double().cpu()) < 2e-5


def xchg_buffers(R, N, W=130):
    """R exchange buffers of 2*R*N*W words of 8 bytes (value bits, step number), zeroed; returns
    the tensors (int32 view [2,R,N,W,2]) and their addresses."""
    bufs = [torch.zeros(2, R, N, W, 2, dtype=torch.int32, device=DEV) for _ in range(R)]
    return bufs, [b_.data_ptr() for b_ in bufs]


def xchg_place(buf, par, r, triple, seq):
    """A rank's packed rows [N, W] as (value, step) words in slot [par][r] of a buffer."""
    buf[par, r, :, :, 0] = triple.contiguous().view(torch.int32)
    buf[par, r, :, :, 1] = seq


def xchg_rows(buf, par, r):
    """(values [N, W] as fp32, steps [N, W]) of slot [par][r]."""
    return buf[par, r, :, :, 0].contiguous().view(torch.float32), buf[par, r, :, :, 1]


def test_exchange_merge_single_rank():
    """The fused exchange kernel with one rank (its own buffer is the only peer): the merge of one
    triple is the identity, step numbers alternate the buffer set, nothing times out."""
    torch.manual_seed(5)
    N, D = 32, 128
    bufs, bp = xchg_buffers(1, N)          # (keep the tensors alive: the kernels get their addresses)
    fp = [0]
    for seq in (1, 2, 3):
        o = torch.randn(N, D, device=DEV)
        lse = torch.randn(N, device=DEV) * 3
        lse[3] = float("-inf")
        o[3] = 0
        out, o32, l2 = K.ext().exchange_merge(o, lse, bp, fp, 0, seq)
        assert torch.allclose(o32, o, rtol=2e-6, atol=1e-7) and torch.equal(out, o32.to(torch.bfloat16))
        assert torch.allclose(l2[torch.isfinite(lse)], lse[torch.isfinite(lse)], rtol=0, atol=1e-5)
        assert torch.isinf(l2[3]) and (o32[3] == 0).all()
    assert K.ext().device_status() == 0


def test_decode_exchange_single_rank(path):
    """Attention + exchange + merge in one kernel with one rank (its own buffer is the only peer):
    the outputs are those of the plain launch with the same split count."""
    if path == "exact":
        pytest.skip("the exchange inside the kernel exists on the tensor-core path")
    q, k, v, scale, keep = synth.sink_body_case(8, T=8192 + 13, B=2)
    qc, kc, vc = cuda(q, k, v)
    N, D = 2 * 32, 128
    bufs, bp = xchg_buffers(1, N)          # (keep the tensors alive: the kernels get their addresses)
    fp = [0]
    plan = K.make_plan(keep.to(DEV))
    for seq, pl in ((1, None), (2, plan), (3, None)):
        bi, bc = (None, None) if pl is None else (pl.block_idx, pl.block_cnt)
        out, lse, _, _, o32, _ = K.ext().decode_exchange(qc, kc, vc, scale, bi, bc, 6, bp, fp, 0, seq)
        ref = K.decode(qc, kc, vc, scale, plan=pl, num_splits=6, out_f32=True)
        assert torch.equal(o32, ref["out_f32"]) and torch.equal(out, ref["out"])
        assert torch.allclose(lse, ref["lse"], rtol=0, atol=1e-5)
    with pytest.raises(RuntimeError, match="num_splits > 1"):
        K.ext().decode_exchange(qc, kc, vc, scale, None, None, 1, bp, fp, 0, 4)
    assert K.ext().device_status() == 0


def test_decode_exchange_four_ranks_emulated(path):
    """The one-launch sequence-sharded step as rank 0 of four, on one GPU and without any kernel
    waiting for another: the triples and flags of ranks 1..3 are placed in rank 0's buffer
    beforehand (as their kernels would have stored them), the peers' own buffers are scratch.
    The result equals pack -> merge of the four partials."""
    if path == "exact":
        pytest.skip("the exchange inside the kernel exists on the tensor-core path")
    from kvskip_b200 import shard
    R, B = 4, 1
    q, k, v, scale, keep = synth.sink_body_case(12, T=16384 + 50, B=B)
    qc, kc, vc = cuda(q, k, v)
    nb = keep.shape[-1]
    N, D, W = B * 32, 128, 130
    bufs, bp = xchg_buffers(R, N)
    fp = [0] * R
    parts = []
    for r in range(R):
        lo, hi = shard.block_range(nb, r, R)
        parts.append(shard.local_partial(qc, kc[:, :, lo * 64:hi * 64], vc[:, :, lo * 64:hi * 64], scale, num_splits=5))
    want = shard.merge_partials(torch.stack(parts), B, 32)
    for seq in (1, 2):
        par = seq & 1
        for r in range(1, R):
            xchg_place(bufs[0], par, r, parts[r], seq)
        lo, hi = shard.block_range(nb, 0, R)
        out, lse, _, _, o32, _ = K.ext().decode_exchange(qc, kc[:, :, lo * 64:hi * 64], vc[:, :, lo * 64:hi * 64], scale,
                                                         None, None, 5, bp, fp, 0, seq)
        assert torch.equal(o32.view(B, 32, D), want["out_f32"]) and torch.equal(lse.view(B, 32), want["lse"])
        # rank 0's own triple reached every peer's buffer, every word carrying the step number
        for r in range(1, R):
            vals, steps = xchg_rows(bufs[r], par, 0)
            assert torch.equal(vals, parts[0]) and (steps == seq).all()
    assert K.ext().device_status() == 0


def test_decode_exchange_short_and_empty_lists_emulated(path):
    """The one-launch sequence-sharded step with block lists, as rank 0 of two, in the regime where
    the kernel cuts lists into pieces of at least 24 blocks (more CTAs than SMs): a head whose local
    list is short and a head with no local block at all must still store their rows to the peer,
    flag them and take part in the merge.  The peer's triples and flags are placed beforehand so
    that no kernel waits for another; the result equals pack -> merge of the two partials."""
    if path == "exact":
        pytest.skip("the exchange inside the kernel exists on the tensor-core path")
    from kvskip_b200 import shard
    R, B, splits = 2, 8, 4                                  # 8 x 8 heads x 4 splits = 256 CTAs > 148 SMs
    q, k, v, scale, keep = synth.sink_body_case(14, T=8192, B=B, stored_frac=0.6)
    qc, kc, vc = cuda(q, k, v)
    nb = keep.shape[-1]
    lo, hi = shard.block_range(nb, 0, R)
    keep0 = shard.shard_plan(keep, 0, R).clone()
    keep0[0, 1] = False
    keep0[0, 1, :5] = True                                  # a short list: one piece
    keep0[1, 2] = False                                     # nothing to read on this rank
    keep0[2, 3] = False
    keep0[2, 3, 7] = True                                   # a single block
    assert int(keep0.sum(-1).max()) > 24
    plan0 = K.make_plan(keep0.to(DEV))
    plan1 = K.make_plan(shard.shard_plan(keep, 1, R).to(DEV))
    lo1, hi1 = shard.block_range(nb, 1, R)
    parts = [shard.local_partial(qc, kc[:, :, lo * 64:hi * 64], vc[:, :, lo * 64:hi * 64], scale, plan=plan0,
                                 num_splits=splits),
             shard.local_partial(qc, kc[:, :, lo1 * 64:hi1 * 64], vc[:, :, lo1 * 64:hi1 * 64], scale, plan=plan1)]
    want = shard.merge_partials(torch.stack(parts), B, 32)
    N, D, W = B * 32, 128, 130
    bufs, bp = xchg_buffers(R, N)
    fp = [0] * R
    for seq in (1, 2):
        par = seq & 1
        xchg_place(bufs[0], par, 1, parts[1], seq)
        out, lse, _, _, o32, _ = K.ext().decode_exchange(qc, kc[:, :, lo * 64:hi * 64], vc[:, :, lo * 64:hi * 64], scale,
                                                         plan0.block_idx, plan0.block_cnt, splits, bp, fp, 0, seq)
        assert torch.equal(o32.view(B, 32, D), want["out_f32"]) and torch.equal(lse.view(B, 32), want["lse"])
        # every row of rank 0, the short and the empty heads included, reached the peer, every word
        # carrying the step number
        vals, steps = xchg_rows(bufs[1], par, 0)
        assert torch.equal(vals, parts[0]) and (steps == seq).all()
    assert K.ext().device_status() == 0
    # against the CPU oracle on the whole sequence with the combined lists
    full = torch.cat([keep0, shard.shard_plan(keep, 1, R)], dim=-1)
    bi, bc = synth.keep_to_plan(full)
    ref = oracle.decode_f64(q, k, v, scale, bi, bc)
    assert rel_err(want["out_f32"], ref["out"]) < TOL_F32


def test_exchange_wait_runs_out_and_reports(path):
    """Failure detection on the device, without faulting anything: rank 0 of two runs the exchange
    while rank 1's words never arrive.  With the poll limit lowered ("spin_limit") the kernel
    gives up after about a millisecond, sets the status word to 0x500 + peer (0x510 + peer from the
    attention kernel's own exchange), returns, and the context stays usable: the same call with the
    peer's rows and flags in place is clean and correct."""
    if path == "exact":
        pytest.skip("one path is enough: the exchange kernels do not depend on it")
    from kvskip_b200 import shard
    ext = K.ext()
    R, N, D, W = 2, 64, 128, 130
    bufs, bp = xchg_buffers(R, N)
    fp = [0] * R
    torch.manual_seed(3)
    o = torch.randn(N, D, device=DEV)
    lse = torch.randn(N, device=DEV)
    peer = torch.randn(N, W, device=DEV)
    peer[:, D + 1] = 1.0
    assert ext.device_status() == 0
    ext.set_option("spin_limit", 4096)
    try:
        assert ext.get_option("spin_limit") == 4096
        ext.exchange_merge(o, lse, bp, fp, 0, 1)                      # rank 1 never arrives
        assert ext.device_status() == 0x501
        assert ext.device_status() == 0                               # reading clears the word
        with pytest.raises(K.DeviceWaitError) as ei:
            ext.exchange_merge(o, lse, bp, fp, 0, 2)
            K.check_status("exchange")
        assert ei.value.code == 0x501
        # the peer's rows and flags in place: clean, and equal to pack -> merge
        seq = 3
        xchg_place(bufs[0], seq & 1, 1, peer, seq)
        out, o32, l2 = ext.exchange_merge(o, lse, bp, fp, 0, seq)
        want = ext.merge_packed(torch.stack([ext.pack_partial(o, lse), peer]).contiguous())
        assert ext.device_status() == 0
        assert torch.equal(o32, want[1]) and torch.equal(l2, want[2])
        # the same through the attention kernel's own exchange
        q, k, v, scale, _ = synth.sink_body_case(15, T=4096, B=2)
        qc, kc, vc = cuda(q, k, v)
        ext.decode_exchange(qc, kc, vc, scale, None, None, 4, bp, fp, 0, 4)
        assert ext.device_status() == 0x511
        local = shard.local_partial(qc, kc, vc, scale, num_splits=4)
        seq = 5
        xchg_place(bufs[0], seq & 1, 1, peer, seq)
        _, lse5, _, _, o5, _ = ext.decode_exchange(qc, kc, vc, scale, None, None, 4, bp, fp, 0, seq)
        want = ext.merge_packed(torch.stack([local, peer]).contiguous())
        assert ext.device_status() == 0
        assert torch.equal(o5.view(N, D), want[1]) and torch.equal(lse5.view(N), want[2])
    finally:
        ext.set_option("spin_limit", 0)
    assert ext.get_option("spin_limit") == 1 << 21


def _xchg_rank(rank, world, port, ret):
    import os
    import torch.distributed as dist
    from kvskip_b200 import shard
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        q, k, v, scale, keep = synth.sink_body_case(31, T=16384 + 77, B=2)
        nb = keep.shape[-1]
        lo, hi = shard.block_range(nb, rank, world)
        qc = q.cuda()
        kl, vl = k[:, :, lo * 64:hi * 64].cuda(), v[:, :, lo * 64:hi * 64].cuda()
        xchg = shard.PeerExchange(2 * 32, 128)
        ok = True
        for step in range(4):
            a = shard.decode_sequence_sharded(qc, kl, vl, scale)
            b = shard.decode_sequence_sharded(qc, kl, vl, scale, exchange=xchg)
            ok = ok and torch.equal(a["out_f32"], b["out_f32"]) and torch.equal(a["lse"], b["lse"])
            c = shard.decode_sequence_sharded(qc, kl, vl, scale, exchange=xchg, fused=True)   # one launch in all
            ok = ok and torch.equal(a["out_f32"], c["out_f32"]) and torch.equal(a["lse"], c["lse"])
            ok = ok and torch.equal(a["out"], c["out"])
        if rank == 0:
            ref = oracle.decode_f64(q, k, v, scale)
            ret["err"] = rel_err(b["out_f32"], ref["out"])
        ret[f"ok{rank}"] = bool(ok)
        ret[f"status{rank}"] = int(K.ext().device_status())
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_exchange_merge_two_gpus_matches_all_gather():
    """Two ranks on two GPUs: the fused peer-memory exchange gives the same bits as pack ->
    all-gather -> merge, step after step, and the whole-sequence result matches the CPU oracle."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import os
    import torch.multiprocessing as mp
    ret = mp.Manager().dict()
    mp.spawn(_xchg_rank, args=(2, 29700 + os.getpid() % 200, ret), nprocs=2, join=True)
    assert ret["ok0"] and ret["ok1"], dict(ret)
    assert ret["status0"] == 0 and ret["status1"] == 0
    assert ret["err"] < TOL_F32


@pytest.mark.parametrize("rule,value", [("topp", 0.99), ("topp", 0.9), ("tau", 1e-4), ("tau", 1e-3)])
def test_device_selection_matches_torch_selection(rule, value):
    """The one-launch selection between the two passes against the reference's torch formulation
    (sort + cumulative sum, kernels/kvskip.py:122-147): same kept blocks except where a block sits
    on the threshold within float rounding, same list, weights to float accuracy."""
    q, k, v, scale, _ = synth.body_union_case(3, 8192 + 40)
    q, k, v = cuda(q, k, v)
    first = K.decode(q, k, v, scale, stats=True, load_v=False)
    logw = first["blk_max"] + torch.log(first["blk_sum"])
    keep_t = K.select_blocks(logw, 4, rule, value, 2)
    keep8, bi, bc, w = K.ext().select(first["blk_max"], first["blk_sum"], 0 if rule == "topp" else 1, value, 2)
    keep_d = keep8.bool()
    assert (keep_d != keep_t).float().mean() < 2e-3
    assert 0.05 < keep_d.float().mean() < 0.999
    plan = K.make_plan(keep_d)
    assert torch.equal(bc, plan.block_cnt)
    n = int(bc.max())
    valid = torch.arange(n, device=bi.device)[None, None, :] < bc[..., None]
    assert torch.equal(torch.where(valid, bi[..., :n], 0), torch.where(valid, plan.block_idx[..., :n], 0))
    kq = keep_d.repeat_interleave(4, dim=1)
    lk = logw.masked_fill(~kq, float("-inf")).logsumexp(-1, keepdim=True)
    w_t = torch.exp(first["blk_max"] - lk).masked_fill(~kq, 0.0).view(*keep_d.shape[:2], 4, -1).transpose(2, 3)
    assert torch.allclose(w, w_t, rtol=2e-5, atol=1e-12)
