"""The reference's own callers of the operator API, run UNMODIFIED on top of this package.

format37/kvskip's `src/kvskip_attn.py` (the attention glue: `refresh_fused_step`, `refresh_pre_step`,
`_pack_fused`) and its test scripts `bench/test_planner.py` / `bench/test_decode.py` import the
kernels as `from kernels import kvskip`.  `__graft_entry__.build()` places copies of those files in
the git-ignored folder `baseline/_ref/` when a reference checkout is present; the tests here load
them from there with this repository's `kernels/` package answering the import, and are skipped
where the folder is absent.  Nothing of the reference is stored in this repository.

  * CPU: the fused driver of the reference and this package's `RefreshLayer` walk the same steps
    with the CPU oracle standing in for the kernels on both sides: every state tensor equal.
  * GPU: the same comparison with the real kernels on both sides; the reference's planner test
    `run_layer` (device planner against its Python planner, its own PASS criterion) on seeded
    synthetic inputs in place of its private dumps; the synthetic edge-case block of its decode
    test, executed from its source text.
"""
import importlib.util
import math
import re
import sys
from pathlib import Path

import pytest
import torch

from kvskip_b200 import kvskip as K
from kvskip_b200 import synth
from kvskip_b200.refresh import RefreshConfig, RefreshLayer

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"
STATE_KEYS = ("keep", "lse_ref", "cs_ref", "csum", "lse_att", "age", "calib", "est", "aix", "cs_now", "trig",
              "block_cnt")


def load_caller(name: str, sub: str):
    path = REF / sub / f"{name}.py"
    if not path.exists():
        pytest.skip("the reference's callers are not staged (no reference checkout at build time)")
    import kernels  # noqa: F401  (this repository's alias package: it must answer `from kernels import kvskip`)
    for p in (REF / "bench", REF / "src"):
        if str(p) not in sys.path:
            sys.path.insert(0, str(p))
    if name in sys.modules and getattr(sys.modules[name], "__file__", "") == str(path):
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    try:
        spec.loader.exec_module(mod)
    except ImportError as e:      # a dependency of the caller (transformers, safetensors) is missing here
        del sys.modules[name]
        pytest.skip(f"cannot import the reference's {name}: {e}")
    return mod


def configure(ka, cfg: RefreshConfig, layer: int):
    """The reference's global configuration set to the same policy as `cfg`."""
    c = ka.KVSKIP
    c.reset()
    c.delta, c.max_age, c.local, c.level = cfg.delta, cfg.max_age, cfg.local, cfg.level
    c.calib, c.calib_warm, c.calib_hold = cfg.calib, cfg.calib_warm, cfg.calib_hold
    c.calib_kind, c.calib_auto_ix, c.calib_free = cfg.calib_kind, cfg.calib_auto_ix, cfg.calib_free
    c.dense_heads = tuple((layer, h) for h in cfg.dense_heads)
    c.index_heads = tuple((layer, h) for h in cfg.index_heads)
    c.index_union = cfg.index_union
    c.count, c.record = False, False


def walk_both(ka, cfg, walk, ids, steps, dev, ops=None):
    """The reference's refresh_fused_step and RefreshLayer side by side; asserts equal state."""
    layer_id = 2
    configure(ka, cfg, layer_id)
    mine = RefreshLayer(cfg, ops=ops)
    q, k, v = walk.q.to(dev), walk.k.to(dev), walk.v.to(dev)
    T0 = k.shape[2] - steps
    try:
        for t in range(steps):
            T = T0 + t + 1
            nb = math.ceil(T / 64)
            idx = synth.index_blocks(ids.to(dev), T, nb) if ids is not None else None
            ka.KVSKIP.idx_blocks = idx
            o_ref = ka.refresh_fused_step(layer_id, q[t], k[:, :, :T], v[:, :, :T], walk.scale)
            o_mine = mine.step(q[t], k[:, :, :T], v[:, :, :T], walk.scale, idx)
            assert torch.equal(o_ref, o_mine), f"step {t}: outputs differ"
            f = ka.KVSKIP.state[layer_id]["fused"]
            for key in STATE_KEYS:
                assert torch.equal(f[key], mine.state[key]), f"step {t}: state tensor {key} differs"
            cnt = f["block_cnt"]
            valid = torch.arange(f["block_idx"].shape[-1], device=dev)[None, None, :] < cnt[..., None]
            assert torch.equal(torch.where(valid, f["block_idx"], 0), torch.where(valid, mine.state["block_idx"], 0))
            assert int(cnt.max()) <= nb
    finally:
        ka.KVSKIP.reset()
        ka.KVSKIP.calib, ka.KVSKIP.calib_warm, ka.KVSKIP.calib_kind, ka.KVSKIP.calib_auto_ix = None, (), "logit", None
        ka.KVSKIP.dense_heads, ka.KVSKIP.index_heads, ka.KVSKIP.idx_blocks = (), (), None
    return mine


POLICIES = {
    "plain": RefreshConfig(dense_heads=(6,)),
    "peak_auto": RefreshConfig(calib=0.05, calib_warm=(32, 8), calib_kind="peak", calib_auto_ix=0.001),
    "index_union": RefreshConfig(dense_heads=(6,), index_heads=(2,), index_union=True),
}


@pytest.mark.parametrize("name", ["plain", "peak_auto"])
def test_reference_fused_driver_equals_refresh_layer_on_cpu(monkeypatch, name):
    """Host logic only: the kernels on both sides are the CPU oracle (plan/update in the kernels'
    float order, attention in double precision)."""
    from helpers import OracleOps
    ka = load_caller("kvskip_attn", "src")
    ops = OracleOps()
    # the module the reference imported as `from kernels import kvskip`
    monkeypatch.setattr(ka.K, "decode", lambda q, k, v, scale, plan=None, stats=False, **kw: ops.decode(q, k, v, scale, plan, stats))
    monkeypatch.setattr(ka.K, "ext", lambda: ops)
    steps = 10
    walk = synth.planner_walk(21, 2048 + 30, steps, B=1)
    ids = synth.token_ids_with_repeats(5, 1, 2048 + 30 + steps)
    walk_both(ka, POLICIES[name], walk, ids, steps, torch.device("cpu"), ops=ops)


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(POLICIES))
def test_reference_fused_driver_equals_refresh_layer_on_gpu(name):
    """32 steps of the reference's refresh_fused_step (first step through its Python planner and
    _pack_fused) against RefreshLayer, the CUDA kernels of this package under both: outputs and
    every planner state tensor bit-equal after every step."""
    ka = load_caller("kvskip_attn", "src")
    steps = 32
    walk = synth.planner_walk(22, 8192 + 21, steps, B=2)
    ids = synth.token_ids_with_repeats(6, 2, 8192 + 21 + steps)
    mine = walk_both(ka, POLICIES[name], walk, ids, steps, torch.device("cuda"))
    assert K.ext().device_status() == 0
    assert 0 < int(mine.state["block_cnt"].sum())


@pytest.mark.gpu
@pytest.mark.parametrize("index,calib", [(None, None), ("auto", "peak"), ("union", "add")])
def test_reference_planner_test_passes_on_synthetic_walk(monkeypatch, index, calib):
    """bench/test_planner.py:run_layer unchanged -- device planner against the reference's Python
    planner over 64 steps, its own criterion (identical read sets on >= 97 % of head-steps, output
    error < 1e-2 where identical, corrections within 0.05) -- with its dump loader replaced by a
    seeded synthetic walk (the dumps are private)."""
    tp = load_caller("test_planner", "bench")
    steps = 64
    walk = synth.planner_walk_device(40, 8192 + 7, steps, torch.device("cuda"), B=3)
    monkeypatch.setattr(tp, "load", lambda layer, genres=None: (walk.q, walk.k, walk.v))
    monkeypatch.setattr(tp, "query_at", lambda qd, t: qd[t])
    assert tp.run_layer(9, steps, index=index, calib=calib)
    assert K.ext().device_status() == 0


@pytest.mark.gpu
def test_reference_decode_test_synthetic_edge_block():
    """The synthetic edge-case block of bench/test_decode.py (D = 64, short and ragged contexts,
    more splits than blocks, a sink ~30 nats above the rest), executed from the staged source text
    with the module's own imports; bf16 outputs within 2e-3 of its fp64 reference."""
    td = load_caller("test_decode", "bench")
    src = (REF / "bench" / "test_decode.py").read_text()
    m = re.search(r"^( *)# synthetic edge cases.*?\n(.*?)^\1summ = rep\.summary\(\)", src, re.S | re.M)
    assert m, "the synthetic block was not found in the staged test_decode.py"
    indent = len(m.group(1))
    block = "\n".join(line[indent:] for line in m.group(2).splitlines())
    torch.manual_seed(0)
    ns = dict(vars(td))
    ns["rep"] = td.Report()
    exec(compile(block, "test_decode.py:synthetic", "exec"), ns)   # noqa: S102
    rows = ns["rep"].summary()
    assert len(rows) == 5, rows
    for name, s in rows.items():
        assert s["max"] < 2e-3, (name, s)


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["dense", "vskip2", "vskip1", "vskip1sink", "refresh", "refresh_pre", "refresh_fused",
                                  "replay"])
def test_reference_attention_forward_every_mode(mode):
    """`kvskip_attention_forward` of the reference's HF glue (src/kvskip_attn.py:481-511), unmodified,
    over every mode it dispatches to: eight decode steps on a growing cache.  The dense mode must
    match the fp64 oracle to the bf16 tolerance; the sparse modes (top-p 0.99 sets, tau 1e-4) stay
    within a few per cent of dense on the planted data and produce finite outputs of the right
    shape; the counters of the glue are filled."""
    import types

    import oracle
    ka = load_caller("kvskip_attn", "src")
    dev = torch.device("cuda")
    steps, T0, B = 8, 4096 + 9, 2
    walk = synth.planner_walk(31, T0, steps, B=B)
    q, k, v = walk.q.to(dev), walk.k.to(dev), walk.v.to(dev)
    c = ka.KVSKIP
    c.reset()
    c.mode, c.dense_layers, c.count, c.record = mode, (), True, False
    c.calib, c.calib_warm, c.calib_kind, c.calib_auto_ix, c.dense_heads, c.index_heads = None, (), "logit", None, (), ()
    layer = types.SimpleNamespace(layer_idx=3)
    try:
        if mode == "replay":          # block lists recorded beforehand: here the sink, the newest and every third block
            plans = []
            for t in range(steps):
                nb = math.ceil((T0 + t + 1) / 64)
                keep = torch.zeros(B, 8, nb, dtype=torch.bool, device=dev)
                keep[..., ::3] = True
                keep[..., 0] = True
                keep[..., -2:] = True
                plans.append(K.make_plan(keep, sync=False))
            c.plans = {3: plans}
        worst = 0.0
        for t in range(steps):
            T = T0 + t + 1
            out, _ = ka.kvskip_attention_forward(layer, q[t][:, :, None], k[:, :, :T], v[:, :, :T], None,
                                                 scaling=walk.scale)
            assert out.shape == (B, 1, 32, 128) and torch.isfinite(out).all()
            ref = oracle.decode_f64(walk.q[t], walk.k[:, :, :T], walk.v[:, :, :T], walk.scale)["out"]
            worst = max(worst, float((out[:, 0].double().cpu() - ref).norm() / ref.norm()))
        limit = {"dense": 2e-3, "vskip1": 5e-3, "vskip1sink": 5e-3, "vskip2": 3e-2, "replay": 1.0}.get(mode, 5e-2)
        assert worst < limit, (mode, worst)
        if mode.startswith("refresh"):
            tot = ka.log_totals()
            assert 0 < tot["blocks_read"] <= tot["blocks_total"]
        assert K.ext().device_status() == 0
    finally:
        c.reset()
        c.mode, c.dense_layers, c.plans = "dense", (0,), {}
