"""Generates the golden vectors under tests/golden/ by running the REFERENCE's own Python code on CPU.

Needs a checkout of format37/kvskip (its location in KVSKIP_REFERENCE); it is only
run by a developer when the fixtures have to be regenerated, never by the tests:

    python tests/golden/make_golden.py

What is imported from the reference (nothing is copied into this repository):
  bench/harness.py      reference_decode, reference_block_stats  (fp64 attention / block statistics)
  kernels/kvskip.py     select_blocks, make_plan, num_splits_for, always_keep  (pure torch / Python)
  src/kvskip_attn.py    refresh_pre_step, the Python planner, with kernels.kvskip.decode replaced by
                        a CPU function built from the two harness functions
  src/lab.py            index_steps  (token-index blocks per decode step)

Inputs are NOT stored: they come from kvskip_b200.synth (numpy PCG64, seeded), which the tests call
again with the same seeds.  Only seeds, parameters and the reference's outputs are written.
"""

import math
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
# the reference checkout: $KVSKIP_REFERENCE, else a directory `reference` beside this repository
REF = Path(os.environ.get("KVSKIP_REFERENCE") or ROOT.parent / "reference")

sys.path.insert(0, str(ROOT))
from kvskip_b200 import synth  # noqa: E402

# the reference's modules: its own `kernels` package must win over this repository's alias package
for p in (REF, REF / "src", REF / "bench"):
    sys.path.insert(0, str(p))
for name in [m for m in sys.modules if m == "kernels" or m.startswith("kernels.")]:
    del sys.modules[name]
import harness  # noqa: E402
from kernels import kvskip as RK  # noqa: E402
assert str(REF) in str(Path(RK.__file__).resolve()), RK.__file__
import kvskip_attn as RA  # noqa: E402
import lab as RL  # noqa: E402

torch.set_grad_enabled(False)


def read_mask(block_idx, block_cnt, nb):
    B, H, n = block_idx.shape
    valid = torch.arange(n)[None, None, :] < block_cnt[..., None]
    m = torch.zeros(B, H, n + 1, dtype=torch.bool)
    m.scatter_(-1, torch.where(valid, block_idx.long(), n), True)
    return m[..., :nb]


def cpu_decode(q, k, v, scale, *, plan=None, stats=False, load_v=True, num_splits=None, stages=2,
               out_f32=False, write_p=False):
    """kernels.kvskip.decode on CPU from the reference's fp64 helpers."""
    if q.dim() == 4:
        q = q.squeeze(2)
    B, Hq, D = q.shape
    Hkv, T = k.shape[1], k.shape[2]
    nb = math.ceil(T / 64)
    keep = None if plan is None else read_mask(plan.block_idx, plan.block_cnt, nb)
    out = harness.reference_decode(q, k, v, scale, keep=keep)
    M, S = harness.reference_block_stats(q, k, scale)
    if keep is not None:
        kq = keep.repeat_interleave(Hq // Hkv, dim=1)
        M = M.masked_fill(~kq, float("-inf"))
        S = S.masked_fill(~kq, 0.0)
    lse = torch.logsumexp(M + torch.log(S), -1)
    d = {"out": out.to(torch.bfloat16) if load_v else None, "lse": lse.float(), "num_splits": 1, "out_f64": out}
    if stats:
        d["blk_max"], d["blk_sum"] = M.float(), S.float()
    return d


def decode_goldens():
    g = {}
    # configuration 1: sink + planted body, dense and masked with statistics
    seed, T = 11, 4096
    q, k, v, scale, keep = synth.sink_body_case(seed, T)
    dense = harness.reference_decode(q, k, v, scale)
    M, S = harness.reference_block_stats(q, k, scale)
    masked = harness.reference_decode(q, k, v, scale, keep=keep)
    g["c1_seed"], g["c1_T"] = seed, T
    g["c1_dense_out"], g["c1_masked_out"] = dense.numpy(), masked.numpy()
    g["c1_blk_max"], g["c1_blk_sum"] = M.numpy(), S.numpy()
    g["c1_keep"] = keep.numpy()
    # selectors and plans on the same statistics
    logw = (M + torch.log(S)).float()
    g["c1_topp099"] = RK.select_blocks(logw, 4, "topp", 0.99, 2).numpy()
    g["c1_topp090"] = RK.select_blocks(logw, 4, "topp", 0.90, 2).numpy()
    g["c1_tau1e3"] = RK.select_blocks(logw, 4, "tau", 1e-3, 2).numpy()
    pl = RK.make_plan(keep)
    g["c1_plan_idx"], g["c1_plan_cnt"], g["c1_plan_max"] = pl.block_idx.numpy(), pl.block_cnt.numpy(), pl.max_cnt
    # edge cases of the reference's test (bench/test_decode.py:168-176): D 64, short and ragged T, sink
    for i, (D, T) in enumerate(((64, 1000), (64, 33), (128, 64), (128, 65), (128, 3000))):
        q, k, v, scale = synth.sink_case(100 + i, 2, T, D)
        g[f"edge{i}_D"], g[f"edge{i}_T"], g[f"edge{i}_seed"] = D, T, 100 + i
        g[f"edge{i}_out"] = harness.reference_decode(q, k, v, scale).numpy()
        M, S = harness.reference_block_stats(q, k, scale)
        g[f"edge{i}_blk_max"], g[f"edge{i}_blk_sum"] = M.numpy(), S.numpy()
    # split heuristic at the B200's SM count
    g["splits_bh"] = np.array([1, 8, 32, 64, 128, 512])
    g["splits_tiles"] = np.array([1, 3, 16, 64, 128, 512, 1024, 8192])
    g["splits_148"] = np.array([[RK.num_splits_for(int(b), int(t), sms=148) for t in g["splits_tiles"]]
                                for b in g["splits_bh"]])
    np.savez_compressed(HERE / "decode_golden.npz", **g)
    print("decode_golden.npz", sum(v.nbytes for v in g.values() if hasattr(v, "nbytes")) // 1024, "KB")


def vskip_goldens():
    """Single-pass V-skip rule as the reference's test states it in fp64 (bench/test_decode.py:132-151)."""
    g = {}
    seed, T = 21, 8192
    q, k, v, scale, _ = synth.body_union_case(seed, T)
    M, S = harness.reference_block_stats(q, k, scale)
    lse_b = M + torch.log(S)
    g["seed"], g["T"] = seed, T
    for tau in (1e-4, 1e-3):
        keep1 = (lse_b - lse_b[..., :1] >= math.log(tau)).view(1, 8, 4, -1).any(2)
        keep1[..., 0] = True
        keep1[..., -2:] = True
        g[f"sink_keep_{tau:g}"] = keep1.numpy()
        g[f"sink_out_{tau:g}"] = harness.reference_decode(q, k, v, scale, keep=keep1).numpy()
        lse_exact = torch.logsumexp(lse_b, -1).float().contiguous()
        keep2 = (lse_b - lse_exact[..., None].double() >= math.log(tau)).view(1, 8, 4, -1).any(2)
        keep2[..., 0] = True
        keep2[..., -2:] = True
        g[f"prev_keep_{tau:g}"] = keep2.numpy()
        g[f"prev_out_{tau:g}"] = harness.reference_decode(q, k, v, scale, keep=keep2).numpy()
        g["lse_exact"] = lse_exact.numpy()
    np.savez_compressed(HERE / "vskip_golden.npz", **g)
    print("vskip_golden.npz")


PLANNER_VARIANTS = {
    # name: (index mode, calib kind, dense heads of the layer)
    "plain": (None, None, (6,)),
    "union": ("union", None, (6,)),
    "only": ("only", None, (6,)),
    "peak_auto": ("auto", "peak", ()),
    "logit": (None, "logit", ()),
    "add_union": ("union", "add", ()),
}
PLANNER_SEED, PLANNER_T0, PLANNER_STEPS, PLANNER_B = 5, 4096 - 24, 48, 2


def planner_goldens():
    """The Python planner (src/kvskip_attn.py:328-396) step by step on the drifting-query
    configuration; the per-step read sets and the final state are what the device planner must
    reproduce (bench/test_planner.py compares exactly these)."""
    RK.decode = cpu_decode
    KV = RA.KVSKIP
    walk = synth.planner_walk(PLANNER_SEED, PLANNER_T0, PLANNER_STEPS, B=PLANNER_B)
    ids = synth.token_ids_with_repeats(PLANNER_SEED + 1, PLANNER_B, PLANNER_T0 + PLANNER_STEPS)
    nb_max = math.ceil((PLANNER_T0 + PLANNER_STEPS) / 64)
    g = {"seed": PLANNER_SEED, "T0": PLANNER_T0, "steps": PLANNER_STEPS, "B": PLANNER_B}
    for name, (index, calib, dense) in PLANNER_VARIANTS.items():
        KV.reset()
        KV.plans.clear()
        KV.delta, KV.max_age, KV.local, KV.level = 0.05, 32, 2, 0.99
        KV.calib, KV.calib_warm, KV.calib_hold = ((0.3 if calib != "peak" else 0.05), (32, 8), 0) if calib \
            else (None, (), 0)
        KV.calib_kind = calib or "logit"
        KV.calib_auto_ix = 0.001 if index == "auto" else None
        KV.dense_heads = tuple((1, h) for h in dense)
        KV.index_heads = ((1, 2),) if index in ("union", "only") else ()
        KV.index_union = index == "union"
        KV.count, KV.record = False, True
        masks = np.zeros((PLANNER_STEPS, PLANNER_B, 8, nb_max), dtype=bool)
        outs = np.zeros((PLANNER_STEPS, PLANNER_B, 32, 128), dtype=np.float32)
        calibs = np.zeros((PLANNER_STEPS, PLANNER_B, 8), dtype=np.float32)
        for t in range(PLANNER_STEPS):
            Tt = PLANNER_T0 + t + 1
            nb = math.ceil(Tt / 64)
            if index:
                KV.idx_blocks = synth.index_blocks(ids, Tt, nb).bool()
            o = RA.refresh_pre_step(1, walk.q[t], walk.k[:, :, :Tt], walk.v[:, :, :Tt], walk.scale)
            masks[t, :, :, :nb] = KV.plans[1][-1].numpy()
            outs[t] = o.float().numpy()
            calibs[t] = KV.state[1]["calib"].numpy()
        st = KV.state[1]
        g[f"{name}_masks"] = np.packbits(masks, axis=-1)
        g[f"{name}_out_last"] = outs[-1]
        g[f"{name}_out_norms"] = np.linalg.norm(outs, axis=-1)
        g[f"{name}_calib"] = calibs
        g[f"{name}_keep"] = st["keep"].numpy()
        g[f"{name}_age"] = st["age"].numpy()
        g[f"{name}_aix"] = st["aix"].numpy()
        g[f"{name}_lse_att"] = st["lse_att"].numpy()
        full = masks[1:].reshape(PLANNER_STEPS - 1, PLANNER_B, 8, -1)
        nbs = np.array([math.ceil((PLANNER_T0 + t + 1) / 64) for t in range(1, PLANNER_STEPS)])
        trig = np.stack([full[i, :, :, :nbs[i]].all(-1) for i in range(PLANNER_STEPS - 1)])
        print(f"planner {name}: refreshing head-steps {int(trig.sum())}/{trig.size}, "
              f"blocks read {masks[1:].sum() / (trig.size * nbs.mean()):.2%}, "
              f"calib max {calibs.max():.3f}, latched {int(st['aix'].sum())}")
    g["nb_max"] = nb_max
    np.savez_compressed(HERE / "planner_golden.npz", **g)
    print("planner_golden.npz")


def index_goldens():
    P, S = 1000, 40
    ids = synth.token_ids_with_repeats(31, 3, P + S, vocab=5000, repeat_p=0.1)
    steps = RL.index_steps(ids, P, S)
    nb_max = math.ceil((P + S) / 64)
    out = np.zeros((S, 3, nb_max), dtype=bool)
    for t, m in enumerate(steps):
        out[t, :, :m.shape[1]] = m.numpy()
    np.savez_compressed(HERE / "index_golden.npz", seed=31, P=P, S=S, vocab=5000, repeat_p=0.1, blocks=out)
    print("index_golden.npz", int(out.sum()), "marked blocks")


if __name__ == "__main__":
    which = sys.argv[1:] or ["decode", "vskip", "planner", "index"]
    if "decode" in which:
        decode_goldens()
    if "vskip" in which:
        vskip_goldens()
    if "index" in which:
        index_goldens()
    if "planner" in which:
        planner_goldens()
