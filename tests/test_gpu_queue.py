"""The persistent queue-fed attention kernel (block lists on more pieces than SMs) against the
one-CTA-per-piece kernel: the same pieces and the same merge orders, so every output must be
bit-identical; and against the CPU oracle."""
import math

import pytest
import torch

import oracle
from kvskip_b200 import kvskip as K
from kvskip_b200 import synth
from kvskip_b200.cache import PagedKV

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def default_options():
    yield
    K.ext().set_option("queue", 1)
    K.ext().set_option("min_blocks", 24)


def mixed_lists(B, nb, seed):
    """Lists of very different lengths: a tenth of the blocks, everything, nothing, one block."""
    g = torch.Generator().manual_seed(seed)
    keep = torch.rand(B, 8, nb, generator=g) < 0.1
    keep[..., 0] = True
    keep[..., -2:] = True
    keep[:, 0] = True
    keep[0, 5] = False
    keep[B - 1, 3] = False
    keep[B - 1, 3, nb // 2] = True
    if B > 2:
        keep[1, 1:4] = torch.rand(3, nb, generator=g) < 0.6
    return keep


def both(fn):
    K.ext().set_option("queue", 0)
    a = fn()
    K.ext().set_option("queue", 1)
    b = fn()
    return a, b


@pytest.mark.parametrize("B,T,splits,min_blocks", [(8, 8192 + 13, 9, 24), (8, 8192 + 13, 20, 6), (4, 16384, 64, 24),
                                                    (5, 4096 + 1, 16, 4), (16, 2048, 5, 2)])
@pytest.mark.parametrize("stats", [False, True])
def test_queue_kernel_equals_piece_kernel(B, T, splits, min_blocks, stats):
    q, k, v, scale = synth.dense_case(300 + B, B, T)
    nb = math.ceil(T / 64)
    keep = mixed_lists(B, nb, T)
    qc, kc, vc = q.to(DEV), k.to(DEV), v.to(DEV)
    plan = K.make_plan(keep.to(DEV), sync=False)
    K.ext().set_option("min_blocks", min_blocks)
    a, b = both(lambda: K.decode(qc, kc, vc, scale, plan=plan, stats=stats, out_f32=True, num_splits=splits))
    assert torch.equal(a["out"], b["out"]) and torch.equal(a["out_f32"], b["out_f32"]) and torch.equal(a["lse"], b["lse"])
    if stats:
        assert torch.equal(a["blk_max"], b["blk_max"]) and torch.equal(a["blk_sum"], b["blk_sum"])
    bi, bc = synth.keep_to_plan(keep)
    ref = oracle.decode_f64(q, k, v, scale, bi, bc, stats=stats)
    live = bc.repeat_interleave(4, dim=1) > 0
    err = float((b["out_f32"].double().cpu() - ref["out"])[live].norm() / ref["out"][live].norm())
    assert err < 5e-5, err
    assert torch.allclose(b["lse"].double().cpu()[live], ref["lse"][live], rtol=0, atol=2e-4)
    assert torch.isinf(b["lse"].cpu()[~live]).all() and (b["out_f32"].cpu()[~live] == 0).all()
    if stats:
        assert torch.equal(torch.isfinite(b["blk_max"]).cpu(), torch.isfinite(ref["blk_max"]))
    assert K.ext().device_status() == 0


def test_queue_kernel_back_to_back_and_on_two_streams():
    """The queue head and the per-head counters put themselves back to zero: many launches in a
    row, and launches interleaved on two streams (each stream owns its counters)."""
    B, T = 8, 8192
    q, k, v, scale = synth.dense_case(41, B, T)
    keep = mixed_lists(B, T // 64, 7)
    qc, kc, vc = q.to(DEV), k.to(DEV), v.to(DEV)
    plan = K.make_plan(keep.to(DEV), sync=False)
    K.ext().set_option("queue", 0)
    want = K.decode(qc, kc, vc, scale, plan=plan, out_f32=True, num_splits=12)
    K.ext().set_option("queue", 1)
    for _ in range(30):
        got = K.decode(qc, kc, vc, scale, plan=plan, out_f32=True, num_splits=12)
    assert torch.equal(got["out_f32"], want["out_f32"]) and torch.equal(got["lse"], want["lse"])
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    outs = []
    for i in range(10):
        with torch.cuda.stream(s1 if i % 2 else s2):
            outs.append(K.decode(qc, kc, vc, scale, plan=plan, out_f32=True, num_splits=12))
    torch.cuda.synchronize()
    for r in outs:
        assert torch.equal(r["out_f32"], want["out_f32"]) and torch.equal(r["lse"], want["lse"])
    assert K.ext().device_status() == 0


def test_queue_kernel_device_length_and_pages():
    B, T, cap = 8, 4000, 4608
    q, k, v, scale = synth.dense_case(52, B, cap)
    qc, kc, vc = q.to(DEV), k.to(DEV), v.to(DEV)
    kc[:, :, T:] = float("nan")
    vc[:, :, T:] = float("nan")
    nb, nbc = math.ceil(T / 64), cap // 64
    keep = mixed_lists(B, nb, 9)
    keep[..., -1] = True
    plan = K.make_plan(keep.to(DEV), sync=False)
    wide = torch.zeros(B, 8, nbc, dtype=torch.int32, device=DEV)
    wide[..., :nb] = plan.block_idx
    t_dev = torch.tensor([T], dtype=torch.int32, device=DEV)
    want = K.decode(qc, kc[:, :, :T], vc[:, :, :T], scale, plan=plan, stats=True, out_f32=True, num_splits=10)
    a, b = both(lambda: K.decode(qc, kc, vc, scale, plan=K.Plan(wide, plan.block_cnt, nbc, nbc), stats=True,
                                 out_f32=True, num_splits=10, t_dev=t_dev))
    for r in (a, b):
        assert torch.equal(r["out_f32"], want["out_f32"]) and torch.equal(r["lse"], want["lse"])
        assert torch.equal(r["blk_max"][..., :nb], want["blk_max"])
        assert torch.isfinite(r["out_f32"]).all()
    pg = PagedKV(B * nbc + 5, B, 8, 128, cap, DEV, order="shuffled", seed=3)
    pg.k.fill_(float("nan"))
    pg.v.fill_(float("nan"))
    pg.write(kc[:, :, :T], vc[:, :, :T])
    if T % 64:                                       # rows past T in the last pages: back to NaN
        last = pg.table[:, nb - 1].long()
        pg.k[last, :, T % 64:] = float("nan")
        pg.v[last, :, T % 64:] = float("nan")
    c, d = both(lambda: K.decode(qc, pg.k, pg.v, scale, plan=plan, stats=True, out_f32=True, num_splits=10,
                                 page_table=pg.table, seq_len=T))
    for r in (c, d):
        assert torch.equal(r["out_f32"], want["out_f32"]) and torch.equal(r["lse"], want["lse"])
    assert K.ext().device_status() == 0
