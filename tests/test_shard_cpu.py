"""Multi-rank host logic on CPU: ownership of units and the sequence-sharded exchange + merge,
run as two `gloo` ranks with the CPU oracle standing in for the kernels."""
import math
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from kvskip_b200 import shard, synth


class OracleBackend:
    def decode(self, q, k, v, scale, plan=None, num_splits=None):
        bi, bc = (None, None) if plan is None else (plan.block_idx, plan.block_cnt)
        r = oracle.decode_f64(q, k, v, scale, bi, bc)
        return {"out_f32": r["out"].float(), "lse": r["lse"].float()}

    def merge(self, acc, ml):
        out, lse = oracle.combine_f32(acc.transpose(0, 1).contiguous(), ml.transpose(0, 1).contiguous())
        return out.to(torch.bfloat16), out, lse


def test_ownership_covers_every_unit_once():
    for B, Hkv, world in ((64, 8, 8), (64, 8, 4), (5, 8, 2), (1, 8, 8), (1, 8, 2), (2, 8, 4)):
        seen = torch.zeros(B, Hkv, dtype=torch.int32)
        for r in range(world):
            bs, hs = shard.unit_slices(B, Hkv, r, world)
            seen[bs, hs] += 1
        assert (seen == 1).all(), (B, Hkv, world)
    for nb, world in ((8192, 8), (1024, 3), (5, 8)):
        cover = []
        for r in range(world):
            lo, hi = shard.block_range(nb, r, world)
            cover += list(range(lo, hi))
        assert cover == list(range(nb))
    with pytest.raises(ValueError):
        shard.unit_slices(1, 8, 0, 3)


def _rank(rank, world, port, T, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v, scale, keep = synth.sink_body_case(77, T=T, B=2)
        nb = math.ceil(T / 64)
        lo, hi = shard.block_range(nb, rank, world)
        kl, vl = k[:, :, lo * 64:min(T, hi * 64)], v[:, :, lo * 64:min(T, hi * 64)]
        be = OracleBackend()
        dense = shard.decode_sequence_sharded(q, kl, vl, scale, backend=be)
        local_keep = shard.shard_plan(keep, rank, world)
        bi, bc = synth.keep_to_plan(local_keep)
        from kvskip_b200.kvskip import Plan
        masked = shard.decode_sequence_sharded(q, kl, vl, scale, plan=Plan(bi, bc, int(bc.max()), hi - lo), backend=be)
        if rank == 0:
            ref = oracle.decode_f64(q, k, v, scale)
            gbi, gbc = synth.keep_to_plan(keep)
            refm = oracle.decode_f64(q, k, v, scale, gbi, gbc)
            ret["dense"] = float((dense["out_f32"].double() - ref["out"]).norm() / ref["out"].norm())
            ret["dense_lse"] = float((dense["lse"].double() - ref["lse"]).abs().max())
            ret["masked"] = float((masked["out_f32"].double() - refm["out"]).norm() / refm["out"].norm())
            ret["masked_lse"] = float((masked["lse"].double() - refm["lse"]).abs().max())
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T", [2048, 1000])
def test_sequence_sharded_two_gloo_ranks(T):
    """Each rank attends its block range, (acc, m, l) triples are all-gathered, every rank merges."""
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + (os.getpid() + T) % 2000
    mp.spawn(_rank, args=(2, port, T, ret), nprocs=2, join=True)
    assert ret["dense"] < 1e-6 and ret["masked"] < 1e-6, dict(ret)
    assert ret["dense_lse"] < 1e-5 and ret["masked_lse"] < 1e-5, dict(ret)


def _rank_missing_peer(rank, world, port, ret):
    """Rank 1 never joins the exchange of the step (a host-side failure: it stays alive but skips
    the collective); rank 0 must get an error from the step instead of waiting for ever."""
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    try:
        q, k, v, scale, _ = synth.sink_body_case(78, T=512, B=1)
        lo, hi = shard.block_range(8, rank, world)
        kl, vl = k[:, :, lo * 64:hi * 64], v[:, :, lo * 64:hi * 64]
        be = OracleBackend()
        good = shard.decode_sequence_sharded(q, kl, vl, scale, backend=be)       # a step both ranks take
        ret[f"good{rank}"] = bool(torch.isfinite(good["out_f32"]).all())
        if rank == 0:
            t0 = time.time()
            try:
                shard.decode_sequence_sharded(q, kl, vl, scale, backend=be)      # rank 1 is not coming
                ret["raised"] = "nothing"
            except shard.ExchangeError as e:
                ret["raised"] = "ExchangeError"
                ret["message"] = str(e)
            ret["waited_s"] = time.time() - t0
        else:
            time.sleep(6.0)          # alive, between steps, no collective in flight
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001  (the group of the rank that saw the timeout is already broken)
            pass


def test_missing_rank_ends_the_exchange_with_an_error():
    """Failure detection on the host: a rank that skips the all-gather makes the other rank's step
    end with shard.ExchangeError after the process group's (short) timeout."""
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 31500 + os.getpid() % 2000
    mp.spawn(_rank_missing_peer, args=(2, port, ret), nprocs=2, join=True)
    assert ret["good0"] and ret["good1"]
    assert ret["raised"] == "ExchangeError", dict(ret)
    assert "rank 0 of 2" in ret["message"]
    assert ret["waited_s"] < 30
