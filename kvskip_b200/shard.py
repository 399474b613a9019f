"""Multi-GPU partitioning of the decode step (one process per GPU, torch.distributed).

The reference is single-GPU; this is the part of the design it has no counterpart for.

Two partitionings, matching how the path shards:
  * by (batch, KV head): every (b, kv head) is independent in every kernel, so ranks own disjoint
    slices of the cache and of the planner state and run the unchanged kernels -- no collective.
  * by sequence, for one very long context: rank r owns a contiguous range of 64-token blocks,
    runs the unchanged attention kernel on its range and produces, per (b, query head), the
    triple (m, l, acc) with m the running max in log2 units, l the sum and acc the un-normalised
    output; the triples are all-gathered (NCCL over NVLink: R x B*Hq x (D+2) floats, 16.6 KB per
    rank at batch 1) and merged on every rank with the split-merge arithmetic in ascending rank
    order.  A normalised local result is itself such a triple: (lse / ln 2, 1, out).
"""

import math

import torch
import torch.distributed as dist

from . import kvskip as K

LOG2E = 1.4426950408889634
BLOCK = 64


def batch_slice(B: int, rank: int, world: int) -> slice:
    """Contiguous slice of the batch owned by `rank` (sizes differ by at most one)."""
    base, extra = divmod(B, world)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


def unit_slices(B: int, Hkv: int, rank: int, world: int):
    """(batch slice, head slice) of the B*Hkv independent units for `rank`: whole batch elements
    when there are enough of them, otherwise KV heads of the same batch elements."""
    if B >= world:
        return batch_slice(B, rank, world), slice(0, Hkv)
    if (B * Hkv) % world:
        raise ValueError(f"B*Hkv={B * Hkv} units do not divide over {world} ranks")
    per = B * Hkv // world                 # heads per rank
    if Hkv % per:
        raise ValueError("a rank's heads must lie inside one batch element")
    first = rank * per
    b, h0 = divmod(first, Hkv)
    return slice(b, b + 1), slice(h0, h0 + per)


def block_range(nb: int, rank: int, world: int):
    """Blocks [lo, hi) of a sequence of nb blocks owned by `rank`."""
    per = -(-nb // world)
    lo = min(nb, rank * per)
    return lo, min(nb, lo + per)


class ExchangeError(RuntimeError):
    """The exchange step of a sequence-sharded decode did not complete: a rank never joined the
    collective (its process died or fell behind), or the process group timed out."""


class CudaBackend:
    """The product backend: the compiled extension (there is no CPU path in this package; tests of
    the host logic pass a stand-in with the same two callables)."""

    def decode(self, q, k, v, scale, plan=None, num_splits=None):
        return K.decode(q, k, v, scale, plan=plan, num_splits=num_splits, out_f32=True)

    def merge(self, acc, ml):
        return K.ext().merge(acc, ml)

    def pack(self, out_f32, lse):
        return K.ext().pack_partial(out_f32, lse)

    def merge_packed(self, parts):
        return K.ext().merge_packed(parts)


def local_partial(q, k_local, v_local, scale, plan=None, num_splits=None, backend=None):
    """Attention over this rank's part of the sequence as a packed (acc, m, l) triple:
    fp32 [B*Hq, D+2] with acc = normalised local output, m = local lse in log2 units, l = 1
    (l = 0 and m = -inf when the rank read nothing)."""
    backend = backend or CudaBackend()
    r = backend.decode(q, k_local, v_local, scale, plan=plan, num_splits=num_splits)
    if hasattr(backend, "pack"):
        return backend.pack(r["out_f32"], r["lse"])         # one small kernel instead of five tensor ops
    B, Hq, D = r["out_f32"].shape
    lse = r["lse"].reshape(B * Hq, 1)
    empty = torch.isinf(lse)
    m = lse * LOG2E
    l = torch.where(empty, torch.zeros_like(lse), torch.ones_like(lse))
    return torch.cat([r["out_f32"].reshape(B * Hq, D), m, l], dim=-1).contiguous()


def merge_partials(parts: torch.Tensor, B: int, Hq: int, backend=None):
    """parts fp32 [R, B*Hq, D+2] -> dict(out bf16 [B,Hq,D], out_f32, lse [B,Hq]) with the split
    merge, ranks in ascending order."""
    R, N, W = parts.shape
    D = W - 2
    backend = backend or CudaBackend()
    if hasattr(backend, "merge_packed"):
        out, o32, lse = backend.merge_packed(parts.contiguous())
        return {"out": out.view(B, Hq, D), "out_f32": o32.view(B, Hq, D), "lse": lse.view(B, Hq)}
    acc = parts[..., :D].contiguous()
    ml = parts[..., D:].contiguous()
    out, o32, lse = backend.merge(acc, ml)
    return {"out": out.view(B, Hq, D), "out_f32": o32.view(B, Hq, D), "lse": lse.view(B, Hq)}


class PeerExchange:
    """Exchange + merge of the per-rank triples in ONE kernel over peer memory, instead of pack ->
    NCCL all-gather -> merge: every rank stores its rows straight into every rank's buffer over
    NVLink as (value, step number) words, waits for its peers' words (bounded) and merges.  Buffers come from
    torch's symmetric memory (one allocation per rank, rendezvous once); results equal the
    all-gather path bit for bit.  All ranks must call it once per step, in the same order."""

    def __init__(self, n_rows: int, D: int, group=None, device=None):
        import os
        # plain peer stores only: no NVLink multicast object is bound to the buffer (a rank that
        # dies while its memory is bound to one can fault its peers' GPUs)
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        group = group or dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        device = device or torch.device("cuda", torch.cuda.current_device())
        # 2 buffer sets x R ranks x rows x (D + 2) words of 8 bytes: (fp32 value, step number)
        n_words = 2 * self.world * n_rows * (D + 2)
        self.mem = symm.empty(2 * n_words, dtype=torch.float32, device=device)
        self.mem.zero_()
        handle = symm.rendezvous(self.mem, group)
        ptrs = [int(p) for p in handle.buffer_ptrs]
        self.buf_ptrs = ptrs
        self.flag_ptrs = [0 for _ in ptrs]         # the flag travels inside every word: no flag arrays
        self.n_rows, self.D, self.seq = n_rows, D, 0
        torch.cuda.synchronize(device)
        dist.barrier(group)                       # every rank's buffer is zero before anyone writes

    def check(self) -> None:
        """Synchronise and raise kvskip.DeviceWaitError if a wait for a peer's rows ran out in one
        of the exchange launches since the last check (the peer is `code & 0xf`).  The waits are
        bounded (`spin_limit` option), so a peer that never arrives costs a delay, not a hang."""
        K.check_status("sequence-sharded exchange")

    def decode(self, q, k_local, v_local, scale, plan=None, num_splits=None):
        """Local attention + exchange + merge in one launch (kvskip_launch_decode_xchg).  Needs at
        least two splits and at most half as many (batch, kv head) pairs as SMs."""
        q = q.squeeze(2) if q.dim() == 4 else q
        B, Hq, D = q.shape
        if num_splits is None:
            n_items = math.ceil(k_local.shape[2] / BLOCK) if plan is None else plan.max_cnt
            num_splits = max(2, K.num_splits_for(B * k_local.shape[1], n_items))
        bi, bc = (None, None) if plan is None else (plan.block_idx, plan.block_cnt)
        self.seq += 1
        out, lse, _, _, o32, _ = K.ext().decode_exchange(q, k_local, v_local, float(scale), bi, bc, int(num_splits),
                                                         self.buf_ptrs, self.flag_ptrs, self.rank, self.seq)
        return {"out": out, "out_f32": o32, "lse": lse}

    def __call__(self, out_f32: torch.Tensor, lse: torch.Tensor):
        self.seq += 1
        return K.ext().exchange_merge(out_f32.reshape(self.n_rows, self.D), lse.reshape(self.n_rows),
                                      self.buf_ptrs, self.flag_ptrs, self.rank, self.seq)


def decode_sequence_sharded(q, k_local, v_local, scale, plan=None, group=None, num_splits=None, backend=None,
                            exchange: "PeerExchange | None" = None, fused: bool = False):
    """One decode step with the sequence split over the ranks of `group`.  k_local / v_local
    hold this rank's block range; `plan` (optional) lists local block indices.  Every rank
    returns the full result.  With `exchange` (a PeerExchange built once for this shape) the
    triples travel by peer stores inside one kernel instead of an all-gather; with `fused` as well
    that kernel is the attention kernel itself (its split merge stores to the peers, waits and
    merges), so the whole step is one launch."""
    B, Hq = q.shape[0], q.shape[1]
    if exchange is not None and fused:
        return exchange.decode(q, k_local, v_local, scale, plan=plan, num_splits=num_splits)
    if exchange is not None:
        r = K.decode(q, k_local, v_local, scale, plan=plan, num_splits=num_splits, out_f32=True)
        out, o32, lse = exchange(r["out_f32"], r["lse"])
        D = o32.shape[-1]
        return {"out": out.view(B, Hq, D), "out_f32": o32.view(B, Hq, D), "lse": lse.view(B, Hq)}
    part = local_partial(q, k_local, v_local, scale, plan=plan, num_splits=num_splits, backend=backend)
    world = dist.get_world_size(group)
    parts = torch.empty(world * part.shape[0], part.shape[1], dtype=part.dtype, device=part.device)
    try:
        dist.all_gather_into_tensor(parts, part, group=group)   # rank-major concatenation
    except RuntimeError as e:   # a rank that never called the collective ends it with the group's timeout
        raise ExchangeError(f"rank {dist.get_rank(group)} of {world}: the all-gather of the per-shard partials "
                            f"failed ({str(e).splitlines()[0][:200]})") from e
    return merge_partials(parts.view(world, *part.shape), B, Hq, backend=backend)


def shard_plan(keep: torch.Tensor, rank: int, world: int):
    """Global bool mask [B,Hkv,nb] -> this rank's local mask over its block range (rebased)."""
    lo, hi = block_range(keep.shape[-1], rank, world)
    return keep[..., lo:hi]
