"""Seeded synthetic inputs with the shapes and sparsity structure of the benchmark configurations.

Everything is drawn from numpy's PCG64 (stable across library versions and machines) in float32
and rounded to bf16 (nearest even) on the host, so the CPU checker and the GPU kernels see the
same bits.  The reference measures on private decode-time dumps of real models; these generators
stand in for them with planted structure (a sink block, per-head "body" blocks aligned with the
query, drifting and jumping queries, repeated token ids), because plain N(0,1) keys give a flat
attention in which nothing can be skipped.
"""

import math
from dataclasses import dataclass

import numpy as np
import torch

BLOCK = 64


def bf16_tensor(x: np.ndarray) -> torch.Tensor:
    """float32 ndarray -> torch.bfloat16 tensor, round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    b = ((u + r) >> 16).astype(np.uint16)
    return torch.from_numpy(b.view(np.int16)).view(torch.bfloat16)


def _unit(x: np.ndarray) -> np.ndarray:
    return x / np.linalg.norm(x, axis=-1, keepdims=True)


def dense_case(seed: int, B: int, T: int, Hq: int = 32, Hkv: int = 8, D: int = 128):
    """K, V ~ N(0,1); q ~ N(0,1)/sqrt(D).  Returns q [B,Hq,D], k, v [B,Hkv,T,D] (bf16), scale."""
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((B, Hq, D), dtype=np.float32) / math.sqrt(D)
    k = rng.standard_normal((B, Hkv, T, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, T, D), dtype=np.float32)
    return bf16_tensor(q), bf16_tensor(k), bf16_tensor(v), D ** -0.5


def sink_case(seed: int, B: int, T: int, D: int = 128, Hq: int = 32, Hkv: int = 8, gain: float = 8.0):
    """Edge-case generator: N(0,1) q/k/v with the keys of token 0 multiplied by `gain`
    (a sink tens of nats above the rest)."""
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((B, Hq, D), dtype=np.float32)
    k = rng.standard_normal((B, Hkv, T, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, T, D), dtype=np.float32)
    k[:, :, 0] *= gain
    return bf16_tensor(q), bf16_tensor(k), bf16_tensor(v), D ** -0.5


def keep_to_plan(keep: torch.Tensor):
    """bool [B,Hkv,nb] -> (block_idx int32 [B,Hkv,nb] kept blocks first ascending, block_cnt int32)."""
    cnt = keep.sum(-1, dtype=torch.int32)
    order = torch.argsort((~keep).to(torch.int8), dim=-1, stable=True).to(torch.int32)
    return order.contiguous(), cnt.contiguous()


def sink_body_case(seed: int, T: int = 4096, B: int = 1, Hq: int = 32, Hkv: int = 8, D: int = 128,
                   body_frac: float = 0.10, body_gain: float = 3.0, sink_gain: float = 5.0,
                   stored_frac: float = 0.30):
    """Single-layer decode step with a sink and a planted body.

    q_dir of a KV head is the unit vector of the mean of its G query vectors.  The keys of a
    random `body_frac` of the blocks get +body_gain*q_dir, block 0 gets +sink_gain*q_dir.
    The stored set is a random `stored_frac` of the blocks plus block 0 and the two newest.
    Returns q, k, v, scale, keep (bool [B,Hkv,nb])."""
    rng = np.random.default_rng(seed)
    G = Hq // Hkv
    nb = math.ceil(T / BLOCK)
    q = rng.standard_normal((B, Hq, D), dtype=np.float32) / math.sqrt(D)
    k = rng.standard_normal((B, Hkv, T, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, T, D), dtype=np.float32)
    qdir = _unit(q.reshape(B, Hkv, G, D).mean(2))                      # [B,Hkv,D]
    keep = np.zeros((B, Hkv, nb), dtype=bool)
    for b in range(B):
        for h in range(Hkv):
            body = rng.permutation(nb)[: max(1, int(round(body_frac * nb)))]
            for blk in body:
                k[b, h, blk * BLOCK:(blk + 1) * BLOCK] += body_gain * qdir[b, h]
            k[b, h, :BLOCK] += sink_gain * qdir[b, h]
            keep[b, h, rng.permutation(nb)[: int(round(stored_frac * nb))]] = True
    keep[..., 0] = True
    keep[..., -2:] = True
    return bf16_tensor(q), bf16_tensor(k), bf16_tensor(v), D ** -0.5, torch.from_numpy(keep)


def body_union_case(seed: int, T: int = 65536, B: int = 1, Hq: int = 32, Hkv: int = 8, D: int = 128,
                    core_frac: float = 0.26, own_frac: float = 0.09, gain: float = 96.0,
                    sink_gain: float = 110.0):
    """Masked / V-skip configuration: every query head has its own body of about
    core_frac + own_frac of the blocks (a core shared by the G heads of a KV head plus a private
    random part), whose keys carry +gain * unit(q_head); the KV-head union is about 55 % of the
    blocks with the defaults.  With |q| ~ 1 and scale 1/sqrt(D) the body stands gain*|q|/sqrt(D)
    nats above the N(0,1) background.  Stored set = union + block 0 + two newest.
    Returns q, k, v, scale, keep."""
    rng = np.random.default_rng(seed)
    G = Hq // Hkv
    nb = math.ceil(T / BLOCK)
    q = rng.standard_normal((B, Hq, D), dtype=np.float32) / math.sqrt(D)
    k = rng.standard_normal((B, Hkv, T, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, T, D), dtype=np.float32)
    qd = _unit(q).reshape(B, Hkv, G, D)
    keep = np.zeros((B, Hkv, nb), dtype=bool)
    kb = k.reshape(B, Hkv, -1, D)
    for b in range(B):
        for h in range(Hkv):
            perm = rng.permutation(nb)
            n_core = int(round(core_frac * nb))
            core, rest = perm[:n_core], perm[n_core:]
            for g in range(G):
                own = rest[rng.random(rest.shape[0]) < own_frac / max(1e-9, 1.0 - core_frac)]
                body = np.concatenate([core, own])
                keep[b, h, body] = True
                for blk in body:
                    kb[b, h, blk * BLOCK:min(T, (blk + 1) * BLOCK)] += gain * qd[b, h, g]
            kb[b, h, :BLOCK] += sink_gain * _unit(qd[b, h].mean(0))
    keep[..., 0] = True
    keep[..., -2:] = True
    return bf16_tensor(q), bf16_tensor(k), bf16_tensor(v), D ** -0.5, torch.from_numpy(keep)


@dataclass
class WalkLayer:
    """One layer of the planner-loop configuration (see planner_walk)."""
    k: torch.Tensor          # [B,Hkv,T0+steps,D] bf16: the whole cache, step t sees the first T0+t+1 tokens
    v: torch.Tensor
    q: torch.Tensor          # [steps,B,Hq,D] bf16
    scale: float


def planner_walk(seed: int, T0: int, steps: int, B: int = 1, Hq: int = 32, Hkv: int = 8, D: int = 128,
                 n_targets: int = 4, target_frac: float = 0.12, gain: float = 100.0, sink_gain: float = 110.0,
                 sigma: float = 0.02, jump_every: int = 24, jump_frac: float = 0.30) -> WalkLayer:
    """Keys/values of one layer and the queries of `steps` decode steps.

    Every KV head owns n_targets (direction u_j, block set S_j) pairs: keys of the blocks in S_j
    carry +gain*u_j; block 0 carries +sink_gain * mean direction.  The G query heads of the KV head
    aim at one target (q = u_j + small per-head offset) and follow a random walk with per-step,
    per-dimension sigma (applied before rounding to bf16).  Every `jump_every` steps a random
    `jump_frac` of the KV heads re-aim at another target, which moves mass outside the stored set."""
    rng = np.random.default_rng(seed)
    G = Hq // Hkv
    T = T0 + steps
    nb0 = T0 // BLOCK
    k = rng.standard_normal((B, Hkv, T, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, T, D), dtype=np.float32)
    u = _unit(rng.standard_normal((B, Hkv, n_targets, D), dtype=np.float32))
    for b in range(B):
        for h in range(Hkv):
            for j in range(n_targets):
                blocks = rng.permutation(nb0)[: max(1, int(round(target_frac * nb0)))]
                for blk in blocks:
                    k[b, h, blk * BLOCK:(blk + 1) * BLOCK] += gain * u[b, h, j]
            k[b, h, :BLOCK] += sink_gain * _unit(u[b, h].mean(0))
    aim = rng.integers(0, n_targets, size=(B, Hkv))
    off = rng.standard_normal((B, Hkv, G, D), dtype=np.float32) / math.sqrt(D) * 0.5
    walk = np.zeros((B, Hkv, G, D), dtype=np.float32)
    qs = np.empty((steps, B, Hq, D), dtype=np.float32)
    for t in range(steps):
        if t and t % jump_every == 0:
            jump = rng.random((B, Hkv)) < jump_frac
            aim = np.where(jump, (aim + 1 + rng.integers(0, n_targets - 1, size=(B, Hkv))) % n_targets, aim)
        walk += sigma * rng.standard_normal((B, Hkv, G, D), dtype=np.float32)
        base = np.take_along_axis(u, aim[..., None, None], axis=2)           # [B,Hkv,1,D]
        qs[t] = (base + off + walk).reshape(B, Hq, D)
    return WalkLayer(bf16_tensor(k), bf16_tensor(v), bf16_tensor(qs), D ** -0.5)


def token_ids_with_repeats(seed: int, n: int, T: int, vocab: int = 128256, repeat_p: float = 0.05,
                           span: int = 8) -> torch.Tensor:
    """Token ids [n, T] uniform over the vocabulary, with planted repeats: with probability
    repeat_p a position starts a copy of `span` tokens taken from a random earlier place, so the
    token-index path (earlier copies of the current token) finds something."""
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, vocab, size=(n, T), dtype=np.int64)
    for r in range(n):
        t = span + 1
        while t < T - span:
            if rng.random() < repeat_p:
                src = int(rng.integers(0, t - span))
                ids[r, t:t + span] = ids[r, src:src + span]
                t += span
            else:
                t += 1
    return torch.from_numpy(ids)


def index_blocks(ids: torch.Tensor, T: int, n_out: int) -> torch.Tensor:
    """Token-index blocks of the step whose current token is ids[:, T-1]: blocks holding an earlier
    copy of it or the position right after one.  uint8 [n, n_out].  (Torch restatement used by the
    host-side driver; same rule as the reference's src/lab.py:149-167.)"""
    x = ids[:, :T]
    same = torch.zeros_like(x, dtype=torch.bool)
    same[:, :T - 1] = x[:, :T - 1] == x[:, T - 1:T]
    pos = same.clone()
    pos[:, 1:] |= same[:, :T - 1]
    nb = math.ceil(T / BLOCK)
    blk = torch.nn.functional.pad(pos, (0, nb * BLOCK - T)).view(-1, nb, BLOCK).any(-1)
    out = torch.zeros(ids.shape[0], n_out, dtype=torch.uint8, device=ids.device)
    out[:, :nb] = blk
    return out


def planner_walk_device(seed: int, T0: int, steps: int, device, B: int = 1, Hq: int = 32, Hkv: int = 8, D: int = 128,
                        n_targets: int = 4, target_frac: float = 0.12, gain: float = 100.0,
                        sink_gain: float = 110.0, sigma: float = 0.02, jump_every: int = 24,
                        jump_frac: float = 0.30) -> WalkLayer:
    """planner_walk with the same construction, drawn on `device` with torch's generator (for the
    benchmark's 32-layer loop, where host generation would take minutes).  Not bit-identical to
    planner_walk: tests that compare against stored goldens use the numpy version."""
    g = torch.Generator(device=device).manual_seed(seed)
    G = Hq // Hkv
    T = T0 + steps
    nb0 = T0 // BLOCK
    k = torch.randn(B, Hkv, T, D, device=device, generator=g)
    u = torch.nn.functional.normalize(torch.randn(B, Hkv, n_targets, D, device=device, generator=g), dim=-1)
    n_t = max(1, int(round(target_frac * nb0)))
    kb = k[:, :, :nb0 * BLOCK].view(B, Hkv, nb0, BLOCK, D)
    for j in range(n_targets):
        sel = torch.rand(B, Hkv, nb0, device=device, generator=g).argsort(-1)[..., :n_t]        # random block set
        add = torch.zeros(B, Hkv, nb0, device=device)
        add.scatter_(-1, sel, 1.0)
        kb += gain * add[..., None, None] * u[:, :, j, None, None, :]
    k[:, :, :BLOCK] += sink_gain * torch.nn.functional.normalize(u.mean(2), dim=-1)[:, :, None, :]
    kbf = k.to(torch.bfloat16)
    del k, kb
    v = torch.randn(B, Hkv, T, D, device=device, generator=g).to(torch.bfloat16)
    aim = torch.randint(0, n_targets, (B, Hkv), device=device, generator=g)
    off = torch.randn(B, Hkv, G, D, device=device, generator=g) / math.sqrt(D) * 0.5
    walk = torch.zeros(B, Hkv, G, D, device=device)
    qs = torch.empty(steps, B, Hq, D, device=device)
    for t in range(steps):
        if t and t % jump_every == 0:
            jump = torch.rand(B, Hkv, device=device, generator=g) < jump_frac
            step = 1 + torch.randint(0, n_targets - 1, (B, Hkv), device=device, generator=g)
            aim = torch.where(jump, (aim + step) % n_targets, aim)
        walk += sigma * torch.randn(B, Hkv, G, D, device=device, generator=g)
        base = torch.gather(u, 2, aim[..., None, None].expand(B, Hkv, 1, D))
        qs[t] = (base + off + walk).reshape(B, Hq, D)
    return WalkLayer(kbf, v, qs.to(torch.bfloat16), D ** -0.5)
