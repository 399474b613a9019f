"""Python front end of the sm_100a decode-attention kernels.

Drop-in for the reference's `kernels/kvskip.py` (format37/kvskip kernels/kvskip.py:24-208): same
module-level names, signatures, defaults and return dictionaries, so `src/kvskip_attn.py` and the
`bench/` scripts of the reference run on top of it unchanged (`from kernels import kvskip` resolves
to this module through the `kernels/` package at the repository root).

    decode(q, k, v, scale)                                  dense
    decode(q, k, v, scale, plan=make_plan(keep))            only the listed blocks are read
    decode(q, k, v, scale, stats=True)                      + per-block max and sum-exp
    decode(q, k, v, scale, stats=True, load_v=False)        statistics only: K is read, V is not
    vskip_one_pass / vskip_two_pass / pv                    V-skip variants

q is [B, Hq, D] or [B, Hq, 1, D]; k, v are [B, Hkv, T, D] views with any batch/head/token strides
and D contiguous.  Blocks are 64 tokens counted from position 0.

There is no CPU path: every call needs the compiled extension and a CUDA device, and raises
otherwise.
"""

import importlib.util
import math
import os
from dataclasses import dataclass
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
TILE = 64
_EXT = None


def ext():
    """The compiled extension module (decode, vskip1, pv, plan, update, read_bw, ...).

    Loaded from the in-tree `_kvskip_ext.so` (from the directory $KVSKIP_BUILD when that is set);
    if it is missing and a CUDA toolkit is present it is built once (`python -m kvskip_b200.build`).  Raises RuntimeError if it cannot be had: nothing
    in this package computes without it."""
    global _EXT
    if _EXT is None:
        from . import build as _build
        so = _build.EXT
        if not so.exists() or not _build.LIB.exists():
            if os.environ.get("KVSKIP_NO_BUILD"):
                raise RuntimeError(f"kvskip_b200: {so} is missing and KVSKIP_NO_BUILD is set")
            try:
                _build.build_all(verbose=bool(os.environ.get("KVSKIP_VERBOSE")))
            except Exception as e:  # noqa: BLE001
                raise RuntimeError("kvskip_b200: the CUDA extension is not built and building it failed "
                                   f"(run `python -m kvskip_b200.build`): {e}") from e
        spec = importlib.util.spec_from_file_location("_kvskip_ext", so)
        mod = importlib.util.module_from_spec(spec)
        try:
            spec.loader.exec_module(mod)
        except Exception as e:  # noqa: BLE001
            raise RuntimeError(f"kvskip_b200: cannot load {so}: {e}") from e
        _EXT = mod
    return _EXT


class DeviceWaitError(RuntimeError):
    """A bounded wait inside a kernel ran out (a load that never arrived, a peer GPU that never
    flagged its rows).  `code` is the kernel's status word: 0x2xx / 0x3xx waits on this GPU's own
    loads, 0x500 + r / 0x510 + r the exchange with rank r of a sequence-sharded step."""

    def __init__(self, code: int, what: str):
        super().__init__(f"{what}: a device-side wait gave up (status word {code:#x}); the results of that launch "
                         "are incomplete")
        self.code = code


def check_status(what: str = "kvskip") -> None:
    """Synchronise the current stream, read the kernels' status word and raise DeviceWaitError if a
    wait timed out (the word is cleared).  Blocks the host: call it where a synchronisation is
    acceptable (end of a decode step, after a failed exchange), or set KVSKIP_CHECK_STATUS=1 to
    have every front-end call do it (debugging)."""
    code = int(ext().device_status())
    if code:
        raise DeviceWaitError(code, what)


def _auto_check(what: str) -> None:
    if os.environ.get("KVSKIP_CHECK_STATUS", "") not in ("", "0"):
        check_status(what)


_SMS: dict = {}


def num_sms() -> int:
    """SMs of the current device (looked up once per device: the query costs microseconds of host
    time, and a decode loop asks on every step)."""
    dev = torch.cuda.current_device()
    n = _SMS.get(dev)
    if n is None:
        n = _SMS[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return n


def num_splits_for(bh: int, n_tiles: int, sms: int | None = None, max_splits: int = 64,
                   min_tiles: int = 4) -> int:
    """Split count for bh = B*Hkv sequences of n_tiles blocks each, one CTA per SM.

    Candidates are scored by how full the last wave is (CTAs / (waves * SMs)) minus a small
    penalty per split, so that of two equally full layouts the one with fewer partials to merge
    wins; a split never gets fewer than `min_tiles` blocks."""
    sms = sms or num_sms()
    choice, top = 1, -1.0
    s = 1
    while s <= max_splits:
        if s > 1 and -(-n_tiles // s) < min_tiles:
            break
        ctas = bh * s
        fill = ctas / (-(-ctas // sms) * sms)
        score = fill - 0.002 * s
        if score > top + 1e-9:
            choice, top = s, score
        s += 1
    return choice


@dataclass
class Plan:
    """Block list of the masked kernel."""
    block_idx: torch.Tensor   # int32 [B, Hkv, >= max_cnt]: blocks to read first, ascending
    block_cnt: torch.Tensor   # int32 [B, Hkv]
    max_cnt: int              # longest list (sizes the split count)
    nb: int


def make_plan(keep: torch.Tensor, sync: bool = True) -> Plan:
    """bool [B, Hkv, nb] -> Plan.  sync=True reads the longest list length back to size the splits;
    sync=False sizes them for nb blocks and never touches the host."""
    nb = keep.shape[-1]
    cnt = keep.sum(-1, dtype=torch.int32).contiguous()
    # stable sort of "dropped" flags: kept blocks come first and stay in ascending order
    order = torch.argsort(keep.logical_not().to(torch.int8), dim=-1, stable=True).to(torch.int32).contiguous()
    return Plan(order, cnt, int(cnt.max()) if sync else nb, nb)


QUEUE_MIN_HEADS = 32      # (batch, kv head) pairs from which block lists go to the persistent queue kernel


def splits_for_unsynced_plan(bh: int, nb: int) -> int:
    """Split count (pieces provisioned per head) for a block list whose true lengths are not known
    on the host (sized for nb).  The tensor-core kernels cut every list into pieces of at least 24
    blocks, so a short list uses few of the provisioned pieces.
      * from 32 (batch, kv head) pairs on, the pieces are pulled from a queue by one persistent CTA
        per SM: 12 pieces per head measured best (a head that reads everything is cut into 12 long
        pieces, which are handed out first; more pieces make the merge of a head the tail of the
        launch);
      * below that every piece is a CTA of its own: enough splits for a head that reads every block
        to spread over many SMs."""
    if bh >= QUEUE_MIN_HEADS and ext().get_option("queue"):
        return max(1, min(12, -(-nb // 24)))
    base = num_splits_for(bh, nb)
    if bh * base <= 2 * num_sms():
        return min(64, max(base, -(-nb // 24)))
    return base


def _q3(q):
    return q.squeeze(2) if q.dim() == 4 else q


def decode(q, k, v, scale: float, *, plan: Plan | None = None, stats: bool = False, load_v: bool = True,
           num_splits: int | None = None, stages: int = 2, out_f32: bool = False, write_p: bool = False,
           t_dev: torch.Tensor | None = None, page_table: torch.Tensor | None = None,
           seq_len: int | None = None) -> dict:
    """One layer's decode attention.  Returns dict(out bf16 [B,Hq,D] (None without load_v),
    lse fp32 [B,Hq], num_splits[, blk_max, blk_sum fp32 [B,Hq,nb]][, out_f32][, p fp16 [B,Hq,nb*64]]).

    t_dev (one-element int32 CUDA tensor, not in the reference): the sequence length is read from
    it on the device; k and v are then views of the whole provisioned cache and their length is
    only a bound (it sizes the launch and the statistics rows).  For captured decode steps.

    page_table (int32 [B, max_pages], not in the reference) with seq_len: k and v are page pools
    [pages, Hkv, 64, D] and block j of sequence b is page page_table[b, j] (`kvskip_b200.cache.PagedKV`)."""
    q = _q3(q)
    B, Hkv, T = q.shape[0], k.shape[1], k.shape[2]
    if page_table is not None:
        if seq_len is None:
            raise ValueError("a paged cache needs seq_len")
        T = int(seq_len)
    if num_splits is None:
        n_items = math.ceil(T / TILE) if plan is None else plan.max_cnt
        # the tensor-core kernel owns an SM; three CTAs of the exact-order kernel share one
        tc = q.shape[-1] == 128 or (q.shape[-1] == 64 and not write_p)
        per_sm = 1 if (tc and ext().get_option("decode_path") != 1) else 3
        if plan is not None and per_sm == 1 and plan.max_cnt == plan.nb and load_v:
            num_splits = splits_for_unsynced_plan(B * Hkv, n_items)
        else:
            num_splits = num_splits_for(B * Hkv, n_items, sms=per_sm * num_sms())
            if (plan is not None and load_v and q.shape[-1] == 128 and per_sm == 1 and B * Hkv >= QUEUE_MIN_HEADS
                    and ext().get_option("queue")):
                # lists of known length on the persistent queue kernel: few, long pieces measured best
                # (every piece costs the consumers a reload of q and of the list, and the merger a merge)
                num_splits = min(num_splits, 8)
    bi, bc = (None, None) if plan is None else (plan.block_idx, plan.block_cnt)
    out, lse, bmax, bsum, o32, pbuf = ext().decode(q, k, v, float(scale), bi, bc, stats, load_v,
                                                   int(num_splits), int(stages), out_f32, write_p, t_dev,
                                                   page_table, int(seq_len or 0))
    _auto_check("decode")
    res = {"out": out if load_v else None, "lse": lse, "num_splits": num_splits}
    if stats:
        res["blk_max"], res["blk_sum"] = bmax, bsum
    if out_f32:
        res["out_f32"] = o32
    if write_p:
        res["p"] = pbuf
    return res


def block_weights(blk_max: torch.Tensor, blk_sum: torch.Tensor) -> torch.Tensor:
    """Softmax mass of every block, [B, Hq, nb], from the statistics outputs."""
    return torch.softmax(blk_max + torch.log(blk_sum), dim=-1)


def always_keep(nb: int, local: int, device) -> torch.Tensor:
    """Blocks every sparse mode reads: block 0 (sink) and the `local` newest."""
    a = torch.zeros(nb, dtype=torch.bool, device=device)
    a[0] = True
    a[-local:] = True
    return a


def select_blocks(logw: torch.Tensor, G: int, rule: str, value: float, local: int = 2) -> torch.Tensor:
    """Block selection per KV head (union over its G query heads) from unnormalised block
    log-weights [B, Hq, nb].  "tau": weight >= value; "topp": fewest blocks whose mass reaches
    value.  Sink and `local` newest blocks are always selected.  Returns bool [B, Hq//G, nb]."""
    B, Hq, nb = logw.shape
    w = torch.softmax(logw, dim=-1)
    if rule == "tau":
        per_head = w >= value
    elif rule == "topp":
        sorted_w, perm = w.sort(dim=-1, descending=True)
        before = sorted_w.cumsum(-1) - sorted_w            # mass of the heavier blocks
        per_head = torch.zeros_like(before, dtype=torch.bool).scatter(-1, perm, before < value)
    else:
        raise ValueError(rule)
    return per_head.view(B, Hq // G, G, nb).any(2) | always_keep(nb, local, logw.device)


def pv_splits(bh: int, max_cnt: int, sms: int | None = None) -> int:
    """Splits of the second pass of the two-pass V-skip (not in the reference, which uses
    num_splits_for): one wave of CTAs -- as many splits per (batch, kv head) as keep the grid within
    the SM count, pieces of at least 16 blocks.  Measured on B200 at 64k with 55 % of the blocks
    selected: batch 4, 4 splits 55 us against 61 us with the reference's 9; batch 8, 2 splits 100 us
    against 104 us with 16; batch 1 (18 splits) and batch 16 (1 split at 32k) as before or better."""
    sms = sms or num_sms()
    return max(1, min(sms // max(1, bh), math.ceil(max_cnt / 16)))


def pv(P, v, blk_scale, plan: Plan, num_splits: int | None = None, out_f32: bool = False,
       t_dev: torch.Tensor | None = None):
    if num_splits is None:
        num_splits = pv_splits(v.shape[0] * v.shape[1], plan.max_cnt)
    return ext().pv(P, v, blk_scale, plan.block_idx, plan.block_cnt, int(num_splits), out_f32, t_dev)


def vskip_two_pass(q, k, v, scale: float, rule: str = "topp", value: float = 0.99, local: int = 2,
                   sync: bool = True, out_f32: bool = False, device_select: bool = True,
                   t_dev: torch.Tensor | None = None) -> dict:
    """Two-pass V-skip: a statistics pass over all of K that also writes P = exp(s - block max) in
    fp16, block selection per GQA union, then a pass over P and V of the selected blocks.
    device_select (not in the reference): the selection between the passes runs as one kernel;
    False gives the reference's torch formulation (sort + cumulative sum).
    t_dev (not in the reference): the length is read on the device by all three launches (k, v are
    views of the whole provisioned cache, sync must be False): for captured decode steps."""
    q = _q3(q)
    B, Hq, _ = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    if t_dev is not None and (sync or not device_select or G != 4):
        raise ValueError("vskip_two_pass with t_dev: sync=False, device_select=True, G = 4")
    first = decode(q, k, v, scale, stats=True, load_v=False, write_p=True, t_dev=t_dev)
    if device_select and G == 4 and rule in ("topp", "tau"):
        # selection, block list and second-pass weights in one launch instead of a dozen torch ops
        keep8, bi, bc, weight = ext().select(first["blk_max"], first["blk_sum"], 0 if rule == "topp" else 1,
                                             float(value), int(local), t_dev, int(k.shape[2]) if t_dev is not None else 0)
        nb = keep8.shape[-1]
        plan = Plan(bi, bc, int(bc.max()) if sync else nb, nb)
        out, o32 = pv(first["p"], v, weight, plan, out_f32=out_f32, t_dev=t_dev)
        keep = keep8.bool()
        res = {"out": out, "keep": keep, "kept_frac": keep.float().mean().item() if sync else None}
        if out_f32:
            res["out_f32"] = o32
        return res
    logw = first["blk_max"] + torch.log(first["blk_sum"])
    keep = select_blocks(logw, G, rule, value, local)
    keep_q = keep.repeat_interleave(G, dim=1)
    lse_kept = logw.masked_fill(~keep_q, float("-inf")).logsumexp(-1, keepdim=True)
    weight = torch.exp(first["blk_max"] - lse_kept).masked_fill(~keep_q, 0.0)
    weight = weight.view(B, Hkv, G, -1).transpose(2, 3).contiguous()          # [B, Hkv, nb, G]
    out, o32 = pv(first["p"], v, weight, make_plan(keep, sync=sync), out_f32=out_f32)
    res = {"out": out, "keep": keep, "kept_frac": keep.float().mean().item() if sync else None}
    if out_f32:
        res["out_f32"] = o32
    return res


def vskip_one_pass(q, k, v, scale: float, tau: float = 1e-4, local: int = 2, num_splits: int | None = None,
                   out_f32: bool = False, count: bool = False, lse_prev: torch.Tensor | None = None,
                   sync: bool = True, page_table: torch.Tensor | None = None, seq_len: int | None = None,
                   t_dev: torch.Tensor | None = None) -> dict:
    """Single-pass V-skip: K is read once; the V block of a tile is read only if some query head of
    the group gives the block an estimated weight >= tau.  The normaliser estimate is `lse_prev`
    (per query head, e.g. the "lse" this function returned one step earlier); without it every
    CTA uses the sink block's log-sum-exp, a lower bound that keeps every block the exact rule
    keeps.  count=True adds "v_tiles" [B, Hkv] (and "kept_frac" when sync).
    page_table with seq_len (not in the reference): k and v are page pools, as in `decode`.
    t_dev (not in the reference): the length is read on the device (k, v views of the whole
    provisioned cache; count with sync=False only): for captured decode steps."""
    q = _q3(q)
    B, Hkv, T = q.shape[0], k.shape[1], k.shape[2]
    if page_table is not None:
        if seq_len is None:
            raise ValueError("a paged cache needs seq_len")
        T = int(seq_len)
    nb = math.ceil(T / TILE)
    if num_splits is None:
        num_splits = num_splits_for(B * Hkv, nb)
    out, lse, o32, cnt = ext().vskip1(q, k, v, float(scale), float(tau), int(local), int(num_splits),
                                      out_f32, count, lse_prev, page_table, int(seq_len or 0), t_dev)
    _auto_check("vskip_one_pass")
    res = {"out": out, "lse": lse, "num_splits": num_splits}
    if out_f32:
        res["out_f32"] = o32
    if count:
        res["v_tiles"] = cnt
        if sync:
            res["kept_frac"] = (cnt.sum() / (B * Hkv * nb)).item()
    return res
