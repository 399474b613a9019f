"""Host-side driver of the refresh policy: plan -> masked attention with block statistics -> update.

Mirrors what the reference's caller does around the kernels (format37/kvskip
src/kvskip_attn.py:402-478, `refresh_fused_step` with `_pack_fused` / `_grow_fused`, and the first
step of `refresh_pre_step`, :339-354): the first decode step of a layer runs a dense pass with
block statistics and builds the planner state with torch ops; every later step is three launches
on the current stream with no host synchronisation.  The state tensors keep the reference's names
and layouts, so they can be handed to either implementation.

The compute backend is `ops`: by default the CUDA extension (there is no CPU path in this
package).  Tests pass a CPU stand-in with the same three callables to check the driver logic.
"""

import math
from dataclasses import dataclass, field

import torch

from . import kvskip as K

BLOCK = 64
CALIB_KINDS = {"logit": 0, "add": 1, "peak": 2}


@dataclass
class RefreshConfig:
    level: float = 0.99            # top-p mass of a stored set
    delta: float = 0.05            # refresh when the estimated missed mass exceeds this
    max_age: int = 32              # forced refresh after this many steps
    local: int = 2                 # newest blocks always read
    dense_heads: tuple = ()        # kv heads refreshed on every step
    index_heads: tuple = ()        # kv heads driven by the token index
    index_union: bool = False      # index blocks join the attended set instead of replacing it
    calib: float | None = None     # rate of the online correction of the estimate (None: off)
    calib_hold: int = 0            # steps before the correction is applied
    calib_warm: tuple = ()         # (W, A): max age A during the first W steps
    calib_free: bool = False
    calib_kind: str = "logit"      # "logit" | "add" | "peak"
    calib_auto_ix: float | None = None   # latch a head onto the token index when its correction exceeds this
    margin: int = 64               # spare block capacity of the state tensors


class CudaOps:
    """The product backend: the compiled extension."""

    def decode(self, q, k, v, scale, plan=None, stats=False):
        return K.decode(q, k, v, scale, plan=plan, stats=stats)

    def plan(self, *a):
        return K.ext().plan(*a)

    def update(self, *a):
        return K.ext().update(*a)

    def fused_step(self, *a, **kw):
        """plan -> masked+stats attention -> update in one extension call."""
        return K.ext().refresh_step(*a, **kw)


def centroid_sums(k: torch.Tensor) -> torch.Tensor:
    """Per-block sums of keys, fp32 [B, Hkv, nb, D] (the last block may be partial)."""
    B, H, T, D = k.shape
    nb, full = math.ceil(T / BLOCK), T // BLOCK
    out = torch.zeros(B, H, nb, D, dtype=torch.float32, device=k.device)
    if full:
        out[:, :, :full] = k[:, :, :full * BLOCK].unflatten(2, (full, BLOCK)).sum(3, dtype=torch.float32)
    if T > full * BLOCK:
        out[:, :, full] = k[:, :, full * BLOCK:].sum(2, dtype=torch.float32)
    return out


def centroid_scores(q32, csum, T, scale):
    """q . (block key mean) * scale, [B, Hq, nb]."""
    nb = csum.shape[2]
    sizes = torch.full((nb,), float(BLOCK), device=csum.device)
    sizes[-1] = T - BLOCK * (nb - 1)
    cen = csum / sizes[None, None, :, None]
    B, Hq, D = q32.shape
    Hkv = cen.shape[1]
    return torch.einsum("bkgd,bknd->bkgn", q32.view(B, Hkv, Hq // Hkv, D), cen).reshape(B, Hq, nb) * scale


class PlannerState:
    """The device planner's tensors of one layer, carved out of ONE allocation.

    Names, shapes and dtypes are the ones the kernels take (and the reference's fused driver
    keeps, src/kvskip_attn.py:420-432), so the views can be handed to either implementation; the
    storage is this package's: a single byte arena per layer with 256-byte aligned segments, sized
    for `nbc` blocks of capacity.  One allocation per layer keeps a long decode loop free of
    allocator traffic, makes a layer's planner state one tensor to save or move, and growing it is
    one new arena plus a copy of the used prefix of the per-block segments."""

    # name -> (dtype, shape as a function of the geometry, value of unused block capacity or None)
    LAYOUT = (
        ("csum", torch.float32, lambda g: (g.B, g.Hkv, g.nbc, g.D), 0.0),
        ("lse_ref", torch.float32, lambda g: (g.B, g.Hq, g.nbc), float("-inf")),
        ("cs_ref", torch.float32, lambda g: (g.B, g.Hq, g.nbc), 0.0),
        ("cs_now", torch.float32, lambda g: (g.B, g.Hq, g.nbc), 0.0),
        ("block_idx", torch.int32, lambda g: (g.B, g.Hkv, g.nbc), 0),
        ("keep", torch.uint8, lambda g: (g.B, g.Hkv, g.nbc), 0),
        ("lse_att", torch.float32, lambda g: (g.B, g.Hq), None),
        ("calib", torch.float32, lambda g: (g.B, g.Hkv), None),
        ("est", torch.float32, lambda g: (g.B, g.Hkv), None),
        ("age", torch.int32, lambda g: (g.B, g.Hkv), None),
        ("block_cnt", torch.int32, lambda g: (g.B, g.Hkv), None),
        ("flags", torch.int32, lambda g: (g.Hkv,), None),
        ("aix", torch.uint8, lambda g: (g.B, g.Hkv), None),
        ("trig", torch.uint8, lambda g: (g.B, g.Hkv), None),
    )

    def __init__(self, B, Hq, Hkv, D, nbc, device, scale=1.0):
        self.B, self.Hq, self.Hkv, self.D, self.nbc, self.scale = B, Hq, Hkv, D, int(nbc), float(scale)
        offsets, total = [], 0
        for _, dtype, shape, _ in self.LAYOUT:
            n = math.prod(shape(self)) * torch.empty((), dtype=dtype).element_size()
            offsets.append((total, n))
            total += (n + 255) & ~255
        self.arena = torch.zeros(total, dtype=torch.uint8, device=device)
        self.views = {}
        for (name, dtype, shape, fill), (off, n) in zip(self.LAYOUT, offsets):
            view = self.arena[off:off + n].view(dtype).view(shape(self))
            if fill:                       # a zero fill is already there
                view.fill_(fill)
            self.views[name] = view
        v = self.views     # the state tensors in the order the fused step takes them
        self.step_args = (v["csum"], v["lse_ref"], v["cs_ref"], v["keep"], v["lse_att"], v["age"], v["flags"],
                          v["cs_now"], v["trig"], v["block_idx"], v["block_cnt"])

    # dictionary-style access under the reference's key names ("NBC" and "scale" included)
    def __getitem__(self, key):
        if key == "NBC":
            return self.nbc
        if key == "scale":
            return self.scale
        return self.views[key]

    def __contains__(self, key):
        return key in self.views or key in ("NBC", "scale")

    def load_blocks(self, name, x):
        """Write x into the first x.shape[2] blocks of a per-block tensor."""
        self.views[name][:, :, :x.shape[2]] = x

    def grown(self, nbc):
        """A state with capacity for nbc blocks holding this one's contents."""
        new = PlannerState(self.B, self.Hq, self.Hkv, self.D, nbc, self.arena.device, self.scale)
        for name, _, _, fill in self.LAYOUT:
            if fill is None:
                new.views[name].copy_(self.views[name])
            else:
                new.views[name][:, :, :self.nbc] = self.views[name]
        return new


@dataclass
class RefreshLayer:
    """overlap_update (CUDA backend, eager steps): `update` runs on a second stream owned by the
    layer.  The attention output does not depend on it -- it prepares this layer's next step -- so
    the launches that follow on the current stream (the rest of the model, the next layer's plan)
    need not wait for it.  The layer joins the current stream with that stream before its next
    step and whenever `state` is read through this object; tensors taken from `state` earlier and
    kept by the caller are only safe to read after `join()`.  Inside a stream capture the step
    stays one chain (`kvskip_b200.graph.StepGraph` forks and joins inside the graph itself)."""
    cfg: RefreshConfig
    ops: object = None
    t: int = 0
    last: dict = field(default_factory=dict)     # tensors of the latest step (block lists, stats), for inspection
    overlap_update: bool = True
    OVERLAP_MIN_WORK = 8192

    def __post_init__(self):
        if self.ops is None:
            self.ops = CudaOps()
        self._state = None
        self._ov = 0
        self._ns_key, self._ns = None, 1

    @property
    def state(self):
        self.join()
        return self._state

    @state.setter
    def state(self, st):
        self._state = st

    def join(self) -> None:
        """The current stream waits for this layer's latest `update` (no-op without one in flight)."""
        if self._ov:
            K.ext().overlap_join(self._ov)

    def _overlap_handle(self, work: int) -> int:
        # below about 8k (batch x kv head x block) units (batch 1 under 64k tokens) a step is shorter
        # than the host needs to issue it, and the fork and join (about 8 us of host time) only add to that:
        # batch 1 at 64k 59 -> 51 us per layer-step with the second stream, at 32k 45 -> 51 us
        if not self.overlap_update or not isinstance(self.ops, CudaOps) or work < self.OVERLAP_MIN_WORK:
            return 0
        if not self._ov:
            self._ov = K.ext().overlap_create()
        return self._ov

    def __del__(self):
        ov = getattr(self, "_ov", 0)
        if ov:
            try:
                K.ext().overlap_join(ov)      # before the tensors of the last step are released
                K.ext().overlap_destroy(ov)
            except Exception:   # interpreter shutdown: the extension may be gone
                pass
            self._ov = 0

    # ---- first decode step: dense + statistics, state built with torch ops ------------------
    def _init(self, q, k, v, scale):
        cfg = self.cfg
        B, Hq, D = q.shape
        Hkv, T = k.shape[1], k.shape[2]
        G = Hq // Hkv
        nb = math.ceil(T / BLOCK)
        dev = q.device
        r = self.ops.decode(q, k, v, scale, stats=True)
        logw = r["blk_max"] + torch.log(r["blk_sum"])
        csum = centroid_sums(k)
        keep = K.select_blocks(logw, G, "topp", cfg.level, cfg.local)
        cs = centroid_scores(q.float(), csum, T, scale)
        always = K.always_keep(nb, cfg.local, dev)
        lse_att = logw.masked_fill(~(keep | always).repeat_interleave(G, dim=1), float("-inf")).logsumexp(-1)
        st = PlannerState(B, Hq, Hkv, D, nb + cfg.margin, dev, scale)
        st.load_blocks("keep", keep)
        st.load_blocks("lse_ref", logw)
        st.load_blocks("cs_ref", cs)
        st.load_blocks("csum", csum)
        st["lse_att"].copy_(lse_att)
        for h in cfg.dense_heads:
            st["flags"][h] = 1
        for h in cfg.index_heads:
            st["flags"][h] = 4 if cfg.index_union else 2
        self.state = st
        self.t = 0
        self.last = {"blk_max": r["blk_max"], "blk_sum": r["blk_sum"], "lse": r["lse"], "first": True}
        return r["out"]

    def _grow(self, NBC):
        self.state = self.state.grown(NBC)

    def max_age_now(self) -> int:
        cfg = self.cfg
        if cfg.calib_warm and self.t < cfg.calib_warm[0]:
            return min(cfg.max_age, cfg.calib_warm[1])
        return cfg.max_age

    def graph_scalars(self) -> tuple:
        """The host-decided scalars the next step passes to the kernels; a captured step is valid
        while they stay the same (`kvskip_b200.graph.StepGraph`)."""
        cfg, t = self.cfg, self.t + 1
        max_age = min(cfg.max_age, cfg.calib_warm[1]) if cfg.calib_warm and t < cfg.calib_warm[0] else cfg.max_age
        return (max_age, cfg.calib is not None and t >= cfg.calib_hold)

    def note_replayed(self) -> None:
        """A captured step of this layer was replayed: keep the step counter in step."""
        self.t += 1

    def uses_index(self) -> bool:
        return bool(self.cfg.index_heads) or self.cfg.calib_auto_ix is not None

    # ---- one decode step ------------------------------------------------------------------
    def step(self, q, k, v, scale, idx_blocks=None, t_dev=None, update_stream=None, page_table=None, seq_len=None):
        """q [B,Hq,D]; k, v [B,Hkv,T,D] views that already hold the token of this step at T-1.
        idx_blocks: bool/uint8 [B, >= nb] token-index blocks of this step (index heads / auto latch).
        t_dev: one-element int32 CUDA tensor holding the sequence length; k and v are then views of
        the whole provisioned cache (their length is a bound) and the three launches can be captured
        in a CUDA graph and replayed while the length grows (see `kvskip_b200.graph`).
        update_stream: a second CUDA stream for `update`.  The attention output does not depend on
        it (it prepares this layer's next step), so it can overlap whatever follows on the current
        stream; the caller makes the current stream wait for update_stream before this layer's
        next step (e.g. once at the end of a decode step).
        page_table, seq_len: k and v are page pools [pages,Hkv,64,D] and page_table int32
        [B, max_pages] names the page of every block (`kvskip_b200.cache.PagedKV`); seq_len is the
        length (the bound, with t_dev).  The first step of a layer needs contiguous views.
        Returns out bf16 [B,Hq,D]."""
        if q.dim() == 4:
            q = q.squeeze(2)
        paged = page_table is not None
        self.join()                        # once; below the state is taken without another join
        if paged and (seq_len is None or self._state is None or not hasattr(self.ops, "fused_step")):
            raise ValueError("a paged cache needs seq_len, the CUDA backend, and a first step on contiguous views")
        if self._state is None:
            if t_dev is not None:
                raise ValueError("the first step of a layer builds the state on the host: run it with views of "
                                 "the current length and without t_dev")
            return self._init(q, k, v, scale)
        cfg = self.cfg
        B, T = q.shape[0], (int(seq_len) if paged else k.shape[2])
        nb = math.ceil(T / BLOCK)
        if nb > self._state.nbc:
            self._grow(nb + cfg.margin)
        s = self._state
        idx = None
        if self.uses_index():
            if idx_blocks is None:
                raise ValueError("this configuration needs idx_blocks on every step")
            if idx_blocks.dtype == torch.uint8 and idx_blocks.shape[1] == s["NBC"] and idx_blocks.is_contiguous():
                idx = idx_blocks
            else:
                idx = torch.zeros(B, s["NBC"], dtype=torch.uint8, device=q.device)
                idx[:, :nb] = idx_blocks[:, :nb]
        self.t += 1
        cal = cfg.calib is not None
        kind = CALIB_KINDS[cfg.calib_kind]
        auto = cfg.calib_auto_ix is not None
        if hasattr(self.ops, "fused_step") and update_stream is not None:
            ns = K.splits_for_unsynced_plan(B * k.shape[1], nb)
            ext = K.ext()
            ext.plan(q, k, s["csum"], s["lse_ref"], s["cs_ref"], s["keep"], s["lse_att"], s["age"], s["flags"],
                     s["cs_now"], s["trig"], s["block_idx"], s["block_cnt"], float(scale), float(cfg.delta),
                     int(self.max_age_now()), int(cfg.local), True, idx, s["calib"] if cal else None, s["est"],
                     bool(cal and self.t >= cfg.calib_hold), kind, s["aix"] if auto else None, t_dev, page_table, T)
            out, lse, bmax, bsum, _, _ = ext.decode(q, k, v, float(scale), s["block_idx"], s["block_cnt"], True, True,
                                                    int(ns), 2, False, False, t_dev, page_table, T)
            update_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(update_stream):
                ext.update(bmax, bsum, s["trig"], s["cs_now"], s["keep"], s["lse_ref"], s["cs_ref"], s["lse_att"], T,
                           float(cfg.level), int(cfg.local), s["flags"], idx, s["est"], s["calib"] if cal else None,
                           float(cfg.calib or 0.0), bool(cfg.calib_free), kind, s["aix"] if auto else None,
                           float(cfg.calib_auto_ix or 0.0), t_dev)
            # the statistics stay referenced here until this layer's next step, past the join
            self.last = {"blk_max": bmax, "blk_sum": bsum, "lse": lse, "first": False}
            return out
        if hasattr(self.ops, "fused_step"):
            bh = B * k.shape[1]
            if self._ns_key != (bh, nb):                         # sized for every block: no host sync
                self._ns_key, self._ns = (bh, nb), int(K.splits_for_unsynced_plan(bh, nb))
            a = s.step_args
            args = (q, k, v, *a, float(scale), float(cfg.delta), int(self.max_age_now()), int(cfg.local),
                    float(cfg.level), self._ns, idx, s.views["calib"] if cal else None, s.views["est"],
                    bool(cal and self.t >= cfg.calib_hold), kind, float(cfg.calib or 0.0), bool(cfg.calib_free),
                    s.views["aix"] if auto else None, float(cfg.calib_auto_ix or 0.0), t_dev, page_table, T)
            if isinstance(self.ops, CudaOps):                    # straight to the extension, one call
                out, lse, bmax, bsum = K.ext().refresh_step(*args, self._overlap_handle(bh * nb))
            else:
                out, lse, bmax, bsum = self.ops.fused_step(*args)
            # (with `update` on the layer's own stream these stay referenced until the join of the next step)
            self.last = {"blk_max": bmax, "blk_sum": bsum, "lse": lse, "first": False, "idx": idx}
            return out
        if t_dev is not None:
            raise ValueError("a device-resident length needs a backend with fused_step")
        self.ops.plan(q, k, s["csum"], s["lse_ref"], s["cs_ref"], s["keep"], s["lse_att"], s["age"], s["flags"],
                      s["cs_now"], s["trig"], s["block_idx"], s["block_cnt"], float(scale), float(cfg.delta),
                      int(self.max_age_now()), int(cfg.local), True, idx, s["calib"] if cal else None, s["est"],
                      bool(cal and self.t >= cfg.calib_hold), kind, s["aix"] if auto else None)
        r = self.ops.decode(q, k, v, scale, plan=K.Plan(s["block_idx"], s["block_cnt"], nb, nb), stats=True)
        self.ops.update(r["blk_max"], r["blk_sum"], s["trig"], s["cs_now"], s["keep"], s["lse_ref"], s["cs_ref"],
                        s["lse_att"], T, float(cfg.level), int(cfg.local), s["flags"], idx, s["est"],
                        s["calib"] if cal else None, float(cfg.calib or 0.0), bool(cfg.calib_free), kind,
                        s["aix"] if auto else None, float(cfg.calib_auto_ix or 0.0))
        self.last = {"blk_max": r["blk_max"], "blk_sum": r["blk_sum"], "lse": r["lse"], "first": False}
        return r["out"]

    def read_mask(self, nb: int) -> torch.Tensor:
        """bool [B,Hkv,nb]: the blocks the latest step read (from block_idx / block_cnt)."""
        s = self.state
        bi, bc = s["block_idx"], s["block_cnt"]
        n = bi.shape[-1]
        valid = torch.arange(n, device=bi.device)[None, None, :] < bc[..., None]
        m = torch.zeros(*bi.shape[:2], n + 1, dtype=torch.bool, device=bi.device)
        m.scatter_(-1, torch.where(valid, bi.long(), n), True)
        return m[..., :nb]
