"""KV caches either side of the decode kernels: a growing contiguous cache and a paged one.

`GrowingKV` has the behaviour of the reference's cache layer (format37/kvskip
src/kvskip_attn.py:67-113, `GrowingLayer`): one [B,Hkv,capacity,D] buffer per tensor that doubles
when it runs out, capacity a multiple of the 64-token block, `update()` returning views of the
current length, `crop()`.  It does not depend on transformers; an HF cache layer can delegate to it.
A single decode token is written by the library's append kernel (one launch for K and V), which
can also take the length from device memory, so the append is part of a captured step.

`PagedKV` stores the cache in 64-token pages, [pages,Hkv,64,D] per tensor, with a page table
int32 [B, max_pages]: block j of sequence b lives in page table[b, j].  The attention kernels read
a block straight from its page (the tensor map runs over the pool), so the planner's block list
and the page table together decide which pages a step touches; nothing is gathered.  The reference
reads [B,Hkv,T,D] views only; its notes name this layout as the natural one for block skipping
(docs/03-gate-digest.md:364).
"""

import math

import torch

from . import kvskip as K

BLOCK = 64


class GrowingKV:
    """One layer's contiguous cache.  capacity: tokens to allocate at first (no doubling below it)."""

    def __init__(self, capacity: int = 0):
        self.capacity = capacity
        self._k = self._v = None
        self._n = 0

    def _ensure(self, need: int, ref: torch.Tensor) -> None:
        cap = 0 if self._k is None else self._k.shape[-2]
        if need <= cap:
            return
        new_cap = math.ceil(max(need + 512, 2 * cap, self.capacity) / BLOCK) * BLOCK
        B, H, _, D = ref.shape
        k = torch.empty(B, H, new_cap, D, dtype=ref.dtype, device=ref.device)
        v = torch.empty_like(k)
        if self._n:
            k[:, :, :self._n] = self._k[:, :, :self._n]
            v[:, :, :self._n] = self._v[:, :, :self._n]
        self._k, self._v = k, v

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor):
        """Appends [B,Hkv,t,D] and returns (keys, values): views of the whole current length."""
        t = key_states.shape[-2]
        self._ensure(self._n + t, key_states)
        if t == 1 and key_states.is_cuda:
            K.ext().append(self._k, self._v, key_states[:, :, 0].contiguous(), value_states[:, :, 0].contiguous(),
                           self._n + 1)
        else:
            self._k[:, :, self._n:self._n + t] = key_states
            self._v[:, :, self._n:self._n + t] = value_states
        self._n += t
        return self.views()

    def views(self):
        return self._k[:, :, :self._n], self._v[:, :, :self._n]

    def full(self):
        """The whole buffers (for launches that read the length from device memory)."""
        return self._k, self._v

    def get_seq_length(self) -> int:
        return self._n

    def room(self) -> int:
        """Tokens that fit before the next re-allocation (a captured step is valid that long)."""
        return 0 if self._k is None else self._k.shape[-2] - self._n

    def crop(self, tokens_to_remove: int) -> None:
        """Negative: drop that many tokens from the end; positive: keep that many (legacy form)."""
        if tokens_to_remove > 0:
            tokens_to_remove = max(0, self._n - tokens_to_remove)
        self._n -= abs(tokens_to_remove)


class PagedKV:
    """A page pool shared by B sequences of equal length (the kernels take one length per launch).

    pages are handed out from a free list on the host; `order` ("ascending", "shuffled") only
    matters for tests, which use a shuffled pool to show that no layout is assumed."""

    def __init__(self, num_pages: int, B: int, Hkv: int, D: int, max_tokens: int, device, dtype=torch.bfloat16,
                 order: str = "ascending", seed: int = 0):
        self.k = torch.empty(num_pages, Hkv, BLOCK, D, dtype=dtype, device=device)
        self.v = torch.empty_like(self.k)
        self.max_pages = math.ceil(max_tokens / BLOCK)
        self.table_host = torch.full((B, self.max_pages), -1, dtype=torch.int32)
        self.table = self.table_host.to(device)
        free = list(range(num_pages))
        if order == "shuffled":
            perm = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed)).tolist()
            free = perm
        self._free = free[::-1]          # pop() hands out from the front of the order
        self.B, self.n = B, 0
        self._blocks = 0                 # blocks per sequence that have a page

    def _ensure(self, T: int) -> None:
        """Pages for every block below ceil(T/64), for all sequences; the table goes to the device
        only when a block boundary is crossed."""
        have = self._blocks
        need = math.ceil(T / BLOCK)
        if need <= have:
            return
        if need > self.max_pages:
            raise RuntimeError(f"PagedKV: {T} tokens exceed max_tokens")
        for j in range(have, need):
            for b in range(self.B):
                if not self._free:
                    raise RuntimeError("PagedKV: the pool is exhausted")
                self.table_host[b, j] = self._free.pop()
        self._blocks = need
        self.table.copy_(self.table_host, non_blocking=True)

    def write(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """Prefill: [B,Hkv,T,D] into pages (sequence length becomes T)."""
        B, H, T, D = k.shape
        self._ensure(T)
        self.n = T
        nb = math.ceil(T / BLOCK)
        pad = nb * BLOCK - T
        if pad:
            k = torch.nn.functional.pad(k, (0, 0, 0, pad))
            v = torch.nn.functional.pad(v, (0, 0, 0, pad))
        pages = self.table[:, :nb].long().reshape(-1)                                     # [B*nb]
        self.k[pages] = k.reshape(B, H, nb, BLOCK, D).permute(0, 2, 1, 3, 4).reshape(B * nb, H, BLOCK, D)
        self.v[pages] = v.reshape(B, H, nb, BLOCK, D).permute(0, 2, 1, 3, 4).reshape(B * nb, H, BLOCK, D)

    def append(self, k_new: torch.Tensor, v_new: torch.Tensor, t_dev: torch.Tensor | None = None) -> None:
        """One token per sequence, [B,Hkv,D] each.  With t_dev the row index comes from the device
        (t_dev already holds the length after the append)."""
        self._ensure(self.n + 1)
        self.n += 1
        K.ext().append(self.k, self.v, k_new.contiguous(), v_new.contiguous(),
                       self.n if t_dev is None else self.max_pages * BLOCK, t_dev, self.table)

    def reserve(self, T: int) -> None:
        """Hand out pages up to length T now (a captured step must not run out of pages)."""
        self._ensure(T)

    # hooks of kvskip_b200.graph.StepGraph: an append inside a captured step is replayed without
    # this object seeing it
    def graph_scalars(self) -> tuple:
        return ()

    def note_replayed(self) -> None:
        if math.ceil((self.n + 1) / BLOCK) > self._blocks:
            raise RuntimeError("PagedKV: a replayed append ran past the reserved pages (call reserve() first)")
        self.n += 1

    def gather(self):
        """Contiguous copies [B,Hkv,n,D] of the cache (tests, debugging)."""
        nb = math.ceil(self.n / BLOCK)
        pages = self.table[:, :nb].long()
        k = self.k[pages].permute(0, 2, 1, 3, 4).reshape(self.B, self.k.shape[1], nb * BLOCK, -1)[:, :, :self.n]
        v = self.v[pages].permute(0, 2, 1, 3, 4).reshape(self.B, self.v.shape[1], nb * BLOCK, -1)[:, :, :self.n]
        return k.contiguous(), v.contiguous()

    def get_seq_length(self) -> int:
        return self.n
