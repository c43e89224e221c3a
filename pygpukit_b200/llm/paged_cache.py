"""Paged key/value cache for many sequences (net-new: the reference's Python layers keep one fixed cache per
sequence; its paged-attention kernels, native/ops/nn/attention/paged_attention.cuh:46-283, are not wired to them).

`PagePool` is the host-side bookkeeping, pure Python so that it is tested without a GPU: a pool of pages of
`page_size` positions, a free list, and per sequence a slot (row of the device page table), its page list and its
length.  `PagedKVCache` adds the device side: per layer one K and one V array of `[pages, kv_heads, page_size, dim]`
(bfloat16 or float32) and the int32 page table `[slots, max_pages]` that the kernels read.  Sequences are named by
any hashable id; `release(id)` gives the slot and the pages back, and both are handed out again (lowest first).

Per-sequence STATE: a layer may keep, beside or instead of pages, float32 arrays with one row per slot (the state of a
recurrent mixer, the last inputs of a short convolution): `state[i][j]` is `[slots, n]`.  A state row needs no clearing
when its slot is handed out again -- the kernels that read it take a sequence whose first position is 0 as starting from
zero -- and cannot be truncated.

Growth: when the free list runs dry the pool doubles (device arrays are reallocated and the old pages copied, page
numbers stay valid); a page table row grows the same way.  Sizing the pool for the expected number of live tokens up
front (`tokens_hint`) avoids both.
"""
from __future__ import annotations

import heapq

import numpy as np

from .._lib import api
from ..core.array import GPUArray
from ..core.dtypes import bfloat16, float32, int32
from ..core.factory import zeros
from ..core.stream import current_stream_handle as _st


class PagePool:
    def __init__(self, page_size: int, pages: int, slots: int, max_pages_per_seq: int):
        if page_size < 1 or pages < 1 or slots < 1 or max_pages_per_seq < 1:
            raise ValueError("PagePool: sizes must be positive")
        self.page_size, self.pages, self.slots, self.max_pages = page_size, pages, slots, max_pages_per_seq
        self._free_pages = list(range(pages))
        self._free_slots = list(range(slots))
        heapq.heapify(self._free_pages)
        heapq.heapify(self._free_slots)
        self._seq: dict = {}            # id -> [slot, [pages], length, steps that extended it]
        self.table = np.zeros((slots, max_pages_per_seq), np.int32)
        self.dirty = True               # the device copy of `table` is stale

    # ---- queries
    def __contains__(self, seq_id) -> bool:
        return seq_id in self._seq

    def length(self, seq_id) -> int:
        return self._seq[seq_id][2]

    def slot(self, seq_id) -> int:
        return self._seq[seq_id][0]

    def steps(self, seq_id) -> int:
        """How many times the sequence has been extended (double-buffered per-sequence state flips on it)."""
        return self._seq[seq_id][3]

    def page_list(self, seq_id) -> list[int]:
        return list(self._seq[seq_id][1])

    @property
    def free_pages(self) -> int:
        return len(self._free_pages)

    @property
    def live_sequences(self) -> int:
        return len(self._seq)

    # ---- growth hooks (PagedKVCache reallocates the device arrays)
    def _grow_pages(self, need: int) -> None:
        new = max(self.pages * 2, self.pages + need)
        for p in range(self.pages, new):
            heapq.heappush(self._free_pages, p)
        self.pages = new

    def _grow_slots(self) -> None:
        new = self.slots * 2
        for s in range(self.slots, new):
            heapq.heappush(self._free_slots, s)
        self.table = np.concatenate([self.table, np.zeros((new - self.slots, self.max_pages), np.int32)])
        self.slots = new
        self.dirty = True

    def _grow_table(self, need: int) -> None:
        new = max(self.max_pages * 2, need)
        self.table = np.concatenate([self.table, np.zeros((self.slots, new - self.max_pages), np.int32)], axis=1)
        self.max_pages = new
        self.dirty = True

    # ---- allocation
    def extend(self, seq_id, n_tokens: int) -> tuple[int, int]:
        """Make room for `n_tokens` more positions of `seq_id` (a new id starts a sequence at position 0).
        Returns (slot, first new position)."""
        if n_tokens < 1:
            raise ValueError("extend: at least one token")
        ent = self._seq.get(seq_id)
        if ent is None:
            if not self._free_slots:
                self._grow_slots()
            ent = self._seq[seq_id] = [heapq.heappop(self._free_slots), [], 0, 0]
        slot, pages, length, _ = ent
        need = -(-(length + n_tokens) // self.page_size) - len(pages)
        if need > 0:
            if len(pages) + need > self.max_pages:
                self._grow_table(len(pages) + need)
            if need > len(self._free_pages):
                self._grow_pages(need - len(self._free_pages))
            for _ in range(need):
                p = heapq.heappop(self._free_pages)
                self.table[slot, len(pages)] = p
                pages.append(p)
            self.dirty = True
        ent[2] = length + n_tokens
        ent[3] += 1
        return slot, length

    def truncate(self, seq_id, length: int) -> None:
        """Forget the positions from `length` on (rejected speculative tokens); whole pages past it are freed."""
        ent = self._seq[seq_id]
        if not 0 <= length <= ent[2]:
            raise ValueError(f"truncate: length {length} outside 0..{ent[2]}")
        keep = -(-length // self.page_size)
        for p in ent[1][keep:]:
            heapq.heappush(self._free_pages, p)
        del ent[1][keep:]
        ent[2] = length

    def release(self, seq_id) -> None:
        slot, pages, _, _ = self._seq.pop(seq_id)
        for p in pages:
            heapq.heappush(self._free_pages, p)
        heapq.heappush(self._free_slots, slot)


class PagedKVCache:
    """Device arrays of every layer + the page pool.  `layer_shapes` = [(kv_heads, dim, vdim), ...], one entry per cache
    (a layer that runs several times in a loop has one per run); vdim 0: the layer keeps one array whose rows serve as
    keys and, by a prefix, as values (latent attention) -- `v[i]` is then None; kv_heads 0: the layer has no pages at all.
    `state_shapes` = per cache the float32 elements per slot of each of its state arrays."""

    def __init__(self, layer_shapes: list[tuple[int, int, int]], dtype: str = "bfloat16", page_size: int = 64,
                 tokens_hint: int = 4096, slots: int = 8, state_shapes: "list[tuple] | None" = None):
        if dtype not in ("bfloat16", "float32"):
            raise ValueError("PagedKVCache: dtype is 'bfloat16' or 'float32'")
        self.dtype = bfloat16 if dtype == "bfloat16" else float32
        self.dtype_code = 2 if dtype == "bfloat16" else 0
        self.layer_shapes = list(layer_shapes)
        pages = -(-max(1, tokens_hint) // page_size) + slots          # every live sequence may hold one partial page
        self.pool = PagePool(page_size, pages, slots, max(4, -(-max(1, tokens_hint) // page_size) + 1))
        self.k: list[GPUArray | None] = []
        self.v: list[GPUArray | None] = []
        self._alloc(pages, copy_from=None)
        self.state_shapes = [tuple(int(n) for n in sh) for sh in (state_shapes or [()] * len(self.layer_shapes))]
        if len(self.state_shapes) != len(self.layer_shapes):
            raise ValueError("PagedKVCache: one tuple of state sizes per cache")
        self.state: list[list[GPUArray]] = []
        self._alloc_state(self.pool.slots, copy_from=None)
        self.table_dev = zeros((self.pool.slots * self.pool.max_pages,), int32)

    @property
    def page_size(self) -> int:
        return self.pool.page_size

    def _alloc(self, pages: int, copy_from) -> None:
        ps = self.pool.page_size
        k_new, v_new = [], []
        for i, (g, d, dv) in enumerate(self.layer_shapes):
            k = zeros((pages, g, ps, d), self.dtype) if g > 0 else None
            v = zeros((pages, g, ps, dv), self.dtype) if dv > 0 and g > 0 else None
            if copy_from is not None:
                if k is not None:
                    api.memcpy_d2d(k.device_ptr, self.k[i].device_ptr, self.k[i].nbytes, _st())
                if v is not None:
                    api.memcpy_d2d(v.device_ptr, self.v[i].device_ptr, self.v[i].nbytes, _st())
            k_new.append(k)
            v_new.append(v)
        if copy_from is not None:
            api.device_sync()
        self.k, self.v = k_new, v_new
        self._pages_dev = pages

    def _alloc_state(self, slots: int, copy_from) -> None:
        new = []
        for i, sizes in enumerate(self.state_shapes):
            arrs = []
            for j, n in enumerate(sizes):
                a = zeros((slots, n), float32)
                if copy_from is not None:
                    api.memcpy_d2d(a.device_ptr, self.state[i][j].device_ptr, self.state[i][j].nbytes, _st())
                arrs.append(a)
            new.append(arrs)
        if copy_from is not None:
            api.device_sync()
        self.state = new
        self._slots_dev = slots

    @property
    def has_state(self) -> bool:
        return any(self.state_shapes)

    def extend(self, seq_id, n_tokens: int) -> tuple[int, int]:
        out = self.pool.extend(seq_id, n_tokens)
        if self.pool.pages > self._pages_dev:
            self._alloc(self.pool.pages, copy_from=True)
        if self.pool.slots > self._slots_dev:
            self._alloc_state(self.pool.slots, copy_from=True)
        return out

    def release(self, seq_id) -> None:
        self.pool.release(seq_id)

    def truncate(self, seq_id, length: int) -> None:
        if self.has_state and length != self.pool.length(seq_id):
            raise ValueError("PagedKVCache: a sequence with recurrent state cannot be cut back")
        self.pool.truncate(seq_id, length)

    def sync_table(self) -> None:
        """Upload the page table when it changed since the last upload."""
        if not self.pool.dirty:
            return
        t = self.pool.table
        if self.table_dev.size != t.size:
            self.table_dev = GPUArray((t.size,), int32)
        self.table_dev.copy_from_numpy(t.reshape(-1))
        self.pool.dirty = False

    @property
    def nbytes(self) -> int:
        return (sum(a.nbytes for a in self.k if a is not None) + sum(a.nbytes for a in self.v if a is not None)
                + sum(a.nbytes for arrs in self.state for a in arrs))


__all__ = ["PagePool", "PagedKVCache"]
