"""Device side of the cache: the page pools of keys and values and the per-request state arrays.

For every call of the model's order that owns a cache entry there is a pair of tensors ``k, v`` shaped
``[pages, kv_heads, page_size, head_dim]`` (values may have a head size of their own) — a page's rows of one
head are contiguous —, or a state tensor ``[slots, *shape]``, or several of these for a mixer that keeps several
things (``CompositeCacheSpec``: its view holds one view per part).  Calls whose attention has the same window
form a group and share page ids (the same page index addresses the same slice in each of them, as in the
reference's pool: src/model.cpp:642-645).  All state arrays of a dtype are slices of one buffer ``[slots,
words]``, so that a request's whole state is one stretch of memory and one launch zeroes it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..parts.base import KVCacheSpec, StateCacheSpec, CompositeCacheSpec


@dataclass
class CacheView:
    kind: str                      # "kv" | "state" | "multi" | "none"
    group: int = -1
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None
    write: bool = True
    page_size: int = 0
    parts: Optional[list] = None   # "multi": the views of the composite's parts

    def read_only(self) -> "CacheView":
        parts = [p.read_only() for p in self.parts] if self.parts is not None else None
        return CacheView(self.kind, self.group, self.k, self.v, self.state, False, self.page_size, parts)


def _group_key(spec: KVCacheSpec):
    """What layers must share to share page ids: the window, and with a window the number of first positions that
    stay readable behind it."""
    return (spec.window, spec.keep_first) if spec.window > 0 and spec.keep_first > 0 else spec.window


def _leaves(spec):
    """The page and state specs inside a cache spec, composites opened, in order."""
    if isinstance(spec, CompositeCacheSpec):
        for p in spec.parts:
            yield from _leaves(p)
    elif isinstance(spec, (KVCacheSpec, StateCacheSpec)):
        yield spec


class DeviceCache:
    def __init__(self, cache_specs: list, page_size: int, max_slots: int, device, dtype):
        self.page_size, self.device, self.dtype, self.max_slots = page_size, device, dtype, max_slots
        self.specs = cache_specs
        self.windows: list = []                    # one per group: the window, or (window, kept first positions)
        for s in cache_specs:
            for leaf in _leaves(s):
                if isinstance(leaf, KVCacheSpec) and _group_key(leaf) not in self.windows:
                    self.windows.append(_group_key(leaf))
        self.views: list = []
        self.num_pages: list = []
        self.state_buffers: dict = {}              # dtype -> [slots, words of that dtype]

    def _group(self, spec: KVCacheSpec) -> int:
        return self.windows.index(_group_key(spec))

    def bytes_per_page(self) -> list:
        """Per group: bytes of one page over all its entries."""
        item = torch.empty((), dtype=self.dtype).element_size()
        out = [0] * len(self.windows)
        for s in self.specs:
            for leaf in _leaves(s):
                if isinstance(leaf, KVCacheSpec):
                    per_token = leaf.head_dim + (leaf.value_dim if leaf.values else 0)
                    out[self._group(leaf)] += leaf.num_kv_heads * self.page_size * per_token * item
        return out

    def state_bytes_per_slot(self) -> int:
        return sum(b.shape[1] * b.element_size() for b in self.state_buffers.values())

    def allocate(self, num_pages, max_blocks: int = 0) -> None:
        """``max_blocks`` > 0: also the block tables, per group one of every state slot's request
        (``tables[g]`` [slots, max_blocks], kept up to date step by step with what changed) and one of the running
        step's entries (``step_tables[g]`` [slots, max_blocks], the one the kernels read): see ``sync_tables``."""
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(self.windows)
        self.num_pages = list(num_pages)
        self.views = []
        self.max_blocks = max_blocks
        self.tables = self.step_tables = None
        if max_blocks > 0:
            shape = (max(1, self.max_slots), max_blocks)
            self.tables = [torch.full(shape, -1, dtype=torch.int32, device=self.device) for _ in self.windows]
            self.step_tables = [torch.full(shape, -1, dtype=torch.int32, device=self.device) for _ in self.windows]
        # the states, in the order of the specs: every array starts on a 16-byte boundary of its dtype's buffer
        words: dict = {}
        places: list = []
        for s in self.specs:
            for leaf in _leaves(s):
                if isinstance(leaf, StateCacheSpec):
                    item = torch.empty((), dtype=leaf.dtype).element_size()
                    n = 1
                    for d in leaf.shape:
                        n *= int(d)
                    at = words.get(leaf.dtype, 0)
                    places.append((at, n))
                    unit = max(1, 16 // item)
                    words[leaf.dtype] = at + (n + unit - 1) // unit * unit
        self.state_buffers = {dt: torch.zeros((self.max_slots, max(n, 1)), dtype=dt, device=self.device)
                              for dt, n in words.items()}
        places_it = iter(places)
        for s in self.specs:
            if isinstance(s, tuple) and s[0] == "shared":
                self.views.append(None)
            else:
                self.views.append(self._view(s, places_it))
        for i, s in enumerate(self.specs):
            if isinstance(s, tuple) and s[0] == "shared":
                self.views[i] = self.views[s[1]].read_only()

    def _view(self, s, places) -> CacheView:
        if isinstance(s, KVCacheSpec):
            g = self._group(s)
            pages = max(1, self.num_pages[g])
            k = torch.zeros((pages, s.num_kv_heads, self.page_size, s.head_dim), dtype=self.dtype, device=self.device)
            v = None            # (a layer whose values are read where its keys are keeps one array)
            if s.values:
                v = torch.zeros((pages, s.num_kv_heads, self.page_size, s.value_dim), dtype=self.dtype, device=self.device)
            return CacheView("kv", g, k, v, None, True, self.page_size)
        if isinstance(s, StateCacheSpec):
            at, n = next(places)
            st = self.state_buffers[s.dtype][:, at:at + n].view(self.max_slots, *s.shape)
            return CacheView("state", -1, None, None, st, True, self.page_size)
        if isinstance(s, CompositeCacheSpec):
            return CacheView("multi", -1, None, None, None, True, self.page_size, [self._view(p, places) for p in s.parts])
        return CacheView("none")

    def view(self, call_index: int) -> CacheView:
        return self.views[call_index]

    @property
    def has_state(self) -> bool:
        return any(isinstance(leaf, StateCacheSpec) for s in self.specs for leaf in _leaves(s))

    def sync_tables(self, batch) -> None:
        """Before a step runs: the block tables of its entries, in entry order, are put together on the device
        (``batch.block_tables``) from the tables kept per state slot, after the rows that travelled with the step
        (the tables that changed since they last did) have been taken in.  The reference writes every table of a
        step again on the host (src/model_runner.cpp:29-41)."""
        from ..csrc import ops
        if batch.table_updates is None:
            return
        for g, (src, lens, rows) in enumerate(batch.table_updates):
            ops.sync_block_tables(src, lens, rows, batch.entry_slot, self.tables[g], self.step_tables[g], batch.S)

    def reset_fresh(self, batch) -> None:
        """Before a step runs: the state of every entry that starts its request (first position 0) is zeroed, on
        the device, from the step's own index arrays.  A request therefore begins from zero whoever held its slot
        before, also after a preemption (it runs again from its first token), and a captured step does the same
        when it is replayed."""
        from ..csrc import ops
        for buf in self.state_buffers.values():
            ops.reset_fresh_state(buf, batch.entry_slot, batch.entry_pos0)
