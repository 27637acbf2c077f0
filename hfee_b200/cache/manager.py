"""The cache manager: pages of keys and values with a block table per request,
and fixed-size state slots per request.

The reference gives every conversation slot one contiguous key and value array
per layer for the whole context (hostfog/hfee internal/llm/forward.go:10-26) and
keeps no other per-sequence state.  Here caches with equal needs form a *group*;
a paged group owns a pool of pages (one page id addresses the page in every cache
of the group) and one block table ``[max_requests, max_pages]`` whose row is the
request's slot; a state group owns ``[max_requests, ...]`` rows.  Pages go back to
the pool when a request is closed or, in a windowed group, once the window has
passed them.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional

import numpy as np
import torch

from .needs import FixedState, PagedKV
from .pages import OutOfPages, PagePool

_TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


@dataclass
class CacheView:
    """What a mixer gets for one cache id: either pages (``k``, ``v`` of shape
    [num_pages, kv_heads, page_size, head_dim], ``block_table`` int32
    [max_requests, max_pages] on the device, ``page_size``) or ``state``
    ([max_requests, *shape], row = request slot)."""
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None
    page_size: int = 0
    state: Optional[torch.Tensor] = None


class _PagedGroup:
    def __init__(self, need: PagedKV, cache_ids: List[int], num_pages: int, page_size: int, max_requests: int,
                 max_pages: int, dtype: torch.dtype, device):
        self.need, self.cache_ids = need, cache_ids
        self.pool = PagePool(num_pages)
        self.page_size = page_size
        self.table = np.full((max_requests, max_pages), -1, dtype=np.int32)
        self.first_live = [0] * max_requests       # logical pages [first_live, held_to) are held
        self.held_to = [0] * max_requests
        self.dirty = True
        shape = (len(cache_ids), num_pages, need.kv_heads, page_size, need.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.table_dev = torch.full((max_requests, max_pages), -1, dtype=torch.int32, device=device)
        # pinned staging copies of the table, used in turn, so that an upload never makes the host
        # wait for the GPU (a copy from pageable memory would)
        pin = torch.device(device).type == "cuda"
        self.staging = [torch.empty((max_requests, max_pages), dtype=torch.int32, pin_memory=pin) for _ in range(4)]
        self.staging_events = [None] * 4
        self.staging_turn = 0

    def first_needed_page(self, length: int) -> int:
        """First logical page a token at position >= ``length`` can still read."""
        if self.need.window is None:
            return 0
        lowest_key = max(0, length - int(self.need.window) + 1)
        return lowest_key // self.page_size


class _StateGroup:
    def __init__(self, need: FixedState, cache_ids: List[int], max_requests: int, device):
        self.need, self.cache_ids = need, cache_ids
        self.state = torch.zeros((len(cache_ids), max_requests) + tuple(need.shape),
                                 dtype=_TORCH[need.dtype], device=device)


class CacheManager:
    def __init__(self, needs: Mapping[int, Any], page_size: int, num_pages: int, max_requests: int,
                 max_context: int, dtype: torch.dtype, device="cpu"):
        self.page_size, self.num_pages = page_size, num_pages
        self.max_requests, self.max_context = max_requests, max_context
        self.max_pages = -(-max_context // page_size)
        self.device = torch.device(device)
        self.paged: List[_PagedGroup] = []
        self.states: List[_StateGroup] = []
        by_need: Dict[Any, List[int]] = {}
        for cache_id, need in sorted(needs.items()):
            if need is None:
                continue
            if not isinstance(need, (PagedKV, FixedState)):
                raise TypeError(f"cache {cache_id}: a mixer's cache_need() must be PagedKV, FixedState or None, "
                                f"got {type(need).__name__}")
            by_need.setdefault(need, []).append(cache_id)
        for need, ids in by_need.items():
            if isinstance(need, PagedKV):
                self.paged.append(_PagedGroup(need, ids, num_pages, page_size, max_requests, self.max_pages,
                                              dtype, self.device))
            else:
                self.states.append(_StateGroup(need, ids, max_requests, self.device))
        self._views: Dict[int, CacheView] = {}
        for g in self.paged:
            for j, cid in enumerate(g.cache_ids):
                self._views[cid] = CacheView(k=g.k[j], v=g.v[j], block_table=g.table_dev, page_size=page_size)
        for s in self.states:
            for j, cid in enumerate(s.cache_ids):
                self._views[cid] = CacheView(state=s.state[j])
        self.length = [0] * max_requests
        self.open_slots = [False] * max_requests

    # ------------------------------------------------------------------ requests
    def open(self) -> int:
        """Take a free request slot (block-table row and state row); its state is zeroed."""
        for slot, used in enumerate(self.open_slots):
            if not used:
                self.open_slots[slot] = True
                self.length[slot] = 0
                for g in self.paged:
                    g.first_live[slot] = g.held_to[slot] = 0
                for s in self.states:
                    s.state[:, slot].zero_()
                return slot
        raise RuntimeError(f"all {self.max_requests} request slots are in use")

    def free_slots(self) -> int:
        return self.open_slots.count(False)

    def pages_needed(self, slot: int, new_length: int) -> int:
        """Most pages any group must still take to hold ``new_length`` tokens of ``slot``."""
        return max((self._missing(g, slot, new_length) for g in self.paged), default=0)

    def _missing(self, g: _PagedGroup, slot: int, new_length: int) -> int:
        return max(0, -(-new_length // self.page_size) - g.held_to[slot])

    def can_reserve(self, slot: int, new_length: int) -> bool:
        if new_length > self.max_context:
            return False
        return all(self._missing(g, slot, new_length) <= g.pool.free_pages for g in self.paged)

    def reserve(self, slot: int, new_length: int) -> None:
        """Give ``slot`` pages for positions up to ``new_length`` in every paged group;
        takes nothing and raises :class:`OutOfPages` if any group cannot."""
        self._check_open(slot)
        if new_length > self.max_context:
            raise ValueError(f"{new_length} tokens exceed the context limit of {self.max_context}")
        if not self.can_reserve(slot, new_length):
            raise OutOfPages(f"slot {slot}: no pages for {new_length} tokens")
        for g in self.paged:
            want_to = -(-new_length // self.page_size)
            have_to = g.held_to[slot]
            if want_to > have_to:
                g.table[slot, have_to:want_to] = g.pool.take(want_to - have_to)
                g.held_to[slot] = want_to
                g.dirty = True

    def commit(self, slot: int, new_length: int) -> None:
        """Record that ``slot`` now holds ``new_length`` tokens; windowed groups give back
        the pages no later token can read."""
        self._check_open(slot)
        if new_length < self.length[slot]:
            raise ValueError("commit cannot shorten a request")
        self.length[slot] = new_length
        for g in self.paged:
            first = min(g.first_needed_page(new_length), g.held_to[slot])
            if first > g.first_live[slot]:
                row = g.table[slot]
                gone = [int(p) for p in row[g.first_live[slot]:first] if p >= 0]
                g.pool.give_back(gone)
                row[g.first_live[slot]:first] = -1
                g.first_live[slot] = first
                g.dirty = True

    def close(self, slot: int) -> None:
        """The request is over (finished, aborted or preempted): everything it holds goes back."""
        self._check_open(slot)
        for g in self.paged:
            row = g.table[slot]
            g.pool.give_back(int(p) for p in row if p >= 0)
            row[:] = -1
            g.first_live[slot] = g.held_to[slot] = 0
            g.dirty = True
        self.length[slot] = 0
        self.open_slots[slot] = False

    def _check_open(self, slot: int) -> None:
        if not (0 <= slot < self.max_requests) or not self.open_slots[slot]:
            raise ValueError(f"slot {slot} is not open")

    # ------------------------------------------------------------------ device side
    def sync(self) -> None:
        """Copy block tables that changed to the device (before the step that uses them)."""
        for g in self.paged:
            if g.dirty:
                i = g.staging_turn
                g.staging_turn = (i + 1) % len(g.staging)
                if g.staging_events[i] is not None:
                    g.staging_events[i].synchronize()          # that staging copy's last upload is done
                g.staging[i].copy_(torch.from_numpy(g.table))
                g.table_dev.copy_(g.staging[i], non_blocking=True)
                if g.table_dev.is_cuda:
                    ev = torch.cuda.Event()
                    ev.record()
                    g.staging_events[i] = ev
                g.dirty = False

    def view(self, cache_id: int) -> Optional[CacheView]:
        return self._views.get(cache_id)

    def views(self) -> Dict[int, CacheView]:
        return self._views

    # ------------------------------------------------------------------ accounting
    def free_pages(self) -> int:
        return min((g.pool.free_pages for g in self.paged), default=self.num_pages)

    def cache_bytes(self) -> int:
        n = sum(g.k.numel() * g.k.element_size() * 2 for g in self.paged)
        return n + sum(s.state.numel() * s.state.element_size() for s in self.states)

    def check_invariants(self) -> None:
        """Every page is free or in exactly one block-table cell; open rows cover exactly
        the pages their length (and window) needs; closed rows hold nothing."""
        for g in self.paged:
            seen = {}
            for slot in range(self.max_requests):
                row = g.table[slot]
                for logical, p in enumerate(row):
                    if p < 0:
                        continue
                    p = int(p)
                    if p in seen:
                        raise AssertionError(f"page {p} is held by {seen[p]} and by {(slot, logical)}")
                    if not g.pool.is_held(p):
                        raise AssertionError(f"page {p} is in a block table but marked free")
                    if not self.open_slots[slot]:
                        raise AssertionError(f"closed slot {slot} holds page {p}")
                    seen[p] = (slot, logical)
                if self.open_slots[slot]:
                    need_to = -(-self.length[slot] // self.page_size)
                    for logical in range(g.first_needed_page(self.length[slot]), need_to):
                        if row[logical] < 0:
                            raise AssertionError(f"slot {slot} has no page for logical page {logical}")
            if len(seen) + g.pool.free_pages != g.pool.num_pages:
                raise AssertionError(f"{g.pool.num_pages - len(seen) - g.pool.free_pages} pages are lost")
