"""The cache manager: paged keys and values with a block table per request, in groups of caches
with the same needs, and slots of fixed-size per-request state beside them.

* A *cache* belongs to one run of a layer (an entry of the model's run order).  Caches whose
  mixers ask for the same thing (`KVCacheRequest`: kv heads, head size, window) form a *group*.
  A group has a page pool and storage of its own; one page holds `page_tokens` positions of
  every cache of the group: [cache][keys | values][kv head][token in page][head_dim].
  (cuongvng/bare-cuda-4gib has one group: a page holds K for every layer then V for every
  layer, 64 tokens: engine/include/llm/kv_cache.h:14-32.)
* A request owns a *slot*; per group the slot has a block table: the page of its n-th block of
  positions, or -1.  `reserve(slot, n)` takes the pages the next n positions need and, in a
  group with a window, first gives back the pages that every later query has moved past;
  `commit(slot, n)` moves the length once a step has written all layers; `release_slot` gives
  everything back (engine/src/kv_cache.cpp:52-71,131-149).
* State slots: one tensor [slots + 1, *shape] per demand that asks for state, zeroed when a
  request takes the slot.  The last row (`idle_slot`) belongs to no request: the idle rows that
  pad a decode step to a fixed batch size point there, so a mixer that updates its state on the
  device never touches a live request's state for them.  Llama asks for none; the interface is
  whole regardless.
* A run of a layer may state several demands (a block with two mixers, say): `demands[run]` is one
  `CacheDemand` or a list of them, and caches and states are addressed by (run, index in that list).

All bookkeeping is host-side and runs without a GPU (`device="cpu"` or storage disabled).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..errors import CacheError, OutOfPages
from ..kernels.lib import CacheView
from ..parts.base import KVCacheRequest, StateRequest
from .page_pool import PagePool


@dataclass
class CacheDemand:
    """What one part of one entry of the run order wants: paged keys/values, state, or (with
    `cache_from`, the index of an earlier run) the cache and state of that run's part in the same
    place."""

    kv: Optional[KVCacheRequest] = None
    state: Optional[StateRequest] = None
    cache_from: Optional[int] = None


class CacheGroup:
    def __init__(self, request: KVCacheRequest, members: List[int], page_tokens: int, num_pages: int,
                 max_blocks: int, dtype: torch.dtype, device, allocate: bool):
        self.request, self.members = request, members      # members: (run, index in the run's demands)
        self.page_tokens, self.num_pages, self.max_blocks = page_tokens, num_pages, max_blocks
        self.pool = PagePool(num_pages)
        self.tables: Dict[int, List[int]] = {}      # slot -> page per block (-1 = none)
        self.dtype = dtype
        self.cache_elems = 2 * request.kv_heads * page_tokens * request.head_dim
        self.page_stride = len(members) * self.cache_elems
        self.storage = None
        if allocate:
            self.storage = torch.zeros((num_pages, self.page_stride), dtype=dtype, device=device)

    @property
    def bytes(self) -> int:
        return self.num_pages * self.page_stride * torch.empty((), dtype=self.dtype).element_size()

    def first_needed_block(self, length_before: int) -> int:
        """Blocks below this hold only positions that no query at >= length_before can see."""
        if self.request.window is None:
            return 0
        first_key = max(0, length_before - int(self.request.window) + 1)
        return first_key // self.page_tokens

    def blocks_to_take(self, slot: int, length: int, n: int) -> List[int]:
        table = self.tables.get(slot, [])
        last = (length + n - 1) // self.page_tokens
        if self.request.window is None:
            # every block below len(table) is held: only new blocks can be missing
            return list(range(len(table), last + 1)) if last >= len(table) else []
        first = self.first_needed_block(length)
        return [b for b in range(first, last + 1) if b >= len(table) or table[b] < 0]

    def blocks_to_drop(self, slot: int, length: int) -> List[int]:
        if self.request.window is None:
            return []
        table = self.tables.get(slot, [])
        return [b for b in range(min(self.first_needed_block(length), len(table))) if table[b] >= 0]


class CacheManager:
    def __init__(self, demands: Sequence[CacheDemand], *, page_tokens: int, max_seqs: int,
                 max_tokens: int, num_pages: Optional[int] = None, dtype=torch.float32, device="cpu",
                 allocate: bool = True, max_step_tokens: Optional[int] = None):
        """`max_tokens` bounds one request's length; `num_pages` sizes every group's pool (default:
        enough for `max_seqs` requests of `max_tokens`)."""
        if page_tokens <= 0 or max_seqs <= 0 or max_tokens <= 0:
            raise CacheError("page_tokens, max_seqs and max_tokens must be positive")
        self.page_tokens, self.max_seqs, self.max_tokens = page_tokens, max_seqs, max_tokens
        self.max_blocks = -(-max_tokens // page_tokens)
        self.device, self.dtype = torch.device(device), dtype
        # per run a list of demands (most blocks state one: their mixer's)
        self.demands: List[List[CacheDemand]] = [list(d) if isinstance(d, (list, tuple)) else [d] for d in demands]
        self.groups: List[CacheGroup] = []
        self.cache_group: Dict[Tuple[int, int], Tuple[int, int]] = {}    # (run, j) -> (group, index in group)
        by_request: Dict[KVCacheRequest, List[Tuple[int, int]]] = {}
        for i, run in enumerate(self.demands):
            for j, d in enumerate(run):
                if d.cache_from is not None:
                    src = d.cache_from
                    if not (0 <= src < i) or j >= len(self.demands[src]) or self.demands[src][j].cache_from is not None:
                        raise CacheError(f"run {i} reads the cache of run {src}, which must be an "
                                         "earlier run with a cache of its own")
                    continue
                if d.kv is not None:
                    by_request.setdefault(d.kv, []).append((i, j))
        for request, members in by_request.items():
            pages = num_pages if num_pages is not None else max_seqs * self.max_blocks
            g = CacheGroup(request, members, page_tokens, pages, self.max_blocks, dtype, self.device, allocate)
            for at, key in enumerate(members):
                self.cache_group[key] = (len(self.groups), at)
            self.groups.append(g)
        self.lengths: Dict[int, int] = {}
        self._free_slots = list(range(max_seqs - 1, -1, -1))
        self.idle_slot = max_seqs          # a state row that no request owns (see the module's text)
        self.states: Dict[Tuple[int, int], torch.Tensor] = {}
        for i, run in enumerate(self.demands):
            for j, d in enumerate(run):
                if d.state is not None and d.cache_from is None:
                    self.states[(i, j)] = torch.zeros((max_seqs + 1, *d.state.shape), dtype=d.state.dtype,
                                                      device=self.device if allocate else "cpu")
        for i, run in enumerate(self.demands):
            for j, d in enumerate(run):
                if d.cache_from is None:
                    continue
                if (d.cache_from, j) in self.cache_group:
                    self.cache_group[(i, j)] = self.cache_group[(d.cache_from, j)]
                if (d.cache_from, j) in self.states:
                    self.states[(i, j)] = self.states[(d.cache_from, j)]

    def group_of(self, run: int, j: int = 0) -> Optional[Tuple[int, int]]:
        """(group, index in the group) of the cache that part `j` of run `run` reads, or None."""
        return self.cache_group.get((run, j))

    def state_of(self, run: int, j: int = 0) -> Optional[torch.Tensor]:
        """[slots + 1, *shape] state of part `j` of run `run`, or None."""
        return self.states.get((run, j))

    # ------------------------------------------------------------------ slots
    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def acquire_slot(self) -> int:
        if not self._free_slots:
            raise CacheError(f"all {self.max_seqs} request slots are taken")
        slot = self._free_slots.pop()
        self.lengths[slot] = 0
        for g in self.groups:
            g.tables[slot] = []
        for (run, j), state in self.states.items():
            if self.demands[run][j].cache_from is None:
                state[slot].zero_()
        return slot

    def release_slot(self, slot: int) -> None:
        if slot not in self.lengths:
            raise CacheError(f"slot {slot} is not held (released twice?)")
        for g in self.groups:
            for page in g.tables.pop(slot, []):
                if page >= 0:
                    g.pool.release(page)
        del self.lengths[slot]
        self._free_slots.append(slot)

    def length(self, slot: int) -> int:
        if slot not in self.lengths:
            raise CacheError(f"slot {slot} is not held")
        return self.lengths[slot]

    # ------------------------------------------------------------------ pages
    def pages_needed(self, slot: int, n: int) -> List[int]:
        """Per group: pages to take minus pages that reserving would give back first."""
        length = self.length(slot)
        return [len(g.blocks_to_take(slot, length, n)) - len(g.blocks_to_drop(slot, length)) for g in self.groups]

    def pages_for_tokens(self, n_tokens: int, step_tokens: int = 1) -> List[int]:
        """Per group: pages a request holds at most while it grows to `n_tokens` positions in
        steps of at most `step_tokens`."""
        out = []
        for g in self.groups:
            blocks = -(-n_tokens // g.page_tokens)
            if g.request.window is not None:
                span = int(g.request.window) + step_tokens  # the window plus the positions being added
                blocks = min(blocks, -(-span // g.page_tokens) + 1)
            out.append(blocks)
        return out

    def can_reserve(self, wants: Sequence[Tuple[int, int]]) -> bool:
        need = [0] * len(self.groups)
        for slot, n in wants:
            for gi, k in enumerate(self.pages_needed(slot, n)):
                need[gi] += k
        return all(need[gi] <= g.pool.free_pages for gi, g in enumerate(self.groups))

    def reserve(self, slot: int, n: int) -> None:
        """Makes sure positions length .. length + n - 1 have pages in every group; all or nothing."""
        self.reserve_batch([(slot, n)])

    def reserve_batch(self, wants: Sequence[Tuple[int, int]]) -> None:
        """`reserve` for several (slot, tokens) at once: either every request gets its pages or none does."""
        for slot, n in wants:
            length = self.length(slot)
            if n <= 0:
                raise CacheError("reserve needs a positive token count")
            if length + n > self.max_tokens:
                raise CacheError(f"request of {length + n} tokens exceeds the cache's limit of "
                                 f"{self.max_tokens} per request")
        if not self.can_reserve(wants):
            raise OutOfPages(f"out of pages: the pools have {[g.pool.free_pages for g in self.groups]} page(s) "
                             f"free per group, the batch needs more")
        for slot, n in wants:
            self._take(slot, n)

    def _take(self, slot: int, n: int) -> None:
        length = self.lengths[slot]
        for g in self.groups:
            table = g.tables[slot]
            for b in g.blocks_to_drop(slot, length):
                g.pool.release(table[b])
                table[b] = -1
            for b in g.blocks_to_take(slot, length, n):
                while len(table) <= b:
                    table.append(-1)
                table[b] = g.pool.acquire()

    def commit(self, slot: int, n: int) -> None:
        self.lengths[slot] = self.length(slot) + n

    # ------------------------------------------------------------------ views for a step
    def block_table_rows(self, group: int, slots: Sequence[int], out: np.ndarray) -> None:
        """Fills out[i, :] with slot i's block table of `group` (-1 beyond what is held)."""
        g = self.groups[group]
        out[: len(slots)].fill(-1)
        for i, slot in enumerate(slots):
            table = g.tables[slot]
            out[i, : len(table)] = table

    def cache_view(self, run: int, block_table: torch.Tensor, j: int = 0) -> Optional[CacheView]:
        """The kernel-side description of the cache that part `j` of run `run` reads (its own or a
        borrowed one)."""
        if (run, j) not in self.cache_group:
            return None
        gi, j = self.cache_group[(run, j)]
        g = self.groups[gi]
        if g.storage is None:
            return None
        esize = g.storage.element_size()
        k_ptr = g.storage.data_ptr() + j * g.cache_elems * esize
        v_ptr = k_ptr + (g.cache_elems // 2) * esize
        return CacheView(k_ptr, v_ptr, block_table, g.page_stride, block_table.stride(0), g.page_tokens,
                         g.request.kv_heads, g.request.head_dim, g.dtype, g.storage.data_ptr(), g.storage.numel())

    # ------------------------------------------------------------------ accounting
    def pages_in_use(self) -> List[int]:
        return [g.pool.pages_in_use for g in self.groups]

    def check_consistency(self) -> None:
        """No page lost, held twice or freed while listed: used by the tests after every move."""
        for gi, g in enumerate(self.groups):
            seen = {}
            for slot, table in g.tables.items():
                for b, page in enumerate(table):
                    if page < 0:
                        continue
                    if page in seen:
                        raise CacheError(f"group {gi}: page {page} is held by slot {seen[page]} and slot {slot}")
                    if not g.pool.is_held(page):
                        raise CacheError(f"group {gi}: slot {slot} lists page {page}, which the pool has free")
                    seen[page] = slot
            if len(seen) != g.pool.pages_in_use:
                raise CacheError(f"group {gi}: {g.pool.pages_in_use} pages are held, {len(seen)} are listed "
                                 "in block tables (a page was lost)")
