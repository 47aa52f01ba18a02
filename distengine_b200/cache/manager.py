"""The cache manager: keys and values in pages with a block table for each request, pools by
group of layers, and slots for per-request state of fixed size.

* A *group* is the set of plan entries whose mixers need the same thing (kv heads, head size,
  window).  Each group has a pool of pages of its own ([layers of the group, pages, kv_heads, page,
  head_dim] for keys and for values), a free list, and a block table per request.  Groups that keep
  only a window of keys give a page back as soon as every position in it is behind the window of
  all tokens still to come.
* A *slot* is a small integer that a live request holds from admission to release.  Block-table
  rows on the device and every fixed-size state tensor ([layers, slots, *shape]) are indexed by it;
  a state row is zeroed at admission.  An architecture without such state still gets a slot.
* Pages are taken when a step is about to write positions (``reserve``, all requests of the step
  or none) and given back at ``release`` or when a window has passed them (``commit``).  The free
  list is last-in first-out, so pages are used again at once.
* A step may be launched before its caller knows that it counts (the engine keeps the GPU one
  decode step ahead of the host).  Such a step is committed *tentatively*: lengths advance, but no
  page that a window has passed is given back and the state rows of its requests are copied aside
  first.  ``confirm`` makes it final; ``rewind`` puts lengths and state rows back, and the pages
  that the redone positions read are all still there.

The reference's counterparts: ``BlockManager`` (src/distengine/block_manager.py:1-76: free list
popped from the end, grow-only tables, everything returned at ``free``) and ``KVStorage``
(src/distengine/paged_kv_cache.py:4-23: one pool for all layers).  It has no groups, no window, no
slots; errors raised here follow its classes (ValueError for a duplicate, KeyError for an unknown
id, RuntimeError when pages run out: block_manager.py:37-40,58-65,73-74).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..parts.base import PagedKVSpec, StateSpec
from ..parts.context import CacheBinding


class OutOfPages(RuntimeError):
    """Not enough free pages for what a step must write; nothing was taken."""


class OutOfSlots(RuntimeError):
    """Every slot is held by a live request."""


class PagePool:
    """Free list of one group.  ``take`` pops from the end, ``give`` appends: last in, first
    out."""

    def __init__(self, num_pages: int) -> None:
        if type(num_pages) is not int or num_pages <= 0:
            raise ValueError("num_pages must be a positive integer")
        self.num_pages = num_pages
        self._free = list(range(num_pages))
        self._held = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, count: int) -> list[int]:
        if count > len(self._free):
            raise OutOfPages(f"{count} pages wanted, {len(self._free)} free")
        pages = [self._free.pop() for _ in range(count)]
        for p in pages:
            self._held[p] = True
        return pages

    def give(self, pages: list[int]) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages or not self._held[p]:
                raise KeyError(f"page {p} is not held: it cannot be given back")
            self._held[p] = False
            self._free.append(p)

    def free_pages(self) -> list[int]:
        return list(self._free)


class SlotPool:
    def __init__(self, num_slots: int) -> None:
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))       # slot 0 first
        self._owner: dict[int, str] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, request_id: str) -> int:
        if not self._free:
            raise OutOfSlots(f"all {self.num_slots} slots are held")
        slot = self._free.pop()
        self._owner[slot] = request_id
        return slot

    def give(self, slot: int) -> None:
        if slot not in self._owner:
            raise KeyError(f"slot {slot} is not held")
        del self._owner[slot]
        self._free.append(slot)


@dataclass
class _PagedGroup:
    spec: PagedKVSpec
    entries: list[int]                        # plan entries that own a layer here, in order
    pool: PagePool
    k: torch.Tensor                           # [layers, pages, kv_heads, page, head_dim]
    v: torch.Tensor
    host_table: torch.Tensor                  # int32 [slots, max_pages], pinned when possible
    device_table: torch.Tensor
    tables: dict[str, list[int]] = field(default_factory=dict)   # logical page -> id or -1
    dirty: dict[int, list[int]] = field(default_factory=dict)    # slot -> [lo, hi) to upload


@dataclass
class _StateGroup:
    spec: StateSpec
    entries: list[int]
    state: torch.Tensor                       # [layers, slots, *shape]
    saved: "torch.Tensor | None" = None       # rows copied aside before a tentative step


@dataclass
class _Live:
    slot: int
    length: int = 0
    confirmed: "int | None" = None            # length before the tentative steps, if any


class CacheManager:
    def __init__(self, cache_specs: "list[PagedKVSpec | StateSpec | None]",
                 reads_cache_of: "list[int | None]", page_size: int, num_pages: int,
                 max_seqs: int, max_len: int, dtype: torch.dtype,
                 device: "torch.device | str", poison_freed_pages: bool = False) -> None:
        """``cache_specs[i]`` is what plan entry i keeps (None: nothing of its own);
        ``reads_cache_of[i]`` names the entry whose cache entry i reads instead.  ``num_pages``
        is the size of every paged group's pool."""
        if type(page_size) is not int or page_size <= 0:
            raise ValueError("page_size must be a positive integer")
        self.page_size, self.max_seqs, self.max_len = page_size, max_seqs, max_len
        self.max_pages_per_seq = (max_len + page_size - 1) // page_size
        self.dtype, self.device = dtype, torch.device(device)
        self.poison = poison_freed_pages
        self.slots = SlotPool(max_seqs)
        self.live: dict[str, _Live] = {}
        self.paged: list[_PagedGroup] = []
        self.states: list[_StateGroup] = []
        self._where: list[tuple[str, int, int] | None] = [None] * len(cache_specs)
        pin = self.device.type == "cuda"

        for index, spec in enumerate(cache_specs):
            if spec is None:
                continue
            if isinstance(spec, PagedKVSpec):
                group = next((g for g in self.paged if g.spec == spec), None)
                if group is None:
                    host = torch.full((max_seqs, self.max_pages_per_seq), -1, dtype=torch.int32)
                    if pin:
                        host = host.pin_memory()
                    group = _PagedGroup(spec, [], PagePool(num_pages), None, None, host,
                                        torch.full_like(host, -1, device=self.device))
                    self.paged.append(group)
                self._where[index] = ("paged", self.paged.index(group), len(group.entries))
                group.entries.append(index)
            elif isinstance(spec, StateSpec):
                group = next((g for g in self.states if g.spec == spec), None)
                if group is None:
                    group = _StateGroup(spec, [], None)
                    self.states.append(group)
                self._where[index] = ("state", self.states.index(group), len(group.entries))
                group.entries.append(index)
            else:
                raise TypeError(f"plan entry {index}: unknown cache spec {spec!r}")
        for group in self.paged:
            shape = (len(group.entries), num_pages, group.spec.kv_heads, page_size,
                     group.spec.head_dim)
            group.k = torch.zeros(shape, dtype=dtype, device=self.device)
            group.v = torch.zeros(shape, dtype=dtype, device=self.device)
            if self.poison:
                group.k.fill_(float("nan"))
                group.v.fill_(float("nan"))
        for sgroup in self.states:
            sgroup.state = torch.zeros((len(sgroup.entries), max_seqs, *sgroup.spec.shape),
                                       dtype=sgroup.spec.dtype, device=self.device)
        self._reads = list(reads_cache_of)
        # block-table rows travel through a pinned buffer of the manager's own: the host rows may
        # change again (a release, the next reserve) while an earlier upload is still queued
        self._stage: "torch.Tensor | None" = None
        self._staged = torch.cuda.Event() if pin else None
        self._stage_busy = False

    # ------------------------------------------------------------------ sizes
    @staticmethod
    def bytes_per_page(cache_specs, page_size: int, dtype: torch.dtype) -> int:
        """Bytes that one page index costs over all paged groups (keys and values)."""
        size = torch.empty((), dtype=dtype).element_size()
        groups: dict[PagedKVSpec, int] = {}
        for spec in cache_specs:
            if isinstance(spec, PagedKVSpec):
                groups[spec] = groups.get(spec, 0) + 1
        return sum(2 * layers * spec.kv_heads * page_size * spec.head_dim * size
                   for spec, layers in groups.items())

    @property
    def num_pages(self) -> int:
        return self.paged[0].pool.num_pages if self.paged else 0

    def num_free_pages(self) -> int:
        """Free pages of the fullest group."""
        return min((g.pool.num_free for g in self.paged), default=0)

    @property
    def capacity_tokens(self) -> int:
        return self.num_pages * self.page_size

    # ------------------------------------------------------------------ requests
    def admit(self, request_id: str) -> int:
        if not isinstance(request_id, str) or not request_id:
            raise ValueError("request_id must be a nonempty string")
        if request_id in self.live:
            raise ValueError(f"request '{request_id}' is already live")
        slot = self.slots.take(request_id)
        self.live[request_id] = _Live(slot)
        for group in self.paged:
            group.tables[request_id] = []
        for sgroup in self.states:
            sgroup.state[:, slot].zero_()
        return slot

    def has(self, request_id: str) -> bool:
        return request_id in self.live

    def slot(self, request_id: str) -> int:
        return self._get(request_id).slot

    def length(self, request_id: str) -> int:
        return self._get(request_id).length

    def _get(self, request_id: str) -> _Live:
        if request_id not in self.live:
            raise KeyError(f"request '{request_id}' is not live")
        return self.live[request_id]

    def _first_needed(self, group: _PagedGroup, length: int) -> int:
        """First logical page that a token at position >= length can still read."""
        if group.spec.window is None:
            return 0
        return max(0, length - group.spec.window + 1) // self.page_size

    def _missing(self, group: _PagedGroup, request_id: str, old_len: int,
                 new_len: int) -> list[int]:
        table = group.tables[request_id]
        first = self._first_needed(group, old_len)
        if new_len <= len(table) * self.page_size and (old_len // self.page_size
                                                       == (new_len - 1) // self.page_size):
            # the new positions lie in the page that holds the last position: it is held, and so
            # is everything before it unless a window's first page was given back
            if (table and table[(new_len - 1) // self.page_size] >= 0
                    and (group.spec.window is None or table[min(first, len(table) - 1)] >= 0)):
                return []
        last = (new_len + self.page_size - 1) // self.page_size
        return [p for p in range(first, last) if p >= len(table) or table[p] < 0]

    def pages_needed(self, request_id: str, new_len: int) -> int:
        """Pages (of the neediest group) that growing the request to new_len takes."""
        live = self._get(request_id)
        return max((len(self._missing(g, request_id, live.length, new_len)) for g in self.paged),
                   default=0)

    def reserve(self, wanted: "list[tuple[str, int]]") -> None:
        """Take the pages for every (request, new length) of a step, or none at all."""
        plans = []
        for group in self.paged:
            total = 0
            for request_id, new_len in wanted:
                live = self._get(request_id)
                if new_len > self.max_len:
                    raise ValueError(f"request '{request_id}' would reach {new_len} tokens, the "
                                     f"cache was made for {self.max_len}")
                missing = self._missing(group, request_id, live.length, new_len)
                plans.append((group, request_id, live.slot, missing))
                total += len(missing)
            if total > group.pool.num_free:
                raise OutOfPages(f"the step needs {total} pages, {group.pool.num_free} are free")
        for group, request_id, slot, missing in plans:
            if not missing:
                continue
            pages = group.pool.take(len(missing))
            table = group.tables[request_id]
            if len(table) <= missing[-1]:
                table.extend([-1] * (missing[-1] + 1 - len(table)))
            for logical, page in zip(missing, pages):
                table[logical] = page
            # one assignment for the row of the table that goes to the device (a prompt portion
            # takes a hundred pages and more)
            group.host_table.numpy()[slot, missing] = pages
            self._mark(group, slot, missing[0], missing[-1] + 1)

    def commit(self, request_id: str, new_len: int, tentative: bool = False) -> None:
        """The step wrote up to new_len; give back the pages a window has passed.  ``tentative``:
        the step may still be taken back (``rewind``), so nothing is given back until
        ``confirm``; ``save_states`` must have copied the request's state rows aside before the
        step was launched."""
        live = self._get(request_id)
        if new_len < live.length:
            raise ValueError("a request's length never shrinks")
        if tentative:
            if live.confirmed is None:
                live.confirmed = live.length
            live.length = new_len
            return
        if live.confirmed is not None:
            raise ValueError(f"request '{request_id}' has a tentative step: confirm or rewind it "
                             f"before the next final commit")
        live.length = new_len
        self._pass_window(request_id, live)

    def confirm(self, request_id: str) -> None:
        """The tentative steps of the request count: what ``commit`` held back happens now."""
        live = self._get(request_id)
        if live.confirmed is None:
            return
        live.confirmed = None
        self._pass_window(request_id, live)

    def _pass_window(self, request_id: str, live: _Live) -> None:
        new_len = live.length
        for group in self.paged:
            if group.spec.window is None:
                continue
            table = group.tables[request_id]
            first = min(self._first_needed(group, new_len), len(table))
            gone = [p for p in range(first) if table[p] >= 0]
            if gone:
                self._give(group, [table[p] for p in gone])
                row = group.host_table[live.slot]
                for p in gone:
                    table[p] = -1
                    row[p] = -1
                self._mark(group, live.slot, gone[0], gone[-1] + 1)

    def save_states(self, request_ids: "list[str]") -> None:
        """Copy the state rows of these requests aside (on the current stream), before a
        tentative step changes them.  Nothing to do for an architecture without such state."""
        if not self.states:
            return
        index = torch.tensor([self._get(r).slot for r in request_ids], dtype=torch.long,
                             device=self.device)
        for sgroup in self.states:
            if sgroup.saved is None:
                sgroup.saved = torch.empty_like(sgroup.state)
            sgroup.saved.index_copy_(1, index, sgroup.state.index_select(1, index))

    def rewind(self, request_id: str) -> None:
        """Take the request's tentative steps back: its length is what it was before them, its
        state rows are the ones ``save_states`` copied (restored on the current stream, after the
        kernels of the step that is taken back).  Pages stay with the request: it is about to
        need them again, and a tentative commit has given none back."""
        live = self._get(request_id)
        if live.confirmed is None:
            raise ValueError(f"request '{request_id}' has no tentative step to take back")
        live.length, live.confirmed = live.confirmed, None
        for sgroup in self.states:
            sgroup.state[:, live.slot].copy_(sgroup.saved[:, live.slot])

    def release(self, request_id: str) -> None:
        """Give back everything the request holds: its pages in every group and its slot."""
        live = self._get(request_id)
        for group in self.paged:
            table = group.tables.pop(request_id)
            held = [p for p in table if p >= 0]
            if held:
                self._give(group, held)
            if table:
                group.host_table[live.slot, : len(table)] = -1
                self._mark(group, live.slot, 0, len(table))
        self.slots.give(live.slot)
        del self.live[request_id]

    def _give(self, group: _PagedGroup, pages: list[int]) -> None:
        group.pool.give(pages)
        if self.poison:
            index = torch.tensor(pages, dtype=torch.long, device=self.device)
            group.k[:, index] = float("nan")
            group.v[:, index] = float("nan")

    def _mark(self, group: _PagedGroup, slot: int, lo: int, hi: int) -> None:
        span = group.dirty.get(slot)
        if span is None:
            group.dirty[slot] = [lo, hi]
        else:
            span[0], span[1] = min(span[0], lo), max(span[1], hi)

    # ------------------------------------------------------------------ device side
    def flush_tables(self) -> None:
        """Bring the changed parts of the block tables to the device (on the current stream).
        The rows are first copied into a pinned buffer that nothing else writes until the upload
        has happened, so the host may change its tables again at once."""
        spans = [(group, slot, lo, hi) for group in self.paged
                 for slot, (lo, hi) in group.dirty.items() if hi > lo]
        for group in self.paged:
            group.dirty.clear()
        if not spans:
            return
        total = sum(hi - lo for _, _, lo, hi in spans)
        if self._staged is None:                      # no CUDA device (tests of the host side)
            for group, slot, lo, hi in spans:
                group.device_table[slot, lo:hi].copy_(group.host_table[slot, lo:hi])
            return
        if self._stage_busy:
            self._staged.synchronize()                # the earlier upload has left the buffer
        if self._stage is None or self._stage.numel() < total:
            self._stage = torch.empty(max(2 * total, 1024), dtype=torch.int32).pin_memory()
        at = 0
        for group, slot, lo, hi in spans:
            piece = self._stage[at: at + hi - lo]
            piece.copy_(group.host_table[slot, lo:hi])
            group.device_table[slot, lo:hi].copy_(piece, non_blocking=True)
            at += hi - lo
        self._staged.record()
        self._stage_busy = True

    def bindings(self) -> "list[CacheBinding | None]":
        """For every plan entry the cache its run is given."""
        out: "list[CacheBinding | None]" = []
        for index, where in enumerate(self._where):
            source, writes = where, True
            if where is None and self._reads[index] is not None:
                source, writes = self._where[self._reads[index]], False
            if source is None:
                out.append(None)
                continue
            kind, g, layer = source
            if kind == "paged":
                group = self.paged[g]
                out.append(CacheBinding("paged", writes, group.k[layer], group.v[layer],
                                        group.device_table, self.page_size, group.spec.window))
            else:
                out.append(CacheBinding("state", writes, state=self.states[g].state[layer]))
        return out

    # ------------------------------------------------------------------ checks (tests)
    def check_invariants(self) -> None:
        """No page lost, none held twice, tables and free lists add up."""
        for group in self.paged:
            held: list[int] = []
            for table in group.tables.values():
                held += [p for p in table if p >= 0]
            free = group.pool.free_pages()
            if len(set(held)) != len(held):
                raise AssertionError("a page is held twice")
            if set(held) & set(free):
                raise AssertionError("a page is both held and free")
            if len(held) + len(free) != group.pool.num_pages or len(set(free)) != len(free):
                raise AssertionError("a page was lost or freed twice")
            for request_id, table in group.tables.items():
                row = group.host_table[self.live[request_id].slot]
                if [int(x) for x in row[: len(table)]] != table or bool((row[len(table):] >= 0).any()):
                    raise AssertionError("a block-table row disagrees with its request")
        slots = [live.slot for live in self.live.values()]
        if len(set(slots)) != len(slots) or len(slots) + self.slots.num_free != self.max_seqs:
            raise AssertionError("a slot was lost or is held twice")
