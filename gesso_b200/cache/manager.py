"""The cache manager: pages with a block table per request, and fixed-size state slots.

Keys and values live in pages of ``page_size`` positions.  Layers with the same
need (same kv heads, head size and window) form a *group*; a group has a page
pool of its own and every request has one block table per group, so one page
id covers the same ``page_size`` positions in every layer of the group.  Pages
go back to the pool when the request ends, or, in a windowed group, as soon as
every position on them lies behind the window of all queries still to come;
freed pages are reused at once (last freed, first reused).

Beside the pages every request holds one *slot*: the index of its fixed-size
state (the conv history of every conv layer, or whatever state a mixer
declares).  A slot is marked fresh when it is handed out, and the engine zeroes
its state before the first step that uses it.

The manager is host-side bookkeeping only: it owns no device memory and runs no
kernel (the reference's paged manager owns storage and append, and gathers on
read, src/Inference/kv_manager.jl:68-95, 234-297, 370-400; here kernels read
pages in place through the block table, so the manager only hands out
indices).  Running out of pages or slots is a typed error
(:class:`~gesso_b200.errors.GessoError`, ``RESOURCE_LIMIT``) as in the
reference (kv_manager.jl:246-257); what to do about it is the scheduler's
decision.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np

from ..errors import ErrorCode, GessoError, invalid, resource

FREED = -1   # block-table entry of a page that was given back (window) or never held


class IndexPool:
    """``count`` indices handed out and taken back; last freed is first reused."""

    def __init__(self, count: int, what: str):
        if count < 0:
            raise invalid(f"{what} pool size must be >= 0")
        self.count = count
        self.what = what
        self._free: List[int] = list(range(count - 1, -1, -1))   # pop() gives 0 first
        self._held = [False] * count

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.count - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise resource(f"no free {self.what} (all {self.count} in use)")
        i = self._free.pop()
        if self._held[i]:
            raise GessoError(ErrorCode.INTERNAL, f"{self.what} {i} handed out twice")
        self._held[i] = True
        return i

    def free(self, i: int) -> None:
        if not (0 <= i < self.count) or not self._held[i]:
            raise GessoError(ErrorCode.INTERNAL, f"{self.what} {i} freed but not held")
        self._held[i] = False
        self._free.append(i)

    def is_held(self, i: int) -> bool:
        return self._held[i]


@dataclass(frozen=True)
class PagedGroupSpec:
    """One group of layers with the same paging need."""

    name: str
    window: Optional[int] = None      # None: every earlier key is kept


@dataclass
class _Request:
    slot: int
    length: int = 0                               # positions committed so far
    reserved: int = 0                             # positions covered by pages (>= length)
    tables: List[List[int]] = field(default_factory=list)   # per group: page id per page index
    rows: List[np.ndarray] = field(default_factory=list)    # the same as fixed-width int32 rows (FREED padded)
    fresh: bool = True                            # state slot not zeroed yet


class CacheManager:
    def __init__(self, groups: Sequence[PagedGroupSpec], page_size: int, num_pages,
                 num_slots: int, max_positions: int):
        if page_size < 1:
            raise invalid("page_size must be >= 1")
        if max_positions < 1:
            raise invalid("max_positions must be >= 1")
        self.groups = list(groups)
        self.page_size = page_size
        self.max_positions = max_positions
        self.max_pages_per_request = (max_positions + page_size - 1) // page_size
        counts = list(num_pages) if isinstance(num_pages, (list, tuple)) else [num_pages] * len(self.groups)
        if len(counts) != len(self.groups):
            raise invalid("num_pages must give one count per paged group")
        for g in self.groups:
            if g.window is not None and g.window < 1:
                raise invalid(f"group {g.name}: window must be >= 1")
        self.pools = [IndexPool(c, f"page of group {g.name}") for c, g in zip(counts, self.groups)]
        self.slots = IndexPool(num_slots, "state slot")
        self._req: Dict[Hashable, _Request] = {}

    # ---- requests --------------------------------------------------------------------------
    def admit(self, req_id: Hashable) -> int:
        """Start a request: take a state slot (fresh) and empty block tables."""
        if req_id in self._req:
            raise invalid(f"request {req_id!r} is already live")
        slot = self.slots.alloc()
        self._req[req_id] = _Request(slot=slot, tables=[[] for _ in self.groups],
                                     rows=[np.full((self.max_pages_per_request,), FREED, dtype=np.int32)
                                           for _ in self.groups])
        return slot

    def is_live(self, req_id: Hashable) -> bool:
        return req_id in self._req

    def live_requests(self) -> List[Hashable]:
        return list(self._req)

    def _get(self, req_id: Hashable) -> _Request:
        r = self._req.get(req_id)
        if r is None:
            raise invalid(f"request {req_id!r} is not live")
        return r

    def length(self, req_id: Hashable) -> int:
        return self._get(req_id).length

    def slot(self, req_id: Hashable) -> int:
        return self._get(req_id).slot

    def take_fresh(self, req_id: Hashable) -> bool:
        """True exactly once per admission: the caller must zero the slot's state now."""
        r = self._get(req_id)
        was = r.fresh
        r.fresh = False
        return was

    # ---- pages -----------------------------------------------------------------------------
    def _pages_for(self, positions: int) -> int:
        return (positions + self.page_size - 1) // self.page_size

    def pages_needed(self, req_id: Hashable, n_new: int) -> List[int]:
        """Pages each group still has to hand out so that ``n_new`` more positions fit."""
        r = self._get(req_id)
        want = self._pages_for(r.length + n_new)
        return [max(0, want - len(t)) for t in r.tables]

    def can_reserve(self, req_id: Hashable, n_new: int) -> bool:
        r = self._get(req_id)
        if r.length + n_new > self.max_positions:
            return False
        return all(n <= p.free_count for n, p in zip(self.pages_needed(req_id, n_new), self.pools))

    def reserve(self, req_id: Hashable, n_new: int) -> None:
        """Hand out the pages for positions ``length .. length+n_new-1`` (all groups or none)."""
        r = self._get(req_id)
        if n_new < 0:
            raise invalid("n_new must be >= 0")
        if r.length + n_new > self.max_positions:
            raise resource(f"request {req_id!r}: {r.length}+{n_new} positions exceed the context "
                           f"length {self.max_positions}")
        need = self.pages_needed(req_id, n_new)
        for n, p, g in zip(need, self.pools, self.groups):
            if n > p.free_count:
                raise resource(f"group {g.name}: {n} pages needed, {p.free_count} free")
        for n, p, t, row in zip(need, self.pools, r.tables, r.rows):
            for _ in range(n):
                t.append(p.alloc())
                row[len(t) - 1] = t[-1]
        r.reserved = max(r.reserved, r.length + n_new)

    def reserve_single_tokens(self, req_ids: Sequence[Hashable]):
        """One more position for each request (a decoding step), all or none: returns
        ``(starts, slots, fresh_slots, rows)`` where ``rows[g][i]`` is request i's block-table row in
        group g.  The same checks as :meth:`reserve`, with one lookup per request."""
        reqs = []
        need = [0] * len(self.groups)
        ps = self.page_size
        for rid in req_ids:
            r = self._req.get(rid)
            if r is None:
                raise invalid(f"request {rid!r} is not live")
            if r.length + 1 > self.max_positions:
                raise resource(f"request {rid!r}: {r.length}+1 positions exceed the context length "
                               f"{self.max_positions}")
            want = (r.length + ps) // ps                     # pages that cover length + 1 positions
            for g, t in enumerate(r.tables):
                if want > len(t):
                    need[g] += want - len(t)
            reqs.append((r, want))
        for g, (k, p) in enumerate(zip(need, self.pools)):
            if k > p.free_count:
                raise resource(f"step needs {k} pages of group {self.groups[g].name}, {p.free_count} free")
        starts, slots, fresh = [], [], []
        rows: List[List[np.ndarray]] = [[] for _ in self.groups]
        for r, want in reqs:
            for g, (t, row, p) in enumerate(zip(r.tables, r.rows, self.pools)):
                while len(t) < want:
                    t.append(p.alloc())
                    row[len(t) - 1] = t[-1]
                rows[g].append(row)
            if r.length + 1 > r.reserved:
                r.reserved = r.length + 1
            starts.append(r.length)
            slots.append(r.slot)
            if r.fresh:
                r.fresh = False
                fresh.append(r.slot)
        return starts, slots, fresh, rows

    def commit(self, req_id: Hashable, n_new: int) -> None:
        """``n_new`` positions were written; windowed groups give back what no query will read."""
        r = self._get(req_id)
        if r.length + n_new > r.reserved:
            raise GessoError(ErrorCode.INTERNAL,
                             f"request {req_id!r}: commit of {n_new} beyond the reserved {r.reserved}")
        r.length += n_new
        for g, p, t, row in zip(self.groups, self.pools, r.tables, r.rows):
            if g.window is None:
                continue
            # the next query sits at position >= length and reads keys >= length - window + 1
            first_needed = r.length - g.window + 1
            dead_pages = max(0, first_needed) // self.page_size
            for i in range(min(dead_pages, len(t))):
                if t[i] != FREED:
                    p.free(t[i])
                    t[i] = FREED
                    row[i] = FREED

    def release(self, req_id: Hashable) -> None:
        """The request ended: its pages and its slot go back to the pools."""
        r = self._get(req_id)
        for p, t in zip(self.pools, r.tables):
            for page in reversed(t):
                if page != FREED:
                    p.free(page)
        self.slots.free(r.slot)
        del self._req[req_id]

    def block_table(self, req_id: Hashable, group: int) -> List[int]:
        return self._get(req_id).tables[group]

    def block_table_row(self, req_id: Hashable, group: int) -> np.ndarray:
        """The block table as a fixed-width int32 row (``FREED`` where no page is held); a view that the
        manager keeps up to date, for packing a step's metadata without a conversion."""
        return self._get(req_id).rows[group]

    # ---- accounting (derived, as the reference derives kv_bytes from its page table,
    #      src/Inference/kv_manager.jl:446-469) ---------------------------------------------------
    def pages_in_use(self) -> List[int]:
        return [p.held_count for p in self.pools]

    def slots_in_use(self) -> int:
        return self.slots.held_count

    def free_pages(self) -> List[int]:
        return [p.free_count for p in self.pools]

    def check_invariants(self) -> None:
        """No page lost, none held twice, the pools' counts equal what the tables hold."""
        for gi, (p, g) in enumerate(zip(self.pools, self.groups)):
            seen = set()
            for rid, r in self._req.items():
                for page in r.tables[gi]:
                    if page == FREED:
                        continue
                    if page in seen:
                        raise GessoError(ErrorCode.INTERNAL, f"group {g.name}: page {page} is held twice")
                    if not p.is_held(page):
                        raise GessoError(ErrorCode.INTERNAL, f"group {g.name}: page {page} of {rid!r} is not held")
                    seen.add(page)
            if len(seen) != p.held_count:
                raise GessoError(ErrorCode.INTERNAL,
                                 f"group {g.name}: {p.held_count} pages held but tables name {len(seen)}")
            if len(set(p._free)) != len(p._free) or seen & set(p._free):
                raise GessoError(ErrorCode.INTERNAL, f"group {g.name}: free list is inconsistent")
            if p.held_count + p.free_count != p.count:
                raise GessoError(ErrorCode.INTERNAL, f"group {g.name}: a page was lost")
        slots = [r.slot for r in self._req.values()]
        if len(set(slots)) != len(slots) or len(slots) != self.slots.held_count:
            raise GessoError(ErrorCode.INTERNAL, "state slots are inconsistent")
