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

The bookkeeping itself is native (``csrc/host/cache_manager.cpp``, C++ behind a
C ABI); this module gives it the engine's interface: request ids of any hashable
type, typed errors with readable messages, block tables as numpy rows.  It is
host-side bookkeeping only: it owns no device memory and runs no kernel (the
reference's paged manager owns storage and append, and gathers on read,
src/Inference/kv_manager.jl:68-95, 234-297, 370-400; here kernels read pages in
place through the block table, so the manager only hands out indices).  Running
out of pages or slots is a typed error (:class:`~gesso_b200.errors.GessoError`,
``RESOURCE_LIMIT``) as in the reference (kv_manager.jl:246-257); what to do about
it is the scheduler's decision.
"""
from __future__ import annotations

import ctypes
import itertools
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np

from ..csrc import hostlib
from ..errors import ErrorCode, GessoError, invalid, resource

FREED = -1   # block-table entry of a page that was given back (window) or never held

# return codes of the native functions (csrc/host/cache_manager.cpp)
_E_NOT_LIVE, _E_LIVE, _E_NO_SLOT, _E_CONTEXT, _E_PAGES, _E_BAD_ARG, _E_COMMIT, _E_INVARIANT, _E_INDEX, _E_EMPTY = \
    -1, -2, -3, -4, -5, -6, -7, -8, -9, -10


class IndexPool:
    """``count`` indices handed out and taken back; last freed is first reused."""

    def __init__(self, count: int, what: str):
        if count < 0:
            raise invalid(f"{what} pool size must be >= 0")
        self.count = count
        self.what = what
        self._lib = hostlib.library()
        self._p = ctypes.c_void_p(self._lib.gesso_pool_new(count))

    def __del__(self):
        if getattr(self, "_p", None):
            self._lib.gesso_pool_delete(self._p)
            self._p = None

    @property
    def free_count(self) -> int:
        return self._lib.gesso_pool_free_count(self._p)

    @property
    def held_count(self) -> int:
        return self.count - self.free_count

    def alloc(self) -> int:
        i = self._lib.gesso_pool_alloc(self._p)
        if i == _E_EMPTY:
            raise resource(f"no free {self.what} (all {self.count} in use)")
        if i < 0:
            raise GessoError(ErrorCode.INTERNAL, f"{self.what} pool is inconsistent (an index was handed out twice)")
        return i

    def free(self, i: int) -> None:
        if self._lib.gesso_pool_free(self._p, int(i)) != 0:
            raise GessoError(ErrorCode.INTERNAL, f"{self.what} {i} freed but not held")

    def is_held(self, i: int) -> bool:
        return bool(self._lib.gesso_pool_is_held(self._p, int(i)))


@dataclass(frozen=True)
class PagedGroupSpec:
    """One group of layers with the same paging need."""

    name: str
    window: Optional[int] = None      # None: every earlier key is kept


class _PoolView:
    """What the scheduler reads of a pool of the native manager: its size and how much is free."""

    def __init__(self, manager: "CacheManager", index: int, count: int):
        self._m, self._i, self.count = manager, index, count

    @property
    def free_count(self) -> int:
        c = self._m._counts()
        G = len(self._m.groups)
        return c[2 * G + 1] if self._i < 0 else c[G + self._i]

    @property
    def held_count(self) -> int:
        return self.count - self.free_count


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
        if any(c < 0 for c in counts):
            raise invalid("page pool size must be >= 0")
        if num_slots < 0:
            raise invalid("state slot pool size must be >= 0")
        G = len(self.groups)
        self._lib = hostlib.library()
        windows = (ctypes.c_int * max(G, 1))(*[g.window or 0 for g in self.groups])
        pages = (ctypes.c_int * max(G, 1))(*counts)
        self._cm = ctypes.c_void_p(self._lib.gesso_cm_new(G, windows, page_size, pages, num_slots, max_positions))
        if not self._cm:
            raise invalid("cache manager: sizes out of range")
        self.pools = [_PoolView(self, i, c) for i, c in enumerate(counts)]
        self.slots = _PoolView(self, -1, num_slots)
        self._handle: Dict[Hashable, int] = {}          # request id -> native handle
        self._rows: Dict[Hashable, List[np.ndarray]] = {}   # request id -> the native block tables as numpy views
        self._length: Dict[Hashable, int] = {}          # request id -> committed positions (mirror, for cheap reads)
        self._slot: Dict[Hashable, int] = {}
        self._next = itertools.count(1)
        self._ibuf = (ctypes.c_int * (2 * G + 8))()

    def __del__(self):
        if getattr(self, "_cm", None):
            self._lib.gesso_cm_delete(self._cm)
            self._cm = None

    # ---- requests --------------------------------------------------------------------------
    def _h(self, req_id: Hashable) -> int:
        h = self._handle.get(req_id)
        if h is None:
            raise invalid(f"request {req_id!r} is not live")
        return h

    def _counts(self):
        self._lib.gesso_cm_counts(self._cm, self._ibuf)
        return self._ibuf

    def _short(self) -> str:
        self._lib.gesso_cm_last_short(self._cm, self._ibuf)
        g, need, free = self._ibuf[0], self._ibuf[1], self._ibuf[2]
        return f"group {self.groups[g].name}: {need} pages needed, {free} free"

    def admit(self, req_id: Hashable) -> int:
        """Start a request: take a state slot (fresh) and empty block tables."""
        if req_id in self._handle:
            raise invalid(f"request {req_id!r} is already live")
        h = next(self._next)
        slot = self._lib.gesso_cm_admit(self._cm, h)
        if slot == _E_NO_SLOT:
            raise resource(f"no free state slot (all {self.slots.count} in use)")
        if slot < 0:
            raise GessoError(ErrorCode.INTERNAL, f"cache manager: admit failed ({slot})")
        self._handle[req_id] = h
        self._length[req_id] = 0
        self._slot[req_id] = slot
        n = ctypes.c_int()
        self._rows[req_id] = [
            np.ctypeslib.as_array(self._lib.gesso_cm_row(self._cm, h, g, ctypes.byref(n)),
                                  shape=(self.max_pages_per_request,))
            for g in range(len(self.groups))]
        return slot

    def is_live(self, req_id: Hashable) -> bool:
        return req_id in self._handle

    def live_requests(self) -> List[Hashable]:
        return list(self._handle)

    def _info(self, req_id: Hashable):
        self._lib.gesso_cm_info(self._cm, self._h(req_id), self._ibuf)
        return self._ibuf

    def length(self, req_id: Hashable) -> int:
        n = self._length.get(req_id)
        if n is None:
            raise invalid(f"request {req_id!r} is not live")
        return n

    def slot(self, req_id: Hashable) -> int:
        self._h(req_id)
        return self._slot[req_id]

    def take_fresh(self, req_id: Hashable) -> bool:
        """True exactly once per admission: the caller must zero the slot's state now."""
        return self._lib.gesso_cm_take_fresh(self._cm, self._h(req_id)) == 1

    # ---- pages -----------------------------------------------------------------------------
    def pages_needed(self, req_id: Hashable, n_new: int) -> List[int]:
        """Pages each group still has to hand out so that ``n_new`` more positions fit."""
        self._lib.gesso_cm_pages_needed(self._cm, self._h(req_id), int(n_new), self._ibuf)
        return list(self._ibuf[:len(self.groups)])

    def can_reserve(self, req_id: Hashable, n_new: int) -> bool:
        if self.length(req_id) + n_new > self.max_positions:
            return False
        need = self.pages_needed(req_id, n_new)
        return all(n <= f for n, f in zip(need, self.free_pages()))

    def reserve(self, req_id: Hashable, n_new: int) -> None:
        """Hand out the pages for positions ``length .. length+n_new-1`` (all groups or none)."""
        h = self._h(req_id)
        if n_new < 0:
            raise invalid("n_new must be >= 0")
        e = self._lib.gesso_cm_reserve(self._cm, h, int(n_new))
        if e == 0:
            return
        if e == _E_CONTEXT:
            raise resource(f"request {req_id!r}: {self.length(req_id)}+{n_new} positions exceed the context "
                           f"length {self.max_positions}")
        if e == _E_PAGES:
            raise resource(self._short())
        raise GessoError(ErrorCode.INTERNAL, f"cache manager: reserve failed ({e})")

    def reserve_single_tokens(self, req_ids: Sequence[Hashable]):
        """One more position for each request (a decoding step), all or none: returns
        ``(starts, slots, fresh_slots, rows)`` where ``rows[g][i]`` is request i's block-table row in
        group g.  The same checks as :meth:`reserve`."""
        need = [0] * len(self.groups)
        free = self.free_pages()
        for rid in req_ids:
            if self.length(rid) + 1 > self.max_positions:
                raise resource(f"request {rid!r}: {self.length(rid)}+1 positions exceed the context length "
                               f"{self.max_positions}")
            for g, k in enumerate(self.pages_needed(rid, 1)):
                need[g] += k
        for g, (k, f) in enumerate(zip(need, free)):
            if k > f:
                raise resource(f"step needs {k} pages of group {self.groups[g].name}, {f} free")
        starts, slots, fresh = [], [], []
        for rid in req_ids:
            self.reserve(rid, 1)
            info = self._info(rid)
            starts.append(info[0])
            slots.append(info[2])
            if self.take_fresh(rid):
                fresh.append(slots[-1])
        rows = [[self._rows[rid][g] for rid in req_ids] for g in range(len(self.groups))]
        return starts, slots, fresh, rows

    # ---- for the step packer (csrc/host/step_packer.cpp), which drives the native manager itself ---------
    def handle(self, req_id: Hashable) -> Optional[int]:
        """The native handle of a live request, ``None`` if it is not live."""
        return self._handle.get(req_id)

    def native(self):
        """The native manager, for calls that take it as an argument."""
        return self._cm

    def last_short(self) -> str:
        """Which group ran short in the refusal just returned, in words."""
        self._lib.gesso_cm_last_short(self._cm, self._ibuf)
        return f"{self._ibuf[1]} pages of group {self.groups[self._ibuf[0]].name}, {self._ibuf[2]} free"

    def reserve_step(self, req_ids: Sequence[Hashable], n_new: Sequence[int]):
        """The pages of a whole step in one native call: ``n_new[i]`` more positions for request i, for
        all requests or for none.  Returns ``(starts, slots, fresh_slots, longest sequence after the
        step, block-table rows per group)``; the state of the fresh slots must be zeroed before the step."""
        n = len(req_ids)
        rids = (ctypes.c_int64 * n)(*[self._h(r) for r in req_ids])
        news = (ctypes.c_int * n)(*[int(k) for k in n_new])
        starts, slots, fresh = (ctypes.c_int * n)(), (ctypes.c_int * n)(), (ctypes.c_int * n)()
        info = (ctypes.c_int * 4)()
        e = self._lib.gesso_cm_reserve_step(self._cm, rids, news, n, starts, slots, fresh, info)
        if e == 0:
            rows = [[self._rows[rid][g] for rid in req_ids] for g in range(len(self.groups))]
            return list(starts), list(slots), list(fresh[:info[0]]), info[1], rows
        if e == _E_PAGES:
            self._lib.gesso_cm_last_short(self._cm, self._ibuf)
            raise resource(f"step needs {self._ibuf[1]} pages of group {self.groups[self._ibuf[0]].name}, "
                           f"{self._ibuf[2]} free")
        if e == _E_CONTEXT:
            rid = req_ids[info[0]]
            raise resource(f"request {rid!r}: {self.length(rid)}+{n_new[info[0]]} positions exceed the context "
                           f"length {self.max_positions}")
        if e == _E_BAD_ARG and 0 <= info[0] < n and list(req_ids).count(req_ids[info[0]]) > 1:
            raise invalid("step: a request appears twice in one step")
        raise GessoError(ErrorCode.INTERNAL, f"cache manager: reserving a step failed ({e})")

    def commit_step(self, req_ids: Sequence[Hashable], n_new: Sequence[int]) -> None:
        """``n_new[i]`` positions of request i were written."""
        n = len(req_ids)
        rids = (ctypes.c_int64 * n)(*[self._h(r) for r in req_ids])
        news = (ctypes.c_int * n)(*[int(k) for k in n_new])
        e = self._lib.gesso_cm_commit_step(self._cm, rids, news, n)
        if e != 0:
            raise GessoError(ErrorCode.INTERNAL, f"cache manager: commit of a step failed ({e})")
        for r, k in zip(req_ids, n_new):
            self._length[r] += int(k)

    def commit(self, req_id: Hashable, n_new: int) -> None:
        """``n_new`` positions were written; windowed groups give back what no query will read."""
        e = self._lib.gesso_cm_commit(self._cm, self._h(req_id), int(n_new))
        if e == _E_COMMIT:
            raise GessoError(ErrorCode.INTERNAL,
                             f"request {req_id!r}: commit of {n_new} beyond the reserved {self._info(req_id)[1]}")
        if e != 0:
            raise GessoError(ErrorCode.INTERNAL, f"cache manager: commit failed ({e})")
        self._length[req_id] += int(n_new)

    def commit_single_tokens(self, req_ids: Sequence[Hashable]) -> None:
        """One position of each request was written (a decoding step)."""
        n = len(req_ids)
        rids = (ctypes.c_int64 * n)(*[self._h(r) for r in req_ids])
        e = self._lib.gesso_cm_commit_many(self._cm, rids, n, 1)
        if e != 0:
            raise GessoError(ErrorCode.INTERNAL, f"cache manager: commit of a decoding step failed ({e})")
        for r in req_ids:
            self._length[r] += 1

    def release(self, req_id: Hashable) -> None:
        """The request ended: its pages and its slot go back to the pools."""
        h = self._h(req_id)
        e = self._lib.gesso_cm_release(self._cm, h)
        del self._handle[req_id]
        del self._rows[req_id]
        del self._length[req_id]
        del self._slot[req_id]
        if e != 0:
            raise GessoError(ErrorCode.INTERNAL, f"cache manager: release of {req_id!r} failed ({e})")

    def block_table(self, req_id: Hashable, group: int) -> List[int]:
        n = ctypes.c_int()
        row = self._lib.gesso_cm_row(self._cm, self._h(req_id), int(group), ctypes.byref(n))
        return [row[i] for i in range(n.value)]

    def block_table_row(self, req_id: Hashable, group: int) -> np.ndarray:
        """The block table as a fixed-width int32 row (``FREED`` where no page is held); a view that the
        manager keeps up to date, for packing a step's metadata without a conversion.  Valid until the
        request is released."""
        self._h(req_id)
        return self._rows[req_id][group]

    # ---- accounting (derived, as the reference derives kv_bytes from its page table,
    #      src/Inference/kv_manager.jl:446-469) ---------------------------------------------------
    def pages_in_use(self) -> List[int]:
        return list(self._counts()[:len(self.groups)])

    def slots_in_use(self) -> int:
        return self._counts()[2 * len(self.groups)]

    def free_pages(self) -> List[int]:
        G = len(self.groups)
        return list(self._counts()[G:2 * G])

    def check_invariants(self) -> None:
        """No page lost, none held twice, the pools' counts equal what the tables hold."""
        if self._lib.gesso_cm_check(self._cm) == 0:
            if self._counts()[2 * len(self.groups) + 2] != len(self._handle):
                raise GessoError(ErrorCode.INTERNAL, "live requests differ between the native manager and its wrapper")
            for rid in self._handle:
                if self._info(rid)[0] != self._length[rid]:
                    raise GessoError(ErrorCode.INTERNAL, f"request {rid!r}: the wrapper's length differs from the manager's")
            return
        self._lib.gesso_cm_last_short(self._cm, self._ibuf)
        g, kind, what = self._ibuf[0], self._ibuf[1], self._ibuf[2]
        name = self.groups[g].name if 0 <= g < len(self.groups) else "slots"
        text = {1: f"page {what} is held twice", 2: f"page {what} of a block table is not held",
                3: f"the pool holds more pages than the tables name ({what})", 4: "free list is inconsistent",
                5: "a page was lost", 6: "state slots are inconsistent"}.get(kind, f"kind {kind}")
        raise GessoError(ErrorCode.INTERNAL, f"group {name}: {text}")
