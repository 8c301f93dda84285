"""One step's batch on the flat token axis.

A step is a list of *entries*: (request, its next tokens, the places among them whose
logits are wanted).  A prompt portion is an entry with several tokens, a decoded token an
entry with one; they share one token axis of ``N = sum(n_tokens)`` rows.  The device-side
description (:class:`StepContext`) is built on the host into one pinned int32 buffer and
copied with a single transfer.

**The layout of that buffer is decided here and nowhere else.**  :data:`CORE_FIELDS` lists the
fields every step has, in order, each with the axis it runs along; the block tables of the paged
groups follow, then any fields registered with :func:`register_step_field` (a mixer that needs one
more array per segment, token, wanted row or tile adds a line there and a function that fills it).
:meth:`StepLayout.offsets` turns the table into offsets; the native packer
(``csrc/host/step_packer.cpp``) is handed those offsets and only knows what goes *into* a core
field, and :class:`StepContext` cuts the device buffer by the same offsets.

``tile_*`` list the 64-token query tiles of the step for the prefill attention kernel; a tile never
crosses a request.  (The reference's only per-pass metadata is the position vector,
src/Inference/Inference.jl:2322-2323, because it runs one sequence at a time.)
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import FREED
from ..csrc import hostlib
from ..errors import ErrorCode, GessoError, invalid, resource


QUERY_TILE = 64   # tokens per query tile of the prefill attention kernel

# (name, axis): what every step carries.  The order is the field numbering of csrc/host/step_packer.cpp.
CORE_FIELDS: Tuple[Tuple[str, str], ...] = (
    ("token_ids", "token"),        # token ids
    ("positions", "token"),        # absolute position of every token
    ("seg_of_token", "token"),     # segment (entry) of every token
    ("seg_start", "seg+1"),        # first token of every segment, and the total
    ("seg_pos0", "seg"),           # position of a segment's first token
    ("slots", "seg"),              # state slot of a segment's request
    ("logit_rows", "row"),         # tokens whose logits are wanted
    ("tile_seg", "tile"),          # the step's query tiles: segment ...
    ("tile_q0", "tile"),           # ... and first token inside the segment
    ("kv_span", "two"),            # the longest sequence after the step and the average one (how decode attention cuts keys)
)

# fields added from outside: name -> (axis, fill(entries, view)); they follow the block tables
_EXTRA_FIELDS: Dict[str, Tuple[str, Callable]] = {}


def register_step_field(name: str, axis: str, fill: Callable[[List["StepEntry"], np.ndarray], None]) -> None:
    """One more int32 array in every step's metadata: ``axis`` is ``token``, ``seg``, ``seg+1``, ``row`` or
    ``tile``; ``fill(entries, view)`` writes it on the host (``entries`` include the stand-ins of a padded
    step, whose ``req_id`` is ``None``).  Parts read it as ``ctx.extra[name]``."""
    if axis not in ("token", "seg", "seg+1", "row", "tile"):
        raise invalid(f"step field {name!r}: unknown axis {axis!r}")
    if name in _EXTRA_FIELDS or any(name == n for n, _ in CORE_FIELDS) or name.startswith("block_table"):
        raise invalid(f"step field {name!r} exists already")
    _EXTRA_FIELDS[name] = (axis, fill)


def unregister_step_field(name: str) -> None:
    _EXTRA_FIELDS.pop(name, None)


def count_tiles(lengths) -> int:
    return sum((n + QUERY_TILE - 1) // QUERY_TILE for n in lengths)


@dataclass
class StepEntry:
    req_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)   # indices into ``tokens``


@dataclass
class StepLayout:
    """Sizes that fix the layout of the packed metadata buffer."""

    n_tokens: int
    n_segs: int
    n_rows: int
    n_groups: int
    max_pages: int
    n_tiles: int = 0

    def _axis(self, axis: str) -> int:
        return {"token": self.n_tokens, "seg": self.n_segs, "seg+1": self.n_segs + 1, "row": self.n_rows,
                "tile": self.n_tiles, "two": 2}[axis]

    def offsets(self) -> Dict[str, int]:
        o = getattr(self, "_offsets", None)
        if o is not None:
            return o
        o, cur = {}, 0
        for name, axis in CORE_FIELDS:
            o[name] = cur
            cur += self._axis(axis)
        for g in range(self.n_groups):
            o[f"block_table{g}"] = cur
            cur += self.n_segs * self.max_pages
        for name, (axis, _) in _EXTRA_FIELDS.items():
            o[name] = cur
            cur += self._axis(axis)
        o["_end"] = cur
        self._offsets = o
        return o

    def sizes(self) -> Dict[str, int]:
        s = {name: self._axis(axis) for name, axis in CORE_FIELDS}
        s.update({name: self._axis(axis) for name, (axis, _) in _EXTRA_FIELDS.items()})
        return s


class StepContext:
    """Device views of one step's metadata plus the host-side sizes kernels are launched with."""

    def __init__(self, layout: StepLayout, buf: torch.Tensor, status: torch.Tensor,
                 max_seg_len: int, max_kv_len: int, rows_are_all_tokens: bool = False):
        self.layout = layout
        self.buf = buf
        self.status = status
        self.n_tokens, self.n_segs, self.n_rows = layout.n_tokens, layout.n_segs, layout.n_rows
        self.max_seg_len = max_seg_len      # longest portion of the step
        self.max_kv_len = max_kv_len        # longest sequence after the step
        self.rows_are_all_tokens = rows_are_all_tokens   # logit_rows == 0..N-1
        o, sizes = layout.offsets(), layout.sizes()
        for name, _ in CORE_FIELDS:         # ctx.token_ids, ctx.positions, ... ctx.tile_q0
            setattr(self, name, buf[o[name]:o[name] + sizes[name]])
        self.n_tiles = layout.n_tiles
        S = self.n_segs
        self.block_tables = [
            buf[o[f"block_table{g}"]:o[f"block_table{g}"] + S * layout.max_pages].view(S, layout.max_pages)
            for g in range(layout.n_groups)]
        self.extra = {name: buf[o[name]:o[name] + sizes[name]] for name in _EXTRA_FIELDS}

    @property
    def decode_only(self) -> bool:
        return self.max_seg_len == 1


# ---- packing -----------------------------------------------------------------------------------------
_E_NOT_LIVE, _E_CONTEXT, _E_PAGES, _E_BAD_ARG = -1, -4, -5, -6
_E_TWICE, _E_EMPTY_SEG, _E_TOKEN, _E_WANT = -20, -21, -22, -23


def _native_offsets(layout: StepLayout):
    arr = getattr(layout, "_native_off", None)
    if arr is None:
        o = layout.offsets()
        vals = [o[name] for name, _ in CORE_FIELDS] + [o[f"block_table{g}"] for g in range(layout.n_groups)]
        layout._native_off = arr = (ctypes.c_int * len(vals))(*vals)
        layout._native_sizes = (ctypes.c_int * 4)(layout.n_tokens, layout.n_segs, layout.n_rows, layout.n_tiles)
    return arr, layout._native_sizes


def prepare_step(cache, entries: Sequence[StepEntry], layout: StepLayout, out: np.ndarray, vocab: int,
                 scratch_slot: int, scratch_pages: Sequence[int], tokens_known: bool = True):
    """Check the entries, reserve the pages of all their requests (or of none) and fill ``out`` (int32,
    ``layout.offsets()["_end"]`` long) in one native call.  An entry whose ``req_id`` is ``None`` is a
    stand-in on the scratch slot and scratch pages.  With ``tokens_known=False`` the token ids are left
    zero, to be filled in later.  Returns ``(fresh slots, longest sequence after the step)``; a refusal is
    a :class:`GessoError` and leaves every request as it was."""
    n = len(entries)
    G = layout.n_groups
    handles = (ctypes.c_int64 * n)()
    n_new = (ctypes.c_int * n)()
    want_n = (ctypes.c_int * n)()
    # token ids go into one int32 array: arrays are copied as they are, runs of lists are converted together
    total = 0
    for e in entries:
        total += len(e.tokens)
    tok_np = np.empty(max(total, 1), dtype=np.int32) if tokens_known else None
    run: List[int] = []                 # ids of consecutive list entries not yet copied, and where they go
    run_at = 0
    wants: List[int] = []

    def flush(upto: int) -> None:
        nonlocal run
        if run:
            a = np.asarray(run)
            if a.dtype.kind not in "iu":
                raise invalid("step: tokens and wanted places must be integers")
            tok_np[run_at:upto] = a
            run = []

    cur = 0
    for i, e in enumerate(entries):
        if e.req_id is not None:
            h = cache.handle(e.req_id)
            if h is None:
                raise invalid(f"step: request {e.req_id!r} is not live (admit it first)")
            handles[i] = h
        k = n_new[i] = len(e.tokens)
        want_n[i] = len(e.want)
        if k < 1:
            raise invalid(f"step: request {e.req_id!r} brings no tokens")
        # ranges are checked here, on the values as given: the 32-bit arrays below would wrap a wider integer
        try:
            if tokens_known:
                t = e.tokens
                if isinstance(t, np.ndarray):
                    if t.ndim != 1 or t.dtype.kind not in "iu":
                        raise TypeError
                    lo, hi = int(t.min()), int(t.max())
                else:
                    lo, hi = (t[0], t[0]) if k == 1 else (min(t), max(t))
                if not (0 <= lo and hi < vocab):
                    bad = next(int(x) for x in t if not (0 <= x < vocab))
                    raise invalid(f"step: token id {bad} of request {e.req_id!r} is outside the vocabulary (0..{vocab - 1})")
                if isinstance(t, np.ndarray):
                    flush(cur)
                    tok_np[cur:cur + k] = t
                else:
                    if not run:
                        run_at = cur
                    run.extend(t)
            if want_n[i]:
                w = e.want.tolist() if isinstance(e.want, np.ndarray) else e.want
                if not (0 <= min(w) and max(w) < k):
                    bad = next(x for x in w if not (0 <= x < k))
                    raise invalid(f"step: wanted place {bad} of request {e.req_id!r} is outside its {k} tokens")
                wants.extend(w)
        except TypeError:
            raise invalid(f"step: tokens and wanted places of request {e.req_id!r} must be flat lists of integers") from None
        cur += k
    try:
        if tokens_known:
            flush(cur)
        tok_arr = tok_np.ctypes.data_as(ctypes.POINTER(ctypes.c_int)) if tokens_known else None
        want_arr = (ctypes.c_int * max(len(wants), 1))(*wants)
    except (TypeError, ValueError, OverflowError):
        raise invalid("step: tokens and wanted places must be integers") from None
    off, sizes = _native_offsets(layout)
    scratch = (ctypes.c_int * (1 + G))(scratch_slot, *scratch_pages)
    fresh = (ctypes.c_int * n)()
    info = (ctypes.c_int * 8)()
    e = hostlib.library().gesso_step_prepare(
        cache.native(), handles, n_new, n, tok_arr, want_n, want_arr, off, len(off), sizes, G, layout.max_pages,
        QUERY_TILE, int(vocab), scratch, ctypes.c_void_p(out.ctypes.data), int(out.size), fresh, info)
    if e != 0:
        raise _refusal(e, info, entries, cache, vocab)
    if _EXTRA_FIELDS:
        o, sz = layout.offsets(), layout.sizes()
        for name, (_, fill) in _EXTRA_FIELDS.items():
            fill(list(entries), out[o[name]:o[name] + sz[name]])
    return list(fresh[:info[0]]), info[1]


def _refusal(e: int, info, entries, cache, vocab) -> GessoError:
    i = info[4] if 0 <= info[4] < len(entries) else 0
    rid = entries[i].req_id
    if e == _E_TWICE:
        return invalid(f"step: request {rid!r} appears twice in one step")
    if e == _E_EMPTY_SEG:
        return invalid(f"step: request {rid!r} brings no tokens")
    if e == _E_TOKEN:
        return invalid(f"step: token id {info[5]} of request {rid!r} is outside the vocabulary (0..{vocab - 1})")
    if e == _E_WANT:
        return invalid(f"step: wanted place {info[5]} of request {rid!r} is outside its {len(entries[i].tokens)} tokens")
    if e == _E_NOT_LIVE:
        return invalid(f"step: request {rid!r} is not live (admit it first)")
    if e == _E_CONTEXT:
        return resource(f"request {rid!r}: {cache.length(rid)}+{len(entries[i].tokens)} positions exceed the context "
                        f"length {cache.max_positions}")
    if e == _E_PAGES:
        return resource("step needs " + cache.last_short())
    return GessoError(ErrorCode.INTERNAL, f"step packer: the step does not fit its layout ({e})")
