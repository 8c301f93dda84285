"""One step's batch on the flat token axis.

A step is a list of *entries*: (request, its next tokens, the places among them whose
logits are wanted).  A prompt portion is an entry with several tokens, a decoded token an
entry with one; they share one token axis of ``N = sum(n_tokens)`` rows.  The device-side
description (:class:`StepContext`) is built on the host into one pinned int32 buffer and
copied with a single transfer:

``token_ids[N]  positions[N]  seg_of_token[N]  seg_start[S+1]  seg_pos0[S]  slots[S]
logit_rows[R]  tile_seg[NT]  tile_q0[NT]  block_table[g][S][max_pages] for each paged group g``

(``tile_*`` list the 64-token query tiles of the step for the prefill attention kernel; a tile never
crosses a request)

(the reference's only per-pass metadata is the position vector,
src/Inference/Inference.jl:2322-2323, because it runs one sequence at a time).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Sequence

import numpy as np
import torch

from ..cache.manager import FREED


QUERY_TILE = 64   # tokens per query tile of the prefill attention kernel


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

    def offsets(self) -> Dict[str, int]:
        N, S, R = self.n_tokens, self.n_segs, self.n_rows
        o, cur = {}, 0
        for name, size in (("token_ids", N), ("positions", N), ("seg_of_token", N),
                           ("seg_start", S + 1), ("seg_pos0", S), ("slots", S), ("logit_rows", R),
                           ("tile_seg", self.n_tiles), ("tile_q0", self.n_tiles)):
            o[name] = cur
            cur += size
        for g in range(self.n_groups):
            o[f"block_table{g}"] = cur
            cur += S * self.max_pages
        o["_end"] = cur
        return o


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
        o = layout.offsets()
        N, S, R = self.n_tokens, self.n_segs, self.n_rows
        self.token_ids = buf[o["token_ids"]:o["token_ids"] + N]
        self.positions = buf[o["positions"]:o["positions"] + N]
        self.seg_of_token = buf[o["seg_of_token"]:o["seg_of_token"] + N]
        self.seg_start = buf[o["seg_start"]:o["seg_start"] + S + 1]
        self.seg_pos0 = buf[o["seg_pos0"]:o["seg_pos0"] + S]
        self.slots = buf[o["slots"]:o["slots"] + S]
        self.logit_rows = buf[o["logit_rows"]:o["logit_rows"] + R]
        self.n_tiles = layout.n_tiles
        self.tile_seg = buf[o["tile_seg"]:o["tile_seg"] + layout.n_tiles]
        self.tile_q0 = buf[o["tile_q0"]:o["tile_q0"] + layout.n_tiles]
        self.block_tables = [
            buf[o[f"block_table{g}"]:o[f"block_table{g}"] + S * layout.max_pages].view(S, layout.max_pages)
            for g in range(layout.n_groups)]

    @property
    def decode_only(self) -> bool:
        return self.max_seg_len == 1


def pack_step(entries: List[StepEntry], starts: List[int], slots: List[int],
              tables: List[List[List[int]]], layout: StepLayout, out: np.ndarray) -> None:
    """Fill the packed host buffer.  ``starts[i]`` is entry i's first position, ``tables[g][i]``
    its block table in group g."""
    o = layout.offsets()
    N = layout.n_tokens
    tok = out[o["token_ids"]:o["token_ids"] + N]
    pos = out[o["positions"]:o["positions"] + N]
    seg = out[o["seg_of_token"]:o["seg_of_token"] + N]
    seg_start = out[o["seg_start"]:o["seg_start"] + layout.n_segs + 1]
    rows = out[o["logit_rows"]:o["logit_rows"] + layout.n_rows]
    tile_seg = out[o["tile_seg"]:o["tile_seg"] + layout.n_tiles]
    tile_q0 = out[o["tile_q0"]:o["tile_q0"] + layout.n_tiles]
    if layout.n_tokens == layout.n_segs:
        # single tokens only (decoding): no per-entry loops
        S = layout.n_segs
        tok[:] = [e.tokens[0] for e in entries]
        pos[:] = starts
        seg[:] = np.arange(S, dtype=np.int32)
        seg_start[:] = np.arange(S + 1, dtype=np.int32)
        tile_seg[:] = seg
        tile_q0[:] = 0
        r = 0
        for i, e in enumerate(entries):
            for w in e.want:
                rows[r] = i + w
                r += 1
        _pack_tail(entries, starts, slots, tables, layout, out, o)
        return
    cur, r, nt = 0, 0, 0
    for i, e in enumerate(entries):
        n = len(e.tokens)
        for q0 in range(0, n, QUERY_TILE):
            tile_seg[nt] = i
            tile_q0[nt] = q0
            nt += 1
        tok[cur:cur + n] = np.asarray(e.tokens, dtype=np.int32)
        pos[cur:cur + n] = np.arange(starts[i], starts[i] + n, dtype=np.int32)
        seg[cur:cur + n] = i
        seg_start[i] = cur
        k = len(e.want)
        if k:
            rows[r:r + k] = np.asarray(e.want, dtype=np.int64) + cur
            r += k
        cur += n
    seg_start[layout.n_segs] = cur
    _pack_tail(entries, starts, slots, tables, layout, out, o)


def _pack_tail(entries, starts, slots, tables, layout, out, o) -> None:
    out[o["seg_pos0"]:o["seg_pos0"] + layout.n_segs] = np.asarray(starts, dtype=np.int32)
    out[o["slots"]:o["slots"] + layout.n_segs] = np.asarray(slots, dtype=np.int32)
    for g in range(layout.n_groups):
        bt = out[o[f"block_table{g}"]:o[f"block_table{g}"] + layout.n_segs * layout.max_pages]
        bt = bt.reshape(layout.n_segs, layout.max_pages)
        bt[:] = FREED
        for i, t in enumerate(tables[g]):
            if isinstance(t, np.ndarray):
                bt[i, :] = t                      # the manager's fixed-width row
            elif t:
                bt[i, :len(t)] = np.asarray(t, dtype=np.int32)
