"""Builders of replay traces and the comparison with the plain implementation."""
from __future__ import annotations

import io
import json
import os
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

Record = Tuple[int, int, int, int]      # (step, row in the step's file, request, position)


def make_requests(vocab: int, lengths: Sequence[int], seed: int) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def round_up(n: int, m: int = 64) -> int:
    return m * ((n + m - 1) // m)


class TraceBuilder:
    def __init__(self):
        self.steps: List[dict] = []
        self.records: List[Record] = []

    def add_step(self, entries: List[Tuple[int, List[int], int, List[int]]], end: Sequence[int] = ()):
        """entries: (request, tokens, position of tokens[0], wanted places)."""
        step = len(self.steps)
        row = 0
        out = []
        for rid, toks, pos0, want in entries:
            out.append({"id": f"r{rid}", "tokens": list(toks), "want": list(want)})
            for w in want:
                self.records.append((step, row, rid, pos0 + w))
                row += 1
        self.steps.append({"step": step, "entries": out, "end": [f"r{r}" for r in end]})

    def text(self) -> str:
        return "".join(json.dumps(s) + "\n" for s in self.steps)


def trace_whole(reqs) -> Tuple[TraceBuilder, int]:
    tb = TraceBuilder()
    for i, t in enumerate(reqs):
        tb.add_step([(i, t, 0, list(range(len(t))))], end=[i])
    return tb, max(round_up(len(t)) for t in reqs)


def trace_tail_decode(reqs, tail: int = 32) -> Tuple[TraceBuilder, int]:
    """Most of each request in one step, the last ``tail`` tokens one by one."""
    tb = TraceBuilder()
    for i, t in enumerate(reqs):
        head = max(1, len(t) - tail)
        tb.add_step([(i, t[:head], 0, list(range(head)))])
        for p in range(head, len(t)):
            tb.add_step([(i, [t[p]], p, [0])], end=[i] if p == len(t) - 1 else [])
        if head == len(t):
            tb.steps[-1]["end"] = [f"r{i}"]
    return tb, max(round_up(len(t)) for t in reqs)


def trace_portions(reqs, sizes=(7, 2, 5, 3, 2, 11, 2, 4)) -> Tuple[TraceBuilder, int]:
    tb = TraceBuilder()
    k = 0
    for i, t in enumerate(reqs):
        p = 0
        while p < len(t):
            n = min(sizes[k % len(sizes)], len(t) - p)
            if len(t) - p - n == 1:      # never leave a single token for a "portion"
                n += 1
            k += 1
            last = p + n == len(t)
            tb.add_step([(i, t[p:p + n], p, list(range(n)))], end=[i] if last else [])
            p += n
    return tb, max(round_up(len(t)) for t in reqs)


def trace_mixed(reqs, seed: int, max_live: int = 4, decode_tail: int = 12,
                sizes=(9, 2, 17, 3, 5, 2, 33)) -> Tuple[TraceBuilder, int]:
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of others,
    requests left out of a step now and then, ends and arrivals interleaved.  Returns the trace and
    the largest sum of rounded-up lengths that was live at once (the pool the replay gets)."""
    rng = np.random.default_rng(seed)
    tb = TraceBuilder()
    waiting = list(range(len(reqs)))
    live: Dict[int, int] = {}            # request -> tokens fed so far
    peak, k = 0, 0
    while waiting or live:
        while waiting and len(live) < max_live:
            live[waiting.pop(0)] = 0
        peak = max(peak, sum(round_up(len(reqs[r])) for r in live))
        entries, end = [], []
        for r in list(live):
            t, p = reqs[r], live[r]
            if len(live) > 1 and rng.random() < 0.2:
                continue                  # left out of this step, goes on later
            left = len(t) - p
            if left <= decode_tail:
                n = 1
            else:
                n = min(sizes[k % len(sizes)], left - decode_tail)
                k += 1
            if rng.random() < 0.6 or n == 1:
                want = list(range(n))
            else:
                want = [n - 1]
            entries.append((r, t[p:p + n], p, want))
            live[r] = p + n
            if live[r] == len(t):
                end.append(r)
        if not entries:
            continue
        order = rng.permutation(len(entries))
        tb.add_step([entries[i] for i in order], end=end)
        for r in end:
            del live[r]
    return tb, peak


# ---- running and comparing --------------------------------------------------------------------------
def run_in_process(model, tb: TraceBuilder, max_tokens: int, out_dir: str, page_size: int = 16, prepare=None,
                   max_requests: int = 4, use_graphs: bool = True):
    """Replay ``tb`` on a fresh engine; ``prepare(engine)`` may touch the engine before the first step."""
    from gesso_b200.engine import trace
    eng = trace.make_engine(model, max_tokens, page_size=page_size, max_requests=max_requests, use_graphs=use_graphs)
    if prepare is not None:
        prepare(eng)
    sink = io.StringIO()
    trace.replay(eng, io.StringIO(tb.text()), out_dir, done=sink)
    assert sink.getvalue().count("done ") == len(tb.steps)
    eng.cache.check_invariants()
    assert eng.cache.live_requests() == []
    assert all(n == 0 for n in eng.cache.pages_in_use()) and eng.cache.slots_in_use() == 0
    return eng


def read_rows(tb: TraceBuilder, out_dir: str, vocab: int) -> Dict[Tuple[int, int], np.ndarray]:
    """(request, position) -> logits row, from the files a replay wrote."""
    files: Dict[int, np.ndarray] = {}
    out: Dict[Tuple[int, int], np.ndarray] = {}
    for step, row, rid, pos in tb.records:
        if step not in files:
            a = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4")
            assert a.size % vocab == 0
            files[step] = a.reshape(-1, vocab)
        out[(rid, pos)] = files[step][row]
    return out


def compare_with_plain(rows, plain_logits: List[np.ndarray], tol: float, what: str):
    """``max|engine - plain| <= tol * max(1, max|plain|)`` per request; reports the first bad place."""
    worst = 0.0
    by_req: Dict[int, List[int]] = {}
    for (rid, pos) in rows:
        by_req.setdefault(rid, []).append(pos)
    for rid, positions in sorted(by_req.items()):
        ref = plain_logits[rid]
        scale = max(1.0, float(np.abs(ref).max()))
        for pos in sorted(positions):
            err = float(np.abs(rows[(rid, pos)].astype(np.float64) - ref[pos]).max())
            worst = max(worst, err / scale)
            assert np.isfinite(rows[(rid, pos)]).all(), f"{what}: request {rid} position {pos}: non-finite logits"
            assert err <= tol * scale, (
                f"{what}: request {rid} position {pos} (of {len(ref)}): max error {err:.3e} "
                f"> {tol:.1e} * {scale:.3f}; first bad position of this request")
    return worst


def poison_free_memory(eng) -> None:
    """Fill every cache page and every state slot with NaN, as requests that went non-finite may have
    left them (on a fresh engine every page and slot is free, so this touches nothing a request owns)."""
    assert eng.cache.live_requests() == []
    for kv in eng.device_cache.kv:
        kv.fill_(float("nan"))
    for st in eng.device_cache.state:
        if st.is_floating_point():
            st.fill_(float("nan"))
