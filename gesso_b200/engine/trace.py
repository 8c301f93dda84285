"""Trace replay: given token ids go through the engine step by step, logits come out.

Nothing is sampled.  The replay drives the same model, step function, cache and kernels
that generation uses; it has no forward pass, cache or loader of its own.  Input is one JSON
object per line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

A request is admitted the first time its id appears; ``end`` lists requests whose pages and
slot are given back after the step.  For a step in which something is wanted the logits at
the wanted places are written to ``<out>/<step>.f32`` as little-endian float32 ``[wanted,
vocab]`` in the order of the entries and of ``want``.  After every step ``done <step>`` is
printed and flushed.

The reference's closest tools are a capturing sampler that records each logits row
(test/test_lfm25.jl:5-12, 178-187) and ``scripts/fill_logits.jl``; it has no batch-level
replay.
"""
from __future__ import annotations

import json
import os
import sys
from typing import IO, Optional

import numpy as np

from ..errors import invalid
from .batch import StepEntry
from .engine import Engine

PAGE_ROUND = 64   # a request's token count is rounded up to this (or to the page size, if larger)


def make_engine(model, max_tokens: int, page_size: int = 16, max_requests: int = 4, use_graphs: bool = True) -> Engine:
    """An engine whose page pool holds exactly ``max_tokens`` positions."""
    unit = max(PAGE_ROUND, page_size)
    if max_tokens < 1:
        raise invalid("--max-tokens must be >= 1")
    max_tokens = unit * ((max_tokens + unit - 1) // unit)
    return Engine(model, max_positions=min(max_tokens, model.rt.max_positions), page_size=page_size,
                  num_pages=max_tokens // page_size, max_requests=max_requests, use_graphs=use_graphs)


def replay(engine: Engine, lines: IO[str], out_dir: str, done: Optional[IO[str]] = None) -> int:
    os.makedirs(out_dir, exist_ok=True)
    done = done or sys.stdout
    n_steps = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        obj = json.loads(line)
        step = obj["step"]
        entries = []
        for e in obj.get("entries", []):
            rid = e["id"]
            if not engine.is_live(rid):
                engine.admit(rid)
            entries.append(StepEntry(rid, [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        if entries:
            logits = engine.step(entries)
            if logits is not None:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(out_dir, f"{step}.f32"))
        for rid in obj.get("end", []):
            if engine.is_live(rid):
                engine.release(rid)
        engine.check_status()
        done.write(f"done {step}\n")
        done.flush()
        n_steps += 1
    return n_steps
