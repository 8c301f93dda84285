"""Token selection: greedy, temperature and nucleus (top-p), one token per logits row.

Semantics are the reference's (src/Inference/sampling.jl:13-74, src/Inference/session.jl:447-458):

* greedy: argmax, ties go to the lowest id; a non-finite logit is a numerical failure and no token
  is emitted;
* ``Sampler(temperature > 0, top_p in (0, 1], seed >= 0)``: weights ``exp((logit - max) / T)`` in
  float64; with ``top_p = 1`` an inverse-CDF walk in id order, else the smallest set of most likely
  ids (ties by lower id) whose mass reaches ``top_p * total``, renormalised, walked in descending
  order; exactly one draw of the request's splitmix64 stream per call.
* ``temperature = 0`` (or no sampler) means greedy, as the reference's server maps it
  (docs/serving.md:103).

Selection runs on the device (``gesso_b200/csrc/sampling.cu``); the host only draws the uniform
numbers, so that a request's tokens depend on its own seed and not on the batch it is in.
:func:`sample_host` is the same rule on the host, for rows that are already there.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..errors import ErrorCode, GessoError, invalid

_M64 = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 0

    def __post_init__(self):
        if not (self.temperature >= 0) or math.isinf(self.temperature):
            raise invalid(f"sampler temperature must be >= 0 and finite, got {self.temperature}")
        if not (0 < self.top_p <= 1):
            raise invalid(f"sampler top_p must be in (0, 1], got {self.top_p}")
        if self.seed < 0:
            raise invalid(f"sampler seed must be >= 0, got {self.seed}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0


class SplitMix64:
    """The reference's generator (src/Inference/sampling.jl:32-39): 53-bit unit floats."""

    def __init__(self, seed: int):
        self.state = int(seed) & _M64

    def unit(self) -> float:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _M64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
        z ^= z >> 31
        return float(z >> 11) * 2.0 ** -53


def greedy_host(row: np.ndarray) -> int:
    if not np.isfinite(row).all():
        raise GessoError(ErrorCode.NUMERICAL_INSTABILITY, "nonfinite logits; no token may be emitted")
    return int(np.argmax(row))     # first index on ties


def sample_host(row: np.ndarray, params: SamplingParams, rng: SplitMix64) -> int:
    """The reference's rule on a host row (float64 weights, stable descending order for top-p)."""
    if params.greedy:
        return greedy_host(row)
    if not np.isfinite(row).all():
        raise GessoError(ErrorCode.NUMERICAL_INSTABILITY, "nonfinite logits; no token may be emitted")
    x = row.astype(np.float64)
    w = np.exp((x - x.max()) / params.temperature)
    total = float(np.add.accumulate(w)[-1])
    if params.top_p >= 1:
        r = rng.unit() * total
        acc = np.add.accumulate(w)
        i = int(np.searchsorted(acc, r, side="right"))
        return min(i, len(w) - 1)
    order = np.argsort(-w, kind="stable")
    acc = np.add.accumulate(w[order])
    keep = int(np.searchsorted(acc, params.top_p * total, side="left")) + 1
    keep = min(keep, len(w))
    cut = float(acc[keep - 1])
    r = rng.unit() * cut
    k = int(np.searchsorted(acc[:keep], r, side="right"))
    return int(order[min(k, keep - 1)])


_pinned: dict = {}
_pinned_turn: dict = {}


def _pinned_rows(R: int) -> torch.Tensor:
    """A pinned [2, R] int32 host buffer (ids and flags): the copy back needs no staging through pageable
    memory.  Four buffers per row count take turns, so that a selection that is still awaited keeps its
    buffer while the next ones are launched."""
    bufs = _pinned.get(R)
    if bufs is None:
        bufs = _pinned[R] = [torch.empty((2, R), dtype=torch.int32, pin_memory=True) for _ in range(4)]
        _pinned_turn[R] = 0
    _pinned_turn[R] = (_pinned_turn[R] + 1) % len(bufs)
    return bufs[_pinned_turn[R]]


class PendingSelection:
    """A selection that has been launched: the ids stay on the device (``ids``: int32 [R], for a next
    step that starts before the host has read them) and are on their way to pinned host memory."""

    def __init__(self, both: torch.Tensor, host: torch.Tensor, event: "torch.cuda.Event", rows: int):
        self.both, self.host, self.event, self.rows = both, host, event, rows

    @property
    def ids(self) -> torch.Tensor:
        return self.both[0]


def select_launch(logits: torch.Tensor, params: Sequence[SamplingParams],
                  rngs: Sequence[Optional[SplitMix64]]) -> Optional[PendingSelection]:
    """Launch the selection of one token per row of ``logits`` [R, V] (device, float32) and the copy of
    the result to the host, without waiting for either.  Sampled rows draw exactly one uniform number
    from their request's generator, now."""
    R = logits.shape[0]
    if R == 0:
        return None
    sampled = [i for i, p in enumerate(params) if not p.greedy]
    host = _pinned_rows(R)
    # all greedy: the selection kernel writes ids and flags into the pinned buffer itself (no copy operation
    # between this step and the next)
    direct = not sampled and ops.KERNEL_COPIES
    ids, bad = ops.argmax_rows(logits, host_out=host if direct else None)
    if not sampled and ids.data_ptr() + 4 * R == bad.data_ptr():
        # all greedy: ids and flags sit in one buffer, one copy brings both
        both = ids.new_empty(0).set_(ids.untyped_storage(), ids.storage_offset(), (2, R))
    else:
        if sampled:
            dev = logits.device
            # temperature, top-p, the uniform numbers and the pick mask in one pinned buffer, one copy
            hp = torch.empty((4, R), dtype=torch.float64, pin_memory=True)
            a = hp.numpy()
            for i in range(R):
                g = params[i].greedy
                a[0, i] = 1.0 if g else params[i].temperature
                a[1, i] = params[i].top_p
                a[2, i] = 0.0 if g else rngs[i].unit()
                a[3, i] = 0.0 if g else 1.0
            dp = hp.to(dev, non_blocking=True)
            sids, sbad = ops.sample_rows(logits, dp[0].contiguous(), dp[1].contiguous(), dp[2].contiguous())
            pick = dp[3] > 0.5
            ids = torch.where(pick, sids, ids)
            bad = torch.where(pick, sbad, bad)
        both = torch.stack([ids, bad])
    if not direct:
        host.copy_(both, non_blocking=True)
    event = torch.cuda.Event()
    event.record()
    return PendingSelection(both, host, event, R)


def select_wait(pending: Optional[PendingSelection]) -> List[object]:
    """The tokens of a launched selection: an ``int`` per row, or a :class:`GessoError` for a row whose
    logits are not finite (the caller fails that request only)."""
    if pending is None:
        return []
    pending.event.synchronize()
    host = pending.host.numpy()
    return [GessoError(ErrorCode.NUMERICAL_INSTABILITY, "nonfinite logits; no token may be emitted")
            if host[1, i] else int(host[0, i]) for i in range(pending.rows)]


def select_tokens(logits: torch.Tensor, params: Sequence[SamplingParams],
                  rngs: Sequence[Optional[SplitMix64]]) -> List[object]:
    """One token per row of ``logits`` [R, V] (device, float32).

    Returns a list with an ``int`` per row, or a :class:`GessoError` for a row whose logits are not
    finite (the caller fails that request only).  Sampled rows draw exactly one uniform number from
    their request's generator.
    """
    return select_wait(select_launch(logits, params, rngs))
