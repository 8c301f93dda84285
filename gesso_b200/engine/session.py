"""The Python entry point, shaped like the reference's ``Session`` / ``generate`` / ``run_batch``.

Reference API (names and meanings kept where this engine has the same thing):

* ``Session(model, tensors; page_size=16, context_length, eos_token_id, ...)``
  (src/Inference/session.jl:87-101, 188-199) -> ``Session(model, context_length=..., page_size=16,
  eos_token_id=...)``;
* ``prefill!(s, tokens) -> logits (V, P)`` (:681) -> ``s.prefill(tokens) -> ndarray [P, V]``;
* ``decode!(s) -> id`` (:840): greedy id from the last position; consumed unless it is the eos id
  (:861-863) -> ``s.decode() -> int``;
* ``generate(s, prompt; max_new_tokens=8, on_token) -> prompt + new ids`` (:1025-1060), and the
  sampling keywords of ``reference_generate`` (``stop_ids``, ``eos_ids``, ``sampler`` with
  ``temperature``, ``top_p``, ``seed``; src/Inference/Inference.jl:2059-2102) ->
  ``s.generate(prompt, max_new_tokens=8, on_token=None, temperature=0, top_p=1, seed=0, ...)``;
* ``run_batch([BatchRequest(session, prompt; max_new_tokens)]) -> [BatchResult(ids, status, error)]``
  with status ``complete | eos | cancelled | failed`` (src/Runtime/Runtime.jl:33-51, 130-182) ->
  ``s.run_batch([BatchRequest(prompt, max_new_tokens=...)])``; the requests share one engine and run
  as one continuously batched stream instead of a round-robin over sessions.

A Session is not re-entrant: a second call while one is running is refused
(src/Inference/session.jl:622-669).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import numpy as np
import torch

from ..errors import ErrorCode, GessoError, invalid
from ..sampling.sampler import SamplingParams, select_launch, select_tokens, select_wait
from .batch import StepEntry
from .engine import Engine
from .scheduler import CANCELLED, COMPLETE, EOS, FAILED, STOP, Request, Scheduler

_SOLO = "__session__"


@dataclass
class BatchRequest:
    prompt: Sequence[int]
    max_new_tokens: int = 8
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 0
    stop_ids: Sequence[int] = ()
    eos_ids: Optional[Sequence[int]] = None     # None: the session's eos_token_id
    on_token: Optional[Callable[[int], Optional[bool]]] = None
    _request: Optional[Request] = field(default=None, repr=False)

    def cancel(self) -> None:
        """Observed before the request is admitted and between its tokens (Runtime.jl:45, 159-163)."""
        if self._request is not None:
            self._request.cancel()
        self._cancel_early = True


@dataclass
class BatchResult:
    ids: List[int]                 # prompt + new ids, the stopping id included
    status: str                    # complete | eos | stop | cancelled | failed
    error: Optional[Exception] = None


class _Select:
    """Token selection for the scheduler: at once, or launched now and awaited later (the scheduler runs
    steady decoding one step ahead of the host)."""

    def __call__(self, logits, requests):
        return select_tokens(logits, [r.sampling for r in requests], [r.rng for r in requests])

    def launch(self, logits, requests):
        return select_launch(logits, [r.sampling for r in requests], [r.rng for r in requests])

    def wait(self, pending):
        return select_wait(pending)


_select = _Select()


class Session:
    def __init__(self, model, *, context_length: Optional[int] = None, page_size: int = 16,
                 num_pages: Optional[int] = None, max_batch: int = 8, eos_token_id: Optional[int] = None,
                 max_tokens_per_step: int = 2048, prefill_chunk: int = 512):
        self.model = model
        ctx = int(context_length or model.rt.max_positions)
        self.engine = Engine(model, max_positions=ctx, page_size=page_size, num_pages=num_pages,
                             max_requests=max_batch)
        self.context_length = ctx
        self.eos_token_id = eos_token_id if eos_token_id is not None else model.spec.eos_token_id
        self.max_batch = max_batch
        self.max_tokens_per_step = max_tokens_per_step
        self.prefill_chunk = prefill_chunk
        self._busy = False
        self._open_batch: Optional[Scheduler] = None         # a stream opened by open_batch that still has work
        self._last_logits: Optional[torch.Tensor] = None     # [V], of the solo sequence's last position
        self.last_scheduler: Optional[Scheduler] = None

    # ---- guards ------------------------------------------------------------------------------------
    def _enter(self):
        if self._open_batch is not None and not self._open_batch.has_work:
            self._open_batch = None                   # the stream a caller stepped has run dry
        if self._busy or self._open_batch is not None:
            raise GessoError(ErrorCode.INVALID_PLAN, "Session is busy: it is not re-entrant")
        self._busy = True

    def _leave(self):
        self._busy = False

    def _eos(self, eos_ids):
        if eos_ids is not None:
            return tuple(int(i) for i in eos_ids)
        return () if self.eos_token_id is None else (int(self.eos_token_id),)

    def reset(self) -> None:
        """Forget the solo sequence (prefill/decode) and give back what it holds."""
        if self.engine.is_live(_SOLO):
            self.engine.release(_SOLO)
        self._last_logits = None

    # ---- prefill / decode of one sequence ---------------------------------------------------------
    def prefill(self, tokens: Sequence[int]) -> np.ndarray:
        """Run a whole prompt from an empty cache; returns float32 logits ``[P, V]``."""
        self._enter()
        try:
            tokens = [int(t) for t in tokens]
            if not tokens:
                raise invalid("prefill: empty prompt")
            self.reset()
            self.engine.admit(_SOLO)
            try:
                logits = self.engine.step([StepEntry(_SOLO, tokens, list(range(len(tokens))))])
                ticket = self.engine.status_read_launch()
                host = logits.to("cpu").numpy()          # waits for the step, and so for the status words
                bad = self.engine.status_read_finish(ticket)
                if bad is not None:
                    raise bad[0]
            except Exception:
                self.reset()
                raise
            self._last_logits = logits[-1]
            return host
        finally:
            self._leave()

    def decode(self) -> int:
        """Greedy id from the last position; it is run through the model unless it is the eos id."""
        self._enter()
        try:
            if self._last_logits is None:
                raise invalid("decode: nothing was prefilled")
            ticket = self.engine.status_read_launch()    # of the step that made these logits
            tok = _select_greedy(self._last_logits)
            bad = self.engine.status_read_finish(ticket)
            if bad is not None:
                self.reset()
                raise bad[0]
            if tok in self._eos(None):
                return tok
            if self.engine.length(_SOLO) >= self.context_length:
                raise GessoError(ErrorCode.RESOURCE_LIMIT, "decode: context length exhausted")
            self._last_logits = self.engine.step([StepEntry(_SOLO, [tok], [0])])[0]
            return tok
        finally:
            self._leave()

    @property
    def kv_len(self) -> int:
        return self.engine.length(_SOLO) if self.engine.is_live(_SOLO) else 0

    # ---- generation ---------------------------------------------------------------------------------
    def generate(self, prompt: Sequence[int], max_new_tokens: int = 8,
                 on_token: Optional[Callable[[int], Optional[bool]]] = None, *, temperature: float = 0.0,
                 top_p: float = 1.0, seed: int = 0, stop_ids: Sequence[int] = (),
                 eos_ids: Optional[Sequence[int]] = None) -> List[int]:
        """Prompt plus up to ``max_new_tokens`` new ids; the stopping id is returned but never run."""
        res = self.run_batch([BatchRequest(prompt, max_new_tokens, temperature, top_p, seed, stop_ids,
                                           eos_ids, on_token)])[0]
        if res.status == FAILED:
            raise res.error
        return res.ids

    def run_batch(self, requests: Sequence[BatchRequest]) -> List[BatchResult]:
        """All requests as one continuously batched stream; one result per request, in order.

        A request that fails (bad prompt, a callback that raises, non-finite logits, a step of the
        engine that raised or whose kernels reported an invalid result) is terminal for itself only
        (src/Runtime/Runtime.jl:151-153, 175-178): the others go on and every request gets a result."""
        self._enter()
        try:
            self.reset()
            sched = Scheduler(self.engine, _select, max_batch=self.max_batch,
                              max_tokens_per_step=self.max_tokens_per_step, prefill_chunk=self.prefill_chunk,
                              vocab_size=self.model.vocab_size)
            self.last_scheduler = sched
            results: List[Optional[BatchResult]] = [None] * len(requests)
            live = []
            for i, br in enumerate(requests):
                try:
                    req = Request(list(br.prompt), br.max_new_tokens,
                                  SamplingParams(float(br.temperature), float(br.top_p), int(br.seed)),
                                  self._eos(br.eos_ids), tuple(int(s) for s in br.stop_ids), br.on_token,
                                  req_id=f"b{i}")
                    br._request = req
                    if getattr(br, "_cancel_early", False):
                        req.cancel()
                    sched.add(req)
                    live.append((i, req))
                except GessoError as e:
                    results[i] = BatchResult([int(t) for t in br.prompt], FAILED, e)
            try:
                sched.run()
            except BaseException as e:
                # the scheduler itself gave up (a step's own failure never gets here): nobody is left
                # holding pages, and everybody still gets a result unless the caller interrupted
                err = e if isinstance(e, GessoError) else GessoError(
                    ErrorCode.INTERNAL, f"the scheduler stopped: {type(e).__name__}: {e}")
                for r in list(sched.running) + list(sched.waiting):
                    if r in sched.waiting:
                        sched.waiting.remove(r)
                    sched._finish(r, FAILED, err)
                if not isinstance(e, Exception):
                    raise
            for i, req in live:
                results[i] = BatchResult(req.ids, req.status or FAILED, req.error)
            return results
        finally:
            self._leave()

    def open_batch(self, requests: Sequence[BatchRequest]) -> Scheduler:
        """The same stream as :meth:`run_batch`, stepped by the caller: returns the scheduler with the
        requests added; every ``step()`` of it runs one engine step and returns the (request, token)
        pairs it emitted, until ``has_work`` is false.  Until then the session is busy: a second call is
        refused, as while ``run_batch`` runs."""
        self._enter()
        try:
            sched = self._open(requests)
        finally:
            self._leave()
        self._open_batch = sched if sched.has_work else None
        return sched

    def _open(self, requests: Sequence[BatchRequest]) -> Scheduler:
        self.reset()
        sched = Scheduler(self.engine, _select, max_batch=self.max_batch,
                          max_tokens_per_step=self.max_tokens_per_step, prefill_chunk=self.prefill_chunk,
                          vocab_size=self.model.vocab_size)
        self.last_scheduler = sched
        for i, br in enumerate(requests):
            req = Request(list(br.prompt), br.max_new_tokens,
                          SamplingParams(float(br.temperature), float(br.top_p), int(br.seed)),
                          self._eos(br.eos_ids), tuple(int(x) for x in br.stop_ids), br.on_token, req_id=f"b{i}")
            br._request = req
            sched.add(req)
        return sched

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """The raw step (:meth:`Engine.step`): ``entries`` of (request id, next tokens, wanted places) run as
        one batch from the cache; float32 logits ``[wanted, vocab]`` on the device.  The caller admits and
        releases its requests through ``session.engine``."""
        self._enter()
        try:
            return self.engine.step(entries)
        finally:
            self._leave()

    def stats(self):
        s = self.engine.stats()
        if self.last_scheduler is not None:
            s["scheduler_steps"] = self.last_scheduler.steps
            s["preemptions"] = self.last_scheduler.preemptions
            s["steps_ahead"] = self.last_scheduler.steps_ahead      # launched before the step before was digested
        return s


def _select_greedy(row: torch.Tensor) -> int:
    tok = select_tokens(row.reshape(1, -1).contiguous(), [SamplingParams()], [None])[0]
    if isinstance(tok, Exception):
        raise tok
    return tok


def generate(model, prompt: Sequence[int], max_new_tokens: int = 8, **kw) -> List[int]:
    """One-call form (the reference's ``reference_generate``, src/Inference/Inference.jl:2059-2102)."""
    ctx = kw.pop("context_length", None)
    s = Session(model, context_length=ctx, max_batch=1,
                num_pages=None)
    return s.generate(prompt, max_new_tokens, **kw)
