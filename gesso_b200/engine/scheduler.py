"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.

The reference runs one sequence at a time: fixed-size prefill passes
(src/Inference/Inference.jl:1765-1773) and a round-robin over independent sessions, one token per
active request per round (src/Runtime/Runtime.jl:130-182), with a typed error as its only answer
to an exhausted cache (src/Inference/kv_manager.jl:246-257).  This scheduler batches, so those
decisions are its own:

* **Admission**: first come, first served, while fewer than ``max_batch`` requests are live, a
  state slot is free and the pages of the request's first portion are free.
* **Budget**: every step first gives each decoding request its one token, then fills what is left
  of ``max_tokens_per_step`` with prompt portions of at most ``prefill_chunk`` tokens, oldest
  request first.  A portion may be cut anywhere.
* **Decoding**: the token sampled from a request's last logits is emitted; if it stops the request
  (``max_new_tokens`` reached, an eos/stop id, the callback returned ``False``) it is NOT run
  through the model (src/Inference/Inference.jl:2585-2592, 2046-2048), else it is the request's
  one token of the next step.
* **Pages run out**: new admissions stop first; then prompt portions are shrunk or dropped, newest
  request first; if the decoding requests alone do not fit, the most recently admitted running
  request is *preempted*: its pages and slot are freed and it goes back to the head of the queue
  with everything it has produced so far kept, to be re-prefilled later (recompute; the conv state
  is rebuilt by the re-prefill; its sampler stream is untouched, so its tokens do not change).
  The oldest request is never preempted, and a request that could not fit an empty pool is refused
  when it is added, so the queue always makes progress.
* **Finish**: pages and slot go back to the pools in the same step.
* **A step that fails** (the engine raises, or a kernel reports through the engine's status words that
  what it computed is not valid) fails the requests of that step only: they end with status ``failed``
  and their pages go back; the queue goes on (a failure is terminal for its own request only,
  src/Runtime/Runtime.jl:151-153, 175-178).  The status words travel back with the sampled ids, so
  reading them costs no wait of its own.

The scheduler needs of its engine only ``cache`` (a CacheManager), ``admit``, ``release``,
``step(entries) -> logits`` and a ``select(logits, requests) -> tokens`` function, so its decisions
are tested on the CPU with a stand-in engine.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..errors import ErrorCode, GessoError, invalid, resource
from ..sampling.sampler import SamplingParams, SplitMix64
from .batch import StepEntry

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
# finish statuses (the reference's BatchResult statuses, src/Runtime/Runtime.jl:46-51, plus "stop")
COMPLETE, EOS, STOP, CANCELLED, FAILED = "complete", "eos", "stop", "cancelled", "failed"


@dataclass(eq=False)      # a request is itself: membership tests must not compare prompts element by element
class Request:
    prompt: List[int]
    max_new_tokens: int = 8
    sampling: SamplingParams = field(default_factory=SamplingParams)
    eos_ids: Tuple[int, ...] = ()
    stop_ids: Tuple[int, ...] = ()
    on_token: Optional[Callable[[int], Optional[bool]]] = None
    req_id: Optional[object] = None
    # ---- scheduler state ----
    state: str = WAITING
    status: Optional[str] = None
    error: Optional[Exception] = None
    generated: List[int] = field(default_factory=list)
    fed: int = 0                      # tokens of prompt+generated that are in the cache
    pending: int = 0                  # tokens selected on the device for it that the host has not read yet
    preemptions: int = 0
    cancelled: bool = False
    rng: Optional[SplitMix64] = None
    admitted_at: int = -1

    def __post_init__(self):
        self.prompt = [int(t) for t in self.prompt]
        try:    # portions of the prompt are handed to the engine as views of this array (no list per step)
            self._prompt_arr = np.asarray(self.prompt, dtype=np.int64) if self.prompt else None
        except OverflowError:
            self._prompt_arr = None         # an id no machine integer holds: the step's check names it
        if self.max_new_tokens < 0:
            raise invalid("request: max_new_tokens must be >= 0")
        self.rng = SplitMix64(self.sampling.seed)

    @property
    def sequence(self) -> List[int]:
        return self.prompt + self.generated

    @property
    def length(self) -> int:
        return len(self.prompt) + len(self.generated)

    def tokens(self, start: int, n: int) -> List[int]:
        """``sequence[start:start+n]`` without building the sequence (it is asked for every step)."""
        p = len(self.prompt)
        if start >= p:
            return self.generated[start - p:start - p + n]
        if start + n <= p:
            return self.prompt[start:start + n] if self._prompt_arr is None or n < 8 else self._prompt_arr[start:start + n]
        return self.prompt[start:] + self.generated[:start + n - p]

    @property
    def ids(self) -> List[int]:
        """Prompt plus new ids, the stopping id included (src/Inference/session.jl:1025-1034)."""
        return self.prompt + self.generated

    def cancel(self) -> None:
        self.cancelled = True


_FAILED_STEP = object()      # what Scheduler._run returns for a step that raised
_UNREAD_TOKEN = (0,)         # stands in a step's entries for a token id that is still on the device
_FIRST_PLACE = (0,)


class _NeedSync(Exception):
    """Planning around tokens that are still on the device met a decision that needs them read first."""


@dataclass
class StepPlan:
    entries: List[Tuple[Request, int, int]]      # (request, first index into its sequence, n tokens)
    preempted: List[Request] = field(default_factory=list)
    admitted: List[Request] = field(default_factory=list)

    @property
    def n_tokens(self) -> int:
        return sum(n for _, _, n in self.entries)


class Scheduler:
    def __init__(self, engine, select: Callable, *, max_batch: int = 8, max_tokens_per_step: int = 2048,
                 prefill_chunk: int = 512, vocab_size: Optional[int] = None, pipeline: bool = True):
        if max_batch < 1 or max_tokens_per_step < 1 or prefill_chunk < 1:
            raise invalid("scheduler: max_batch, max_tokens_per_step and prefill_chunk must be >= 1")
        self.engine = engine
        self.cache = engine.cache
        self.select = select
        self.max_batch = max_batch
        self.max_tokens_per_step = max_tokens_per_step
        self.prefill_chunk = prefill_chunk
        self.vocab_size = vocab_size
        self.waiting: List[Request] = []
        self.running: List[Request] = []          # in admission order
        self._ids = itertools.count()
        self._clock = itertools.count()
        self.steps = 0
        self.preemptions = 0
        self._staged = None                       # the next decoding step, prepared while this one runs
        self._inflight = None                     # (requests, selection) of a step whose tokens are not read yet
        self.pipeline = pipeline
        self._planning_ahead = False              # plan() runs around tokens the host has not read yet
        self._ahead_requests: List[Request] = []
        self.steps_ahead = 0                      # steps launched before the step before them was digested

    # ---- adding --------------------------------------------------------------------------------
    def add(self, req: Request) -> Request:
        if req.req_id is None:
            req.req_id = f"req{next(self._ids)}"
        if not req.prompt:
            raise invalid("request: empty prompt")          # src/Inference/session.jl:688-689
        if self.vocab_size is not None:
            for t in req.prompt:
                if not (0 <= t < self.vocab_size):
                    raise invalid(f"request: token id {t} is outside the vocabulary")   # session.jl:164-177
        total = len(req.prompt) + req.max_new_tokens
        if len(req.prompt) > self.cache.max_positions:
            raise resource(f"request: prompt of {len(req.prompt)} tokens exceeds the context length "
                           f"{self.cache.max_positions}")     # session.jl:699-706
        # what the request holds at its longest: every token but the last sampled one is in the cache
        longest = min(max(len(req.prompt), total - 1), self.cache.max_positions)
        pages = (longest + self.cache.page_size - 1) // self.cache.page_size
        for pool, g in zip(self.cache.pools, self.cache.groups):
            if g.window is None and pages > pool.count:
                raise resource(f"request: needs {pages} pages of group {g.name}, the pool has {pool.count}")
        req.state = WAITING
        if req.max_new_tokens == 0:
            self._finish(req, COMPLETE)       # returns the prompt (test/test_reference_generate.jl:24-28)
            return req
        self.waiting.append(req)
        return req

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running or self._inflight is not None)

    # ---- planning (pure bookkeeping: no device work) ------------------------------------------------
    def _left(self, r: Request) -> int:
        return len(r.prompt) + len(r.generated) + r.pending - r.fed

    def _ending(self, r: Request) -> bool:
        """A token selected for it and not read yet is certainly its last (its count or the context is full):
        it takes no part in a step planned before that token is read."""
        return r.pending > 0 and (len(r.generated) + r.pending >= r.max_new_tokens
                                  or len(r.prompt) + len(r.generated) + r.pending > self.cache.max_positions)

    def _need(self, wants: Dict[object, Tuple[Request, int]]) -> List[int]:
        """Pages per group that the planned tokens still have to be handed."""
        need = [0] * len(self.cache.groups)
        for r, n in wants.values():
            for g, k in enumerate(self.cache.pages_needed(r.req_id, n)):
                need[g] += k
        return need

    def _short(self, need: List[int], extra: Optional[List[int]] = None, spare: int = 0) -> bool:
        free = self.cache.free_pages()
        if extra is None:
            return any(k + spare > f for k, f in zip(need, free))
        return any(k + e + spare > f for k, e, f in zip(need, extra, free))

    def plan(self) -> StepPlan:
        plan = StepPlan(entries=[])
        # cancelled requests leave before anything is planned
        for r in [r for r in self.running if r.cancelled]:
            self._finish(r, CANCELLED)
        for r in [r for r in self.waiting if r.cancelled]:
            self.waiting.remove(r)
            self._finish(r, CANCELLED)

        # steady decoding (nobody waits, everybody has exactly its last sampled token to run, and the
        # pools hold a page for everyone who crosses a page border): nothing to decide
        if not self.waiting and self.running and len(self.running) <= self.max_tokens_per_step \
                and all((r.generated or r.pending) and self._left(r) == 1 and not self._ending(r) for r in self.running):
            ps = self.cache.page_size
            at_border = sum(1 for r in self.running if self.cache.length(r.req_id) % ps == 0)
            free = self.cache.free_pages()
            if (not free or at_border <= min(free)) and \
                    all(self.cache.length(r.req_id) < self.cache.max_positions for r in self.running):
                plan.entries = [(r, r.fed, 1) for r in self.running]
                return plan

        budget = self.max_tokens_per_step
        wants: Dict[object, Tuple[Request, int]] = {}
        going = [r for r in self.running if not self._ending(r)]
        decoders = [r for r in going if self._left(r) == 1 and (r.generated or r.pending)]
        prefillers = [r for r in going if r not in decoders]
        # 1. every decoding request gets its one token; preempt from the newest while they do not fit
        for r in decoders:
            wants[r.req_id] = (r, 1)
        need = self._need(wants)                 # kept in step with `wants` from here on
        while self._short(need) and len(self.running) > 1:
            if self._planning_ahead:
                raise _NeedSync()                # a preemption: first read what the victim was given
            victim = self.running[-1]
            self._preempt(victim)
            plan.preempted.append(victim)
            wants.pop(victim.req_id, None)
            need = self._need(wants)
            if victim in prefillers:
                prefillers.remove(victim)
        if self._short(need):
            if self._planning_ahead:
                raise _NeedSync()
            # a single request is left and its next token has no page: it has outgrown the pool
            for r, _ in list(wants.values()):
                self._finish(r, FAILED, resource(f"request {r.req_id!r} does not fit the cache pool"))
            wants.clear()
            need = self._need(wants)
        budget -= len(wants)
        # 2. prompt portions of running requests, oldest first, shrunk to what the pool can hold
        for r in prefillers:
            if budget <= 0:
                break
            n = min(self._left(r), self.prefill_chunk, budget)
            n = self._fit(r, n, need)
            if n > 0:
                wants[r.req_id] = (r, n)
                budget -= n
        # 3. admissions, first come first served, only while nothing was preempted in this step
        while (self.waiting and not plan.preempted and budget > 0
               and len(self.running) < self.max_batch and self.cache.slots.free_count > 0):
            r = self.waiting[0]
            self.engine.admit(r.req_id)
            n = min(self._left(r), self.prefill_chunk, budget)
            # a newcomer leaves one spare page per running request, so that their next tokens fit
            n = self._fit(r, n, need, spare=len(self.running))
            if n <= 0:
                self.engine.release(r.req_id)      # no room for even one token now: stays queued
                break
            self.waiting.pop(0)
            r.state, r.admitted_at = RUNNING, next(self._clock)
            self.running.append(r)
            plan.admitted.append(r)
            wants[r.req_id] = (r, n)
            budget -= n
        if not wants and self.running:
            if self._planning_ahead:
                raise _NeedSync()
            # nothing fits although requests are live: the oldest alone must be able to move
            r = self.running[0]
            while len(self.running) > 1:
                victim = self.running[-1]
                self._preempt(victim)
                plan.preempted.append(victim)
            n = self._fit(r, min(self._left(r), self.prefill_chunk, self.max_tokens_per_step), [0] * len(self.cache.groups))
            if n <= 0:
                self._finish(r, FAILED, resource(f"request {r.req_id!r} does not fit the cache pool"))
            else:
                wants[r.req_id] = (r, n)
        for r in self.running:                      # admission order
            if r.req_id in wants:
                plan.entries.append((r, r.fed, wants[r.req_id][1]))
        return plan

    def _fit(self, r: Request, n: int, need: List[int], spare: int = 0) -> int:
        """Largest portion <= n of request r that the free pages hold beside what is planned (``need``: the
        pages the plan takes so far; the portion's own pages are added to it when it fits)."""
        n = min(n, self.cache.max_positions - self.cache.length(r.req_id))
        while n > 0:
            own = self.cache.pages_needed(r.req_id, n)
            if not self._short(need, own, spare):
                for g, k in enumerate(own):
                    need[g] += k
                return n
            # shrink to the last page border below n (or give up)
            filled = self.cache.length(r.req_id) + n
            border = ((filled - 1) // self.cache.page_size) * self.cache.page_size
            n = border - self.cache.length(r.req_id)
        return 0

    def _preempt(self, r: Request) -> None:
        self.engine.release(r.req_id)
        self.running.remove(r)
        r.state, r.fed = WAITING, 0
        r.preemptions += 1
        self.preemptions += 1
        self.waiting.insert(0, r)

    def _finish(self, r: Request, status: str, error: Optional[Exception] = None) -> None:
        if r.state == RUNNING:
            self.engine.release(r.req_id)
            self.running.remove(r)
        r.state, r.status, r.error = FINISHED, status, error

    # ---- running a step ---------------------------------------------------------------------------
    # ---- failures of a step ---------------------------------------------------------------------------
    def _fail(self, requests, error: Exception) -> None:
        if not isinstance(error, GessoError):
            error = GessoError(ErrorCode.RUNTIME, f"the step failed: {type(error).__name__}: {error}")
        for r in requests:
            if r.state == RUNNING:
                self._finish(r, FAILED, error)

    def _run(self, requests: List[Request], call):
        """Run one engine step; if it raises, its requests fail (and are released) and ``_FAILED_STEP``
        comes back."""
        try:
            return call()
        except Exception as e:      # not BaseException: an interrupt goes through
            self._fail(requests, e)
            self._staged = None
            return _FAILED_STEP

    def _status_launch(self):
        launch = getattr(self.engine, "status_read_launch", None)
        return None if launch is None else launch()

    def _status_finish(self, ticket) -> None:
        """What the kernels of the steps since the last read reported: their requests fail."""
        if ticket is None:
            return
        res = self.engine.status_read_finish(ticket)
        if res is not None:
            error, req_ids = res
            hit = set(req_ids)
            self._fail([r for r in self.running if r.req_id in hit], error)
            self._staged = None

    def _select_now(self, logits, requests: List[Request]) -> List[object]:
        ticket = self._status_launch()
        tokens = self.select(logits, requests)
        self._status_finish(ticket)
        return tokens

    def _select_launch(self, logits, requests: List[Request]):
        ticket = self._status_launch()          # before the ids' copy: it has landed when they have
        selection = self.select.launch(logits, requests)
        for r in requests:
            r.pending += 1                      # until _digest has read the token
        return selection, ticket

    def _select_wait(self, pending) -> List[object]:
        selection, ticket = pending
        tokens = self.select.wait(selection)
        self._status_finish(ticket)
        return tokens

    def _digest(self, requests: List[Request], tokens: List[object]) -> List[Tuple[Request, int]]:
        """Take the selected tokens in: append, call hooks, finish what has ended."""
        emitted: List[Tuple[Request, int]] = []
        for r, tok in zip(requests, tokens):
            if r.pending > 0:
                r.pending -= 1
            if r.state != RUNNING:
                continue                    # failed with its step: what was selected for it is dropped
            if isinstance(tok, Exception):
                self._finish(r, FAILED, tok)
                continue
            r.generated.append(int(tok))
            emitted.append((r, int(tok)))
            stop_by_hook = False
            if r.on_token is not None:
                try:
                    stop_by_hook = r.on_token(int(tok)) is False
                except Exception as e:      # a failing callback fails only its request
                    self._finish(r, FAILED, GessoError(ErrorCode.RUNTIME, f"on_token raised: {e!r}"))
                    continue
            if int(tok) in r.eos_ids:
                self._finish(r, EOS)
            elif int(tok) in r.stop_ids or stop_by_hook:
                self._finish(r, STOP)
            elif len(r.generated) >= r.max_new_tokens:
                self._finish(r, COMPLETE)
            elif len(r.prompt) + len(r.generated) > self.cache.max_positions:
                # the sampled token would not fit the context (src/Inference/session.jl:903-909)
                self._finish(r, COMPLETE)
        return emitted

    def _stage_next(self, requests: List[Request], pending_tokens: int) -> None:
        """While the device runs, prepare the decoding step after the ones in flight if it will most
        likely be the same requests with one more token each (``pending_tokens``: tokens per request that
        are selected but not digested yet); only the sampled ids are missing then."""
        self._staged = None
        stage = getattr(self.engine, "stage_single_tokens", None)
        if (stage is None or self.waiting or len(requests) != len(self.running)
                or any(r.state != RUNNING or r.cancelled
                       or len(r.generated) + pending_tokens + 1 > r.max_new_tokens for r in requests)):
            return
        try:
            self._staged = stage([r.req_id for r in requests])
        except GessoError:
            self._staged = None               # no page or no room: the ordinary path decides

    def step(self) -> List[Tuple[Request, int]]:
        """Plan, run and digest one step; returns the (request, token) pairs emitted by it.

        Steady decoding runs one step ahead of the host: the next step is launched with the token ids
        that the selection kernel left on the device, before the host has read them, so the device never
        waits for the host between two steps.  What a call returns is then the step before the one it
        launched.  A request that turns out to have ended is simply part of one step too many, whose
        result for it is dropped."""
        if self._inflight is not None:
            return self._advance()
        plan = self.plan()
        if not plan.entries:
            return []
        entries, samplers = [], []
        for r, start, n in plan.entries:      # (nothing is pending here: the step before has been digested)
            last = start + n == r.length
            entries.append(StepEntry(r.req_id, r.tokens(start, n), [n - 1] if last else []))
            if last:
                samplers.append(r)
        staged, self._staged = self._staged, None
        decoding = len(samplers) == len(entries) and all(n == 1 for _, _, n in plan.entries)
        step_requests = [r for r, _, _ in plan.entries]
        if staged is not None and decoding and staged.req_ids == tuple(e.req_id for e in entries):
            logits = self._run(step_requests, lambda: self.engine.step_staged(staged, [e.tokens[0] for e in entries]))
        else:
            logits = self._run(step_requests, lambda: self.engine.step(entries))
        self.steps += 1
        if logits is _FAILED_STEP:
            return []
        for r, _, n in plan.entries:
            r.fed += n
        if decoding:
            self._stage_next(samplers, pending_tokens=1)
        if not samplers:
            return []
        launch = getattr(self.select, "launch", None)
        if launch is not None and self.pipeline and (self._staged is not None or self._can_go_ahead()):
            # the selection is launched, not awaited: the next call takes it from there
            self._inflight = (samplers, self._select_launch(logits, samplers))
            return self._advance()
        return self._digest(samplers, self._select_now(logits, samplers))

    def _can_go_ahead(self) -> bool:
        """Any step, not only a steady decoding one, can be launched before the step before it is digested if
        the engine takes token ids that are still on the device."""
        return self.pipeline and getattr(self.engine, "accepts_device_tokens", False)

    def _launch_ahead(self, prev_requests: List[Request], prev_selection):
        """Plan and launch the step after the one in flight around the tokens that one is still selecting:
        the requests it selects for take part with a token id that is copied on the device; a request whose
        unread token is certainly its last sits the step out.  What the plan cannot decide without reading
        the tokens (a preemption, a request that has outgrown the pool) makes it give up: ``None``.
        Returns ``(samplers, selection or None)`` of the launched step."""
        self._planning_ahead = True
        try:
            plan = self.plan()
        except _NeedSync:
            return None
        finally:
            self._planning_ahead = False
        if not plan.entries:
            return None
        place = {id(r): i for i, r in enumerate(prev_requests)}
        unread, known = [], []
        for r, start, n in plan.entries:
            if start >= len(r.prompt) + len(r.generated):
                unread.append((place[id(r)], r, start, n))       # its token is the one being selected
            else:
                known.append((r, start, n))
        unread.sort(key=lambda x: x[0])                          # in the order of the selection's rows
        entries, samplers, runs, requests = [], [], [], []
        for k, (i, r, start, n) in enumerate(unread):
            entries.append(StepEntry(r.req_id, _UNREAD_TOKEN, _FIRST_PLACE))
            samplers.append(r)
            requests.append((r, n))
            if runs and runs[-1][0] + runs[-1][2] == i:
                runs[-1] = (runs[-1][0], runs[-1][1], runs[-1][2] + 1)
            else:
                runs.append((i, k, 1))
        for r, start, n in known:
            last = start + n == len(r.prompt) + len(r.generated) + r.pending
            entries.append(StepEntry(r.req_id, r.tokens(start, n), [n - 1] if last else []))
            requests.append((r, n))
            if last:
                samplers.append(r)
        self._ahead_requests = [r for r, _ in requests]          # whom a failure of this step concerns
        logits = self.engine.step(entries, device_tokens=(prev_selection.ids, runs) if runs else None)
        self.steps += 1
        self.steps_ahead += 1
        for r, n in requests:
            r.fed += n
        return samplers, (self._select_launch(logits, samplers) if samplers else None)

    def _advance(self) -> List[Tuple[Request, int]]:
        """One turn of the pipelined decoding: launch the step after the one in flight from the ids on the
        device, then wait for the one in flight and digest it."""
        requests, pending = self._inflight
        staged, self._staged = self._staged, None
        ahead = None
        ahead_error = None
        if (staged is not None and staged.req_ids == tuple(r.req_id for r in requests) and not self.waiting
                and not any(r.cancelled for r in requests)):
            try:
                logits = self.engine.step_staged(staged, device_tokens=pending[0].ids)
                self.steps += 1
                for r in requests:
                    r.fed += 1
                ahead = self._select_launch(logits, requests)
            except Exception as e:
                ahead_error = e                   # the step in flight is still good: digest it first
        elif self._can_go_ahead():
            # not a steady decoding step (somebody waits, prompts are being read, the batch changes): plan
            # around the unread tokens and launch; whoever turns out to have ended has run one step too many
            launched, failed_with = None, None
            self._ahead_requests = []
            try:
                launched = self._launch_ahead(requests, pending[0])
            except Exception as e:
                failed_with = e                   # the step in flight is still good: digest it first
            emitted = self._digest(requests, self._select_wait(pending))
            if failed_with is not None:
                self._fail(self._ahead_requests or list(self.running), failed_with)
                self._inflight = None
                return emitted
            if launched is None or launched[1] is None:
                self._inflight = None             # nothing launched, or a step that selects nothing
                return emitted
            samplers, selection = launched
            self._inflight = (samplers, selection)
            if all(r.state == RUNNING for r in samplers) and len(samplers) == len(self.running) and not self.waiting:
                self._stage_next(samplers, pending_tokens=1)     # steady decoding from here on
            return emitted
        emitted = self._digest(requests, self._select_wait(pending))
        if ahead_error is not None:
            self._fail(requests, ahead_error)
        if ahead is None:
            self._inflight = None                     # back to one step at a time
            return emitted
        if any(r.state != RUNNING or r.cancelled for r in requests) or self.waiting:
            # somebody ended (or arrived): the step ahead has run with the old batch; take what it
            # gives to the requests that go on, drop the rest
            tokens = self._select_wait(ahead)
            alive = [(r, t) for r, t in zip(requests, tokens) if r.state == RUNNING]
            emitted += self._digest([r for r, _ in alive], [t for _, t in alive])
            self._inflight = None
            return emitted
        self._inflight = (requests, ahead)
        self._stage_next(requests, pending_tokens=1)
        return emitted

    def drain(self) -> List[Tuple[Request, int]]:
        """Wait for a step that is still in flight and digest it (before the scheduler is left alone)."""
        if self._inflight is None:
            return []
        requests, pending = self._inflight
        self._inflight, self._staged = None, None
        return self._digest(requests, self._select_wait(pending))

    def run(self, max_steps: Optional[int] = None) -> None:
        n = 0
        while self.has_work:
            before = (len(self.waiting), len(self.running), self.steps)
            self.step()
            n += 1
            if max_steps is not None and n >= max_steps:
                break
            if (len(self.waiting), len(self.running), self.steps) == before and not self.running and self.waiting:
                # nothing ran and nothing is live: the head of the queue cannot be admitted
                r = self.waiting.pop(0)
                self._finish(r, FAILED, resource(f"request {r.req_id!r} cannot be admitted"))
