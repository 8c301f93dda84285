"""The scheduler's decisions on the CPU, with a stand-in engine around a real cache manager."""
import pytest

from gesso_b200.cache import CacheManager, PagedGroupSpec
from gesso_b200.engine.scheduler import (CANCELLED, COMPLETE, EOS, FAILED, STOP, Request, Scheduler)
from gesso_b200.errors import ErrorCode, GessoError
from gesso_b200.sampling import SamplingParams


class FakeEngine:
    """Keeps the cache manager honest and records every step; 'logits' are the entries themselves."""

    def __init__(self, num_pages=16, page_size=4, slots=4, ctx=64):
        self.cache = CacheManager([PagedGroupSpec("kv")], page_size, num_pages, slots, ctx)
        self.log = []

    def admit(self, rid):
        self.cache.admit(rid)

    def release(self, rid):
        self.cache.release(rid)

    def step(self, entries):
        for e in entries:
            self.cache.reserve(e.req_id, len(e.tokens))
        for e in entries:
            self.cache.commit(e.req_id, len(e.tokens))
        self.cache.check_invariants()
        self.log.append([(e.req_id, list(e.tokens), list(e.want)) for e in entries])
        return [e for e in entries if e.want]


def next_token(logits, requests):
    """Deterministic 'model': the next token is a function of the request's sequence so far."""
    return [(sum(r.sequence) * 31 + len(r.sequence)) % 97 for r in requests]


def make(engine=None, **kw):
    engine = engine or FakeEngine()
    return engine, Scheduler(engine, next_token, vocab_size=100, **kw)


def solo(prompt, n):
    eng, s = make()
    r = s.add(Request(prompt, n))
    s.run()
    return r.ids


def test_single_request_runs_to_completion_and_frees():
    eng, s = make(prefill_chunk=3)
    r = s.add(Request([1, 2, 3, 4, 5, 6, 7], 4))
    s.run()
    assert r.status == COMPLETE and len(r.generated) == 4
    # prompt in portions of 3, 3, 1; then one token per step; the last sampled token is never run
    assert [len(st[0][1]) for st in eng.log] == [3, 3, 1, 1, 1, 1]
    assert eng.log[0][0][2] == [] and eng.log[2][0][2] == [0]
    assert eng.cache.pages_in_use() == [0] and eng.cache.slots_in_use() == 0


def test_max_new_tokens_zero_returns_the_prompt():
    eng, s = make()
    r = s.add(Request([5, 6], 0))
    assert r.status == COMPLETE and r.ids == [5, 6] and not s.has_work and eng.log == []


def test_batched_equals_solo():
    prompts = [[1, 2, 3], [9] * 11, [4], [7, 8, 9, 10, 11, 12]]
    eng, s = make(max_batch=3, max_tokens_per_step=8, prefill_chunk=4)
    reqs = [s.add(Request(p, 5)) for p in prompts]
    s.run()
    for p, r in zip(prompts, reqs):
        assert r.status == COMPLETE and r.ids == solo(p, 5)
    assert max(len(st) for st in eng.log) <= 3
    assert all(sum(len(e[1]) for e in st) <= 8 for st in eng.log)          # the token budget
    # decoding requests come first in the budget: once a request decodes it is in every later step
    assert eng.cache.pages_in_use() == [0]


def test_decodes_before_portions_and_fifo():
    eng, s = make(max_batch=4, max_tokens_per_step=6, prefill_chunk=6)
    a = s.add(Request([1] * 4, 3))
    b = s.add(Request([2] * 9, 2))
    s.step()                                        # a: 4 tokens, b: 2 tokens (budget 6)
    assert eng.log[-1] == [("req0", [1] * 4, [3]), ("req1", [2] * 2, [])]
    s.step()                                        # a decodes (1), b gets the other 5
    assert [len(e[1]) for e in eng.log[-1]] == [1, 5]
    s.run()
    assert a.status == b.status == COMPLETE


def test_stops():
    # eos and stop ids end the request with the id returned but not run; the hook can stop too
    first = solo([3, 4], 1)[-1]
    eng, s = make()
    r = s.add(Request([3, 4], 5, eos_ids=(first,)))
    s.run()
    assert r.status == EOS and r.ids == [3, 4, first] and len(eng.log) == 1
    eng, s = make()
    r = s.add(Request([3, 4], 5, stop_ids=(first,)))
    s.run()
    assert r.status == STOP and r.ids == [3, 4, first]
    seen = []
    eng, s = make()
    r = s.add(Request([3, 4], 5, on_token=lambda t: (seen.append(t), len(seen) < 2)[1]))
    s.run()
    assert r.status == STOP and seen == r.generated and len(seen) == 2


def test_callback_failure_is_contained():
    def boom(t):
        raise ValueError("no")
    eng, s = make()
    bad = s.add(Request([1, 2], 4, on_token=boom))
    good = s.add(Request([5, 6, 7], 4))
    s.run()
    assert bad.status == FAILED and bad.error.code == ErrorCode.RUNTIME
    assert good.status == COMPLETE and good.ids == solo([5, 6, 7], 4)
    assert eng.cache.pages_in_use() == [0] and eng.cache.slots_in_use() == 0


def test_cancel():
    eng, s = make()
    a = s.add(Request([1, 2, 3], 50))
    b = s.add(Request([4, 5], 3))
    c = s.add(Request([6], 3))
    c.cancel()                                      # before it is admitted
    s.step()
    s.step()
    a.cancel()                                      # between tokens
    s.run()
    assert a.status == CANCELLED and 1 <= len(a.generated) < 50
    assert c.status == CANCELLED and c.generated == []
    assert b.status == COMPLETE and b.ids == solo([4, 5], 3)
    assert eng.cache.pages_in_use() == [0]


def test_refusals_at_add():
    eng, s = make(FakeEngine(num_pages=4, ctx=32))
    with pytest.raises(GessoError):
        s.add(Request([], 3))                       # empty prompt
    with pytest.raises(GessoError):
        s.add(Request([1, 200], 3))                 # outside the vocabulary
    with pytest.raises(GessoError) as e:
        s.add(Request([1] * 33, 1))                 # longer than the context
    assert e.value.code == ErrorCode.RESOURCE_LIMIT
    with pytest.raises(GessoError) as e:
        s.add(Request([1] * 10, 20))                # 29 cached tokens need 8 pages, the pool has 4
    assert e.value.code == ErrorCode.RESOURCE_LIMIT
    with pytest.raises(GessoError):
        Request([1], -1)


def test_context_limit_ends_generation():
    eng, s = make(FakeEngine(num_pages=16, ctx=8))
    r = s.add(Request([1] * 6, 50))
    s.run()
    assert r.status == COMPLETE and len(r.prompt) + len(r.generated) == 9     # 8 cached + the last sampled id
    assert eng.cache.pages_in_use() == [0]


def test_pages_run_out_preempts_newest_and_results_do_not_change():
    # 6 pages of 4 positions; three requests that together outgrow them
    prompts = [[1] * 6, [2] * 6, [3] * 5]
    eng = FakeEngine(num_pages=6, page_size=4, slots=4, ctx=24)
    _, s = make(eng, max_batch=3, prefill_chunk=8)
    reqs = [s.add(Request(p, 12)) for p in prompts]
    s.run()
    assert s.preemptions >= 1
    assert reqs[0].preemptions == 0                 # the oldest request is never preempted
    for p, r in zip(prompts, reqs):
        assert r.status == COMPLETE and r.ids == solo(p, 12)
    assert eng.cache.pages_in_use() == [0] and eng.cache.slots_in_use() == 0
    # a preempted request was prefilled again from its first token
    rid = next(r.req_id for r in reqs if r.preemptions)
    starts = [e for st in eng.log for e in st if e[0] == rid and len(e[1]) > 1]
    assert len(starts) >= 2


def test_admission_waits_for_slots_and_pages():
    eng = FakeEngine(num_pages=16, slots=2)
    _, s = make(eng, max_batch=8)
    reqs = [s.add(Request([i + 1] * 3, 2)) for i in range(5)]
    s.step()
    assert len(s.running) == 2 and len(s.waiting) == 3     # two slots
    s.run()
    assert all(r.status == COMPLETE for r in reqs)
    order = []
    for st in eng.log:
        for e in st:
            if e[0] not in order:
                order.append(e[0])
    assert order == [r.req_id for r in reqs]                # first come, first served


def test_sampling_params_validation():
    for bad in (dict(temperature=-1), dict(top_p=0), dict(top_p=1.5), dict(seed=-1)):
        with pytest.raises(GessoError):
            SamplingParams(**bad)
    assert SamplingParams().greedy and not SamplingParams(temperature=0.7).greedy


# ---- staged decoding steps: the next step is prepared while the device runs this one -----------------
class StagingEngine(FakeEngine):
    """A stand-in with the engine's staging interface: reserves at staging time, commits at run time."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.staged_made = self.staged_run = 0

    def stage_single_tokens(self, req_ids):
        self.cache.reserve_single_tokens(list(req_ids))
        self.staged_made += 1

        class Staged:
            pass
        st = Staged()
        st.req_ids = tuple(req_ids)
        return st

    def step_staged(self, staged, tokens):
        from gesso_b200.engine.batch import StepEntry
        self.staged_run += 1
        for rid in staged.req_ids:
            self.cache.commit(rid, 1)
        self.cache.check_invariants()
        entries = [StepEntry(rid, [int(t)], [0]) for rid, t in zip(staged.req_ids, tokens)]
        self.log.append([(e.req_id, list(e.tokens), list(e.want)) for e in entries])
        return entries


def test_staged_steps_give_the_same_tokens_and_are_used():
    prompts = [[1, 2, 3], [9] * 11, [4]]
    eng = StagingEngine()
    s = Scheduler(eng, next_token, vocab_size=100, max_batch=3, prefill_chunk=4)
    reqs = [s.add(Request(p, n)) for p, n in zip(prompts, (9, 5, 7))]
    s.run()
    for p, r, n in zip(prompts, reqs, (9, 5, 7)):
        assert r.status == COMPLETE and r.ids == solo(p, n)
    assert eng.staged_run > 0
    assert eng.cache.pages_in_use() == [0] and eng.cache.slots_in_use() == 0


def test_staged_step_is_dropped_when_the_batch_changes():
    eng = StagingEngine()
    s = Scheduler(eng, next_token, vocab_size=100, max_batch=3, prefill_chunk=8)
    a = s.add(Request([1, 2, 3], 12))
    for _ in range(3):
        s.step()
    assert s._staged is not None                    # a alone, decoding: its next step is staged
    made = eng.staged_made
    b = s.add(Request([5, 6, 7, 8], 6))             # a newcomer: the staged step no longer fits
    s.step()
    assert eng.staged_made == made and s._staged is None
    assert [e[0] for e in eng.log[-1]] == [a.req_id, b.req_id]
    s.run()
    assert a.ids == solo([1, 2, 3], 12) and b.ids == solo([5, 6, 7, 8], 6)
    assert eng.cache.pages_in_use() == [0]


def test_staging_yields_to_page_pressure():
    # a pool so small that staging one step ahead finds no page: the ordinary path decides, as before
    eng = StagingEngine(num_pages=3, page_size=4, slots=2, ctx=12)
    s = Scheduler(eng, next_token, vocab_size=100, max_batch=2, prefill_chunk=8)
    a = s.add(Request([1, 2, 3], 9))
    b = s.add(Request([4, 5, 6], 3))
    s.run()
    assert a.status == COMPLETE and b.status == COMPLETE
    assert a.ids == solo([1, 2, 3], 9) and b.ids == solo([4, 5, 6], 3)
    assert eng.cache.pages_in_use() == [0]


# ---- steady decoding one step ahead of the host ---------------------------------------------------------
class PipelinedEngine(FakeEngine):
    """A stand-in that keeps every request's history itself (as a cache would), so that a step can be
    launched from ids the host has not seen: 'logits' are the histories after the step."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.history = {}
        self.from_device = 0

    def admit(self, rid):
        super().admit(rid)
        self.history[rid] = []

    def release(self, rid):
        super().release(rid)
        self.history.pop(rid, None)

    def step(self, entries):
        super().step(entries)
        for e in entries:
            self.history[e.req_id] += [int(t) for t in e.tokens]
        return [list(self.history[e.req_id]) for e in entries if e.want]

    def stage_single_tokens(self, req_ids):
        self.cache.reserve_single_tokens(list(req_ids))

        class Staged:
            pass
        st = Staged()
        st.req_ids = tuple(req_ids)
        return st

    def step_staged(self, staged, tokens=None, device_tokens=None):
        if device_tokens is not None:
            tokens, self.from_device = device_tokens, self.from_device + 1
        for rid, t in zip(staged.req_ids, tokens):
            self.history[rid].append(int(t))
        self.cache.commit_single_tokens(list(staged.req_ids))
        self.cache.check_invariants()
        self.log.append([(rid, [int(t)], [0]) for rid, t in zip(staged.req_ids, tokens)])
        return [list(self.history[rid]) for rid in staged.req_ids]


class HistorySelect:
    """next token = a function of the whole history, as `next_token` computes it from a request."""

    @staticmethod
    def pick(history):
        return (sum(history) * 31 + len(history)) % 97

    def __call__(self, logits, requests):
        return [self.pick(h) for h in logits]

    def launch(self, logits, requests):
        class Pending:
            pass
        p = Pending()
        p.ids = [self.pick(h) for h in logits]
        return p

    def wait(self, pending):
        return list(pending.ids)


def test_pipelined_decoding_gives_the_same_tokens():
    prompts, news = [[1, 2, 3], [9] * 11, [4]], (12, 7, 9)
    eng = PipelinedEngine()
    s = Scheduler(eng, HistorySelect(), vocab_size=100, max_batch=3, prefill_chunk=4)
    reqs = [s.add(Request(p, n)) for p, n in zip(prompts, news)]
    s.run()
    for p, r, n in zip(prompts, reqs, news):
        assert r.status == COMPLETE and r.ids == solo(p, n)
    assert eng.from_device > 5                       # steps were launched from ids the host had not read
    assert eng.cache.pages_in_use() == [0] and eng.cache.slots_in_use() == 0 and not s.has_work


def test_pipelined_decoding_drops_the_step_too_many():
    """A request ends on a stop id while the next step is already running with it; the others go on."""
    eng = PipelinedEngine()
    s = Scheduler(eng, HistorySelect(), vocab_size=100, max_batch=2)
    full_a, full_b = solo([5, 6, 7], 14), solo([8, 1], 14)
    a = s.add(Request([5, 6, 7], 14, stop_ids=[full_a[3 + 6]]))       # its 7th new token stops it
    b = s.add(Request([8, 1], 14))
    late = None
    for i in range(40):
        if not s.has_work:
            break
        s.step()
        if i == 9:
            late = s.add(Request([3, 3, 3, 3], 5))                   # an arrival in the middle of the pipeline
    assert a.status == STOP and a.ids == full_a[:3 + 7]
    assert b.status == COMPLETE and b.ids == full_b
    assert late.status == COMPLETE and late.ids == solo([3, 3, 3, 3], 5)
    assert eng.from_device > 0 and eng.cache.pages_in_use() == [0]


def test_pipelined_decoding_with_cancel_and_hooks():
    eng = PipelinedEngine()
    s = Scheduler(eng, HistorySelect(), vocab_size=100, max_batch=2)
    seen = []
    a = s.add(Request([5, 6, 7], 20, on_token=lambda t: (seen.append(t), len(seen) < 5)[1]))
    b = s.add(Request([2, 2], 20))
    for i in range(60):
        if not s.has_work:
            break
        s.step()
        if i == 8:
            b.cancel()
    assert a.status == STOP and a.ids == solo([5, 6, 7], 20)[:3 + 5] and len(seen) == 5
    assert b.status == CANCELLED and b.ids == solo([2, 2], 20)[:len(b.ids)]
    assert eng.cache.pages_in_use() == [0] and not s.has_work


# ---- any step one step ahead of the host (prompt portions, arrivals, a batch that changes) ------------------
class AheadEngine(PipelinedEngine):
    """Takes token ids that are 'still on the device' in any step: ``device_tokens = (ids, runs)``."""

    accepts_device_tokens = True

    def __init__(self, raise_at=(), **kw):
        super().__init__(**kw)
        self.raise_at, self.n, self.ahead_steps = set(raise_at), 0, 0

    def step(self, entries, device_tokens=None):
        k, self.n = self.n, self.n + 1
        if k in self.raise_at:
            raise GessoError(ErrorCode.LAUNCH, f"step {k}: a kernel refused its sizes")
        if device_tokens is not None:
            ids, runs = device_tokens
            flat = [t for e in entries for t in e.tokens]
            for src, dst, n in runs:
                flat[dst:dst + n] = ids[src:src + n]
            filled, cur = [], 0
            for e in entries:
                filled.append(type(e)(e.req_id, flat[cur:cur + len(e.tokens)], e.want))
                cur += len(e.tokens)
            entries = filled
            self.ahead_steps += 1
        return super().step(entries)


def ahead(**kw):
    eng = AheadEngine(**{k: kw.pop(k) for k in ("raise_at", "num_pages", "page_size", "slots", "ctx") if k in kw})
    return eng, Scheduler(eng, HistorySelect(), vocab_size=100, **kw)


def test_steps_with_prompt_portions_run_ahead_and_give_the_same_tokens():
    prompts = [[1, 2, 3], [9] * 11, [4], [7, 8, 9, 10, 11, 12], [5] * 7, [6, 1]]
    news = (5, 9, 1, 4, 2, 7)
    eng, s = ahead(max_batch=3, max_tokens_per_step=8, prefill_chunk=4)
    reqs = [s.add(Request(p, n)) for p, n in zip(prompts, news)]
    s.run()
    for p, r, n in zip(prompts, reqs, news):
        assert r.status == COMPLETE and r.ids == solo(p, n), (p, r.ids)
    assert s.steps_ahead > 5 and eng.ahead_steps > 5        # steps planned around tokens the host had not read
    assert all(sum(len(e[1]) for e in st) <= 8 for st in eng.log)          # the token budget holds
    assert eng.cache.pages_in_use() == [0] and eng.cache.slots_in_use() == 0 and not s.has_work
    # a request whose unread token is certainly its last sits the next step out: no request was ever run
    # on a token beyond its count
    fed = {}
    for st in eng.log:
        for rid, toks, _ in st:
            fed[rid] = fed.get(rid, 0) + len(toks)
    for r in reqs:
        assert fed[r.req_id] == len(r.prompt) + len(r.generated) - 1


def test_running_ahead_drops_the_step_too_many_and_takes_arrivals():
    full_a, full_b = solo([5, 6, 7], 14), solo([8, 1] * 5, 14)
    eng, s = ahead(max_batch=3, prefill_chunk=3)
    a = s.add(Request([5, 6, 7], 14, stop_ids=[full_a[3 + 6]]))       # its 7th new token stops it
    b = s.add(Request([8, 1] * 5, 14))
    seen = []
    c = s.add(Request([2, 2, 2, 2, 2], 20, on_token=lambda t: (seen.append(t), len(seen) < 4)[1]))
    late = None
    for i in range(80):
        if not s.has_work:
            break
        s.step()
        if i == 6:
            late = s.add(Request([3, 3, 3, 3], 5))
    assert a.status == STOP and a.ids == full_a[:3 + 7]
    assert b.status == COMPLETE and b.ids == full_b
    assert c.status == STOP and c.ids == solo([2, 2, 2, 2, 2], 20)[:5 + 4]
    assert late.status == COMPLETE and late.ids == solo([3, 3, 3, 3], 5)
    assert s.steps_ahead > 0 and eng.cache.pages_in_use() == [0] and not s.has_work


def test_running_ahead_yields_where_a_preemption_is_needed():
    """Pages run out: a plan made around unread tokens gives up, the tokens are read, the newest request is
    preempted as ever, and nobody's tokens change."""
    prompts = [[1] * 6, [2] * 6, [3] * 6]
    eng, s = ahead(num_pages=7, page_size=4, slots=3, ctx=40, max_batch=3, prefill_chunk=8)
    reqs = [s.add(Request(p, 10)) for p in prompts]
    s.run()
    for p, r in zip(prompts, reqs):
        assert r.status == COMPLETE and r.ids == solo(p, 10)
    assert s.preemptions > 0 and eng.cache.pages_in_use() == [0]


def test_a_step_launched_ahead_that_raises_fails_its_requests_only():
    prompts = [[1, 2, 3], [4, 5], [6, 7, 8, 9], [10]]
    eng, s = ahead(raise_at={2}, max_batch=2)
    reqs = [s.add(Request(p, 4)) for p in prompts]
    s.run()
    failed = [r for r in reqs if r.status == FAILED]
    done = [r for r in reqs if r.status == COMPLETE]
    assert failed and done and len(failed) + len(done) == 4
    for r in failed:
        assert r.error.code == ErrorCode.LAUNCH
        assert r.ids == solo(r.prompt, 4)[:len(r.ids)]          # what was read before the failure stands
    for r in done:
        assert r.ids == solo(r.prompt, 4)
    assert eng.cache.pages_in_use() == [0] and eng.cache.slots_in_use() == 0


# ---- a step that fails is terminal for its own requests only (src/Runtime/Runtime.jl:151-153, 175-178) ----
class FailingEngine(FakeEngine):
    """Raises in the steps whose numbers are in ``raise_at``; reports a bad status word after the steps in
    ``bad_status_at`` (through the same two calls the real engine offers)."""

    def __init__(self, raise_at=(), bad_status_at=(), **kw):
        super().__init__(**kw)
        self.raise_at, self.bad_status_at = set(raise_at), set(bad_status_at)
        self.n = 0
        self.unchecked = set()
        self.bad = False

    def step(self, entries):
        k = self.n
        self.n += 1
        if k in self.raise_at:
            raise GessoError(ErrorCode.LAUNCH, f"step {k}: a kernel refused its sizes")
        out = super().step(entries)
        self.unchecked.update(e.req_id for e in entries)
        if k in self.bad_status_at:
            self.bad = True
        return out

    def status_read_launch(self):
        ticket = (self.bad, self.unchecked)
        self.bad, self.unchecked = False, set()
        return ticket

    def status_read_finish(self, ticket):
        bad, covered = ticket
        if not bad:
            return None
        return GessoError(ErrorCode.RUNTIME, "a kernel reported an invalid result"), \
            [rid for rid in covered if self.cache.is_live(rid)]


def test_a_step_that_raises_fails_its_requests_and_the_queue_goes_on():
    prompts = [[1, 2, 3], [4, 5], [6, 7, 8, 9], [10]]
    # two live at a time; step 1 is the first decoding step of the first two requests
    eng, s = make(FailingEngine(raise_at={1}), max_batch=2)
    reqs = [s.add(Request(p, 4)) for p in prompts]
    s.run()
    assert [r.status for r in reqs] == [FAILED, FAILED, COMPLETE, COMPLETE]
    for r in reqs[:2]:
        assert isinstance(r.error, GessoError) and r.error.code == ErrorCode.LAUNCH and "step 1" in str(r.error)
        assert len(r.generated) == 1              # what it had been given before the step failed stays
    for p, r in zip(prompts[2:], reqs[2:]):
        assert r.ids == solo(p, 4)
    assert eng.cache.pages_in_use() == [0] and eng.cache.slots_in_use() == 0
    eng.cache.check_invariants()
    assert not s.has_work


def test_a_foreign_exception_in_a_step_is_wrapped_and_contained():
    class Boom(FailingEngine):
        def step(self, entries):
            if self.n == 0:
                self.n += 1
                raise RuntimeError("CUDA out of memory")
            return super().step(entries)
    eng, s = make(Boom(), max_batch=1)
    a, b = s.add(Request([1, 2], 3)), s.add(Request([3], 3))
    s.run()
    assert a.status == FAILED and a.error.code == ErrorCode.RUNTIME and "out of memory" in str(a.error)
    assert b.status == COMPLETE and b.ids == solo([3], 3)
    assert eng.cache.pages_in_use() == [0]


def test_a_bad_status_word_fails_the_requests_of_the_steps_it_covers():
    # step 0: the prompts of r0 and r1 (both sample); the status read with their ids is bad
    eng, s = make(FailingEngine(bad_status_at={0}), max_batch=2)
    reqs = [s.add(Request(p, 3)) for p in ([1, 2, 3], [4, 5], [6])]
    s.run()
    assert [r.status for r in reqs] == [FAILED, FAILED, COMPLETE]
    assert all(r.error.code == ErrorCode.RUNTIME and r.generated == [] for r in reqs[:2])    # the ids were dropped
    assert reqs[2].ids == solo([6], 3)
    assert eng.cache.pages_in_use() == [0] and eng.cache.slots_in_use() == 0


def test_a_bad_status_of_a_step_without_samples_is_seen_at_the_next_read():
    # prompt of 9 in portions of 4: steps 0 and 1 sample nothing, so nothing is read; the word set in step 0
    # is seen with the ids of step 2 and fails the request then
    eng, s = make(FailingEngine(bad_status_at={0}), prefill_chunk=4, max_batch=1)
    a, b = s.add(Request(list(range(9)), 2)), s.add(Request([7], 2))
    s.run()
    assert a.status == FAILED and a.generated == [] and len(eng.log) >= 3
    assert b.status == COMPLETE and b.ids == solo([7], 2)
