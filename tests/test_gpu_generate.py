"""Generation through the Python entry point and the command line, long decoding, the first tokens of
a sequence, and weights made so that cache faults would show."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import configs

pytestmark = pytest.mark.gpu

TOL32 = 1e-4
TOL16 = 32 * 2.0 ** -9


@pytest.fixture(scope="module")
def models(model_dirs):
    import gesso_b200
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            cache[(name, dtype)] = gesso_b200.load(model_dirs[name], dtype=dtype, max_positions=512)
        return cache[(name, dtype)]
    return get


def prompts_for(name, lengths, seed=0):
    vocab = configs.TINY[name][0]["vocab_size"]
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


# ---- greedy generation ---------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_greedy_generate_equals_plain_float32(name, models, plain_models):
    import gesso_b200
    model = models(name, "float32")
    s = gesso_b200.Session(model, context_length=128, page_size=16, max_batch=4)
    for p in prompts_for(name, [7, 13, 1, 30]):
        got = s.generate(p, max_new_tokens=8)
        assert got == plain_models[name].greedy(p, 8)
        assert got[:len(p)] == p and len(got) == len(p) + 8
    assert s.generate([3, 4], max_new_tokens=0) == [3, 4]          # test/test_reference_generate.jl:24-28
    assert s.engine.cache.pages_in_use() == [0] and s.engine.cache.slots_in_use() == 0


def near_max(plain, ids, n_prompt, tol):
    """Every generated id is a maximum of the plain logits up to the tolerance of the run type."""
    lg = plain.logits(ids[:-1])
    for k in range(n_prompt, len(ids)):
        row = lg[k - 1]
        assert float(row.max() - row[ids[k]]) <= tol * max(1.0, float(row.abs().max())), (k, ids[k])


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_greedy_generate_bfloat16(name, models, plain_models):
    import gesso_b200
    s = gesso_b200.Session(models(name, "bfloat16"), context_length=128, max_batch=4)
    for p in prompts_for(name, [7, 40, 1]):
        ids = s.generate(p, max_new_tokens=12)
        near_max(plain_models[name], ids, len(p), TOL16)


def test_batch_equals_solo_and_is_deterministic(models, plain_models):
    """Continuous batching with chunked prefill does not change anybody's tokens (greedy and sampled)."""
    import gesso_b200
    model = models("b", "float32")
    prompts = prompts_for("b", [40, 1, 23, 5, 17], seed=3)
    s = gesso_b200.Session(model, context_length=128, max_batch=3, max_tokens_per_step=24, prefill_chunk=8)
    reqs = [gesso_b200.BatchRequest(p, max_new_tokens=9, temperature=0.7 if i % 2 else 0.0, top_p=0.9, seed=1 + i)
            for i, p in enumerate(prompts)]
    res = s.run_batch(reqs)
    assert [r.status for r in res] == ["complete"] * 5
    # steps with prompt portions were planned and launched around tokens the host had not read yet
    assert s.stats()["steps_ahead"] >= 5
    solo = gesso_b200.Session(model, context_length=128, max_batch=1)
    for i, (p, r) in enumerate(zip(prompts, res)):
        assert r.ids == solo.generate(p, 9, temperature=0.7 if i % 2 else 0.0, top_p=0.9, seed=1 + i)
        if i % 2 == 0:
            assert r.ids == plain_models["b"].greedy(p, 9)
    assert [r.ids for r in s.run_batch(reqs)] == [r.ids for r in res]        # same seeds, same ids
    assert s.stats()["pages_in_use"] == [0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_steps_staged_ahead_keep_the_tokens(dtype, models, plain_models):
    """Decoding steps are prepared one ahead while the device runs; requests of different lengths end
    at different steps (a staged step is dropped then), pages are crossed, and nobody's ids change."""
    import gesso_b200
    model = models("c", dtype)
    prompts = prompts_for("c", [14, 3, 31], seed=11)
    news = [40, 9, 22]
    s = gesso_b200.Session(model, context_length=128, page_size=16, max_batch=3)
    res = s.run_batch([gesso_b200.BatchRequest(p, max_new_tokens=n) for p, n in zip(prompts, news)])
    assert s.stats()["staged_steps"] >= 20
    solo = gesso_b200.Session(model, context_length=128, page_size=16, max_batch=1)
    for p, n, r in zip(prompts, news, res):
        assert r.status == "complete"
        if dtype == "float32":
            assert r.ids == plain_models["c"].greedy(p, n)
            assert r.ids == solo.generate(p, n)
        else:
            near_max(plain_models["c"], r.ids, len(p), TOL16)
    assert s.stats()["pages_in_use"] == [0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_repeated_portion_shapes_replay_a_graph(dtype, models):
    """Prompt portions of a length that has come before run as a captured graph: three requests with
    prompts of one length (a chunked prompt's full portions) give, position by position, the logits of
    an engine that launches every kernel itself."""
    from gesso_b200.engine import Engine, StepEntry
    model = models("c", dtype)
    prompts = prompts_for("c", [96, 96, 96, 96], seed=21)
    outs = {}
    for graphs in (False, True):
        eng = Engine(model, max_positions=256, page_size=16, num_pages=40, max_requests=2, use_graphs=graphs)
        res = []
        for i, p in enumerate(prompts):
            eng.admit(i)
            res.append(eng.step([StepEntry(i, p, [0, 95])]).clone())
            res.append(eng.step([StepEntry(i, p[:70], [69])]).clone())       # a second portion shape, positions 96..
            eng.release(i)
        outs[graphs] = res
        eng.check_status()
        if graphs:
            assert sum(1 for k in eng._graphs if k[0] > k[1]) == 2            # both shapes were captured
    for a, b in zip(outs[False], outs[True]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype,tol", [("float32", TOL32), ("bfloat16", TOL16)])
def test_mixed_steps_in_padded_shapes_replay_graphs(dtype, tol, models, plain_models):
    """Mixed steps whose padded shape has come before are filled up with stand-in requests (scratch slot,
    scratch page) and replay a graph: portions of changing length beside a changing number of single
    tokens, requests that end and others that take over their pages; every wanted row against the plain
    implementation, and the same rows as an engine that launches every kernel itself."""
    from gesso_b200.engine import Engine, StepEntry
    model = models("c", dtype)
    plain = plain_models["c"]
    seqs = prompts_for("c", [150, 90, 61, 33, 120], seed=31)
    want_rows = {i: plain.logits(seq, list(range(len(seq)))).numpy() for i, seq in enumerate(seqs)}

    def run(graphs):
        eng = Engine(model, max_positions=256, page_size=16, num_pages=30, max_requests=4, use_graphs=graphs)
        fed = {i: 0 for i in range(len(seqs))}
        got = []
        for i in (0, 1, 2):
            eng.admit(i)
        live, waiting = [0, 1, 2], [3, 4]
        portion_of, sizes, turn = 0, [17, 5, 30, 2, 9, 23, 3, 12], 0
        while live:
            entries, places = [], []
            # one request feeds a portion, the others one token each
            if portion_of not in live:
                portion_of = live[0]
            for i in live:
                n = min(sizes[turn % len(sizes)] if i == portion_of else 1, len(seqs[i]) - fed[i])
                entries.append(StepEntry(i, seqs[i][fed[i]:fed[i] + n], [n - 1]))
                places.append((i, fed[i] + n - 1))
                fed[i] += n
            turn += 1
            portion_of = live[(live.index(portion_of) + 1) % len(live)]
            logits = eng.step(entries)
            got.append((places, logits.clone()))
            for i in [i for i in live if fed[i] == len(seqs[i])]:
                eng.release(i)
                live.remove(i)
                if waiting:
                    j = waiting.pop(0)
                    eng.admit(j)
                    live.append(j)
        eng.check_status()
        return eng, got

    eng, got = run(True)
    assert eng.stats()["padded_steps"] >= 10
    for places, logits in got:
        for row, (i, pos) in enumerate(places):
            ref = want_rows[i][pos]
            err = float(np.abs(logits[row].cpu().numpy().astype(np.float64) - ref).max())
            assert err <= tol * max(1.0, float(np.abs(ref).max())), (i, pos, err)
    _, plain_run = run(False)
    for (pa, la), (pb, lb) in zip(got, plain_run):
        assert pa == pb
        # the stand-ins change the shapes some kernels are chosen by, not what a row is made of
        assert float((la - lb).abs().max()) <= tol * max(1.0, float(lb.abs().max()))
    assert eng.stats()["pages_in_use"] == [0]


@pytest.mark.parametrize("dtype,tol", [("float32", TOL32), ("bfloat16", TOL16)])
def test_mixed_steps_of_an_engine_with_a_short_context_stay_unpadded(dtype, tol, models, plain_models):
    """The stand-in portion of a padded step sits at positions 0 .. up to 63 of a block table and of the
    rotary table.  An engine whose context is shorter than that (32 positions, two pages a request) has
    neither: its mixed steps must run as they are, and the repeated shapes below must not reach beyond a
    block-table row or the table of angles (a page id read from there once sent K and V of the stand-in
    into a live request's page)."""
    from gesso_b200.engine import Engine, StepEntry
    model = models("c", dtype)
    plain = plain_models["c"]
    seqs = prompts_for("c", [32, 30, 31], seed=77)
    ref = [plain.logits(seq).numpy() for seq in seqs]
    eng = Engine(model, max_positions=32, page_size=16, num_pages=6, max_requests=3)
    for i in range(3):
        eng.admit(i)
    fed = [0, 0, 0]
    for turn in range(40):
        live = [i for i in range(3) if fed[i] < len(seqs[i])]
        if not live:
            break
        entries, places = [], []
        for i in live:          # the same two shapes over and over: 5 + 1 + 1 tokens, then 1 + 5 + 1, ...
            n = min(5 if i == live[turn % len(live)] else 1, len(seqs[i]) - fed[i])
            entries.append(StepEntry(i, seqs[i][fed[i]:fed[i] + n], [n - 1]))
            places.append((i, fed[i] + n - 1))
            fed[i] += n
        logits = eng.step(entries).cpu().numpy().astype(np.float64)
        for row, (i, pos) in enumerate(places):
            err = float(np.abs(logits[row] - ref[i][pos]).max())
            assert err <= tol * max(1.0, float(np.abs(ref[i][pos]).max())), (turn, i, pos, err)
    eng.check_status()
    assert fed == [32, 30, 31] and eng.stats()["padded_steps"] == 0
    for i in range(3):
        eng.release(i)
    eng.cache.check_invariants()


def test_sampled_ids_follow_the_plain_sampler(models, plain_models):
    import gesso_b200
    from plain_lfm2 import PlainSampler
    model = models("a", "float32")
    s = gesso_b200.Session(model, context_length=64, max_batch=1)
    p = prompts_for("a", [9], seed=5)[0]
    got = s.generate(p, 6, temperature=0.8, top_p=0.95, seed=42)
    sampler, ids = PlainSampler(0.8, 0.95, 42), list(p)
    for _ in range(6):
        ids.append(sampler.sample(plain_models["a"].logits(ids)[-1].tolist()))
    assert got == ids


def test_stops_hooks_and_failures(models):
    import gesso_b200
    model = models("a", "float32")
    s = gesso_b200.Session(model, context_length=64, max_batch=4)
    p = [5, 6, 7]
    full = s.generate(p, 6)
    assert s.generate(p, 6, stop_ids=[full[4]]) == full[:5]                 # the stopping id is returned
    assert s.generate(p, 6, eos_ids=[full[3]]) == full[:4]
    seen = []
    assert s.generate(p, 6, on_token=lambda t: (seen.append(t), len(seen) < 3)[1]) == full[:6]
    assert seen == full[3:6]                                                # test/test_generate_hooks.jl:41-81

    def boom(t):
        raise RuntimeError("hook")
    res = s.run_batch([gesso_b200.BatchRequest(p, 4, on_token=boom), gesso_b200.BatchRequest(p, 4),
                       gesso_b200.BatchRequest([], 4), gesso_b200.BatchRequest([9999], 4)])
    assert [r.status for r in res] == ["failed", "complete", "failed", "failed"]
    assert res[1].ids == full[:7] and res[0].error.code == gesso_b200.ErrorCode.RUNTIME
    with pytest.raises(gesso_b200.GessoError):
        s.generate([1] * 65, 1)                                             # longer than the context
    assert s.engine.cache.pages_in_use() == [0]


def test_a_status_word_set_during_a_step_fails_that_steps_requests_only(models):
    """The kernels report a position without a page, or a pipeline wait that ran out, through the engine's
    status words instead of trapping.  The words come back with the sampled ids; when one is set the
    requests of the steps it covers end as failed (what was sampled for them is dropped, their pages go
    back) and the others go on (src/Runtime/Runtime.jl:151-153, 175-178).  The word is set from the host
    here, between two steps: no kernel is made to fail."""
    import gesso_b200
    model = models("a", "float32")         # float32: a request's ids do not depend on who else is in the batch
    prompts = prompts_for("a", [9, 30, 4, 12], seed=5)
    alone = [gesso_b200.Session(model, context_length=128, max_batch=1).generate(p, 8) for p in prompts]
    for word in (0, 1):
        s = gesso_b200.Session(model, context_length=128, max_batch=2)
        sched = s.open_batch([gesso_b200.BatchRequest(p, max_new_tokens=8) for p in prompts])
        with pytest.raises(gesso_b200.GessoError):
            s.generate(prompts[0], 1)                   # the session is busy while its stream is open
        reqs = list(sched.waiting)
        for _ in range(3):
            sched.step()
        assert [r.state for r in reqs] == ["running", "running", "waiting", "waiting"]
        s.engine.status_words[word] = 7                 # as a kernel of the next step would
        sched.run()
        assert [r.status for r in reqs] == ["failed", "failed", "complete", "complete"]
        for r in reqs[:2]:
            assert r.error.code == gesso_b200.ErrorCode.RUNTIME and 1 <= len(r.generated) < 8
        assert ("tcgen05" in str(reqs[0].error)) == (word == 1)
        assert [r.ids for r in reqs[2:]] == alone[2:]
        assert int(s.engine.status_words.abs().sum().item()) == 0          # cleared for the steps to come
        assert s.engine.cache.pages_in_use() == [0] and s.engine.cache.slots_in_use() == 0
        assert s.generate(prompts[0], 8) == alone[0]    # and the session is free again


@pytest.mark.parametrize("use_graphs", [True, False])
def test_a_step_takes_token_ids_that_are_still_on_the_device(use_graphs, models):
    """``Engine.step(entries, device_tokens=(ids, runs))``: the tokens named by the runs come from a device
    tensor, whatever the entries hold in their place; the logits equal those of the same step fed from the
    host, in a decoding step, in a mixed step, and when the shape's graph is replayed a second time."""
    import gesso_b200
    from gesso_b200.engine import Engine, StepEntry
    model = models("b", "float32")
    vocab = model.vocab_size

    def run(from_device):
        eng = Engine(model, max_positions=64, max_requests=4, use_graphs=use_graphs)
        for rid in "abcd":
            eng.admit(rid)
        eng.step([StepEntry("a", [3, 4, 5], []), StepEntry("b", [6], []), StepEntry("c", [7, 8], [])])
        outs = []
        ids = torch.tensor([11 % vocab, 12 % vocab, 13 % vocab, 14 % vocab], dtype=torch.int32, device="cuda")
        for turn in range(2):                  # the second turn replays what the first captured
            real = [int(t) for t in ids.tolist()]
            # a decoding step of a, b, c: ids 0, 2, 3 (two runs)
            if from_device:
                entries = [StepEntry(r, [0], [0]) for r in "abc"]
                outs.append(eng.step(entries, device_tokens=(ids, [(0, 0, 1), (2, 1, 2)])).clone())
            else:
                outs.append(eng.step([StepEntry("a", [real[0]], [0]), StepEntry("b", [real[2]], [0]),
                                      StepEntry("c", [real[3]], [0])]).clone())
            # a mixed step: b and a decode from ids 1 and 0, d brings a portion from the host
            portion = [(5 + 3 * turn + i) % vocab for i in range(5)]
            if from_device:
                entries = [StepEntry("b", [0], [0]), StepEntry("a", [0], [0]), StepEntry("d", portion, [4])]
                outs.append(eng.step(entries, device_tokens=(ids, [(1, 0, 1), (0, 1, 1)])).clone())
            else:
                outs.append(eng.step([StepEntry("b", [real[1]], [0]), StepEntry("a", [real[0]], [0]),
                                      StepEntry("d", portion, [4])]).clone())
            ids = (ids + 17) % vocab
        eng.check_status()
        return outs

    for got, want in zip(run(True), run(False)):
        assert torch.equal(got, want)
    eng = Engine(model, max_positions=64, max_requests=2)
    eng.admit("a")
    ids = torch.zeros(2, dtype=torch.int32, device="cuda")
    with pytest.raises(gesso_b200.GessoError, match="device tokens"):
        eng.step([StepEntry("a", [1], [0])], device_tokens=(ids, [(1, 0, 2)]))          # a run past the ids
    with pytest.raises(gesso_b200.GessoError, match="device tokens"):
        eng.step([StepEntry("a", [1], [0])], device_tokens=(ids.long(), [(0, 0, 1)]))   # not int32
    assert eng.length("a") == 0


def test_a_request_of_a_failed_step_can_only_be_released(models):
    """Driving the engine directly: after a step that failed, or whose status was bad, its requests have
    keys, values and state of a half-run step in the cache; a further step with one of them is refused."""
    import gesso_b200
    from gesso_b200.engine import Engine, StepEntry
    model = models("a", "float32")
    eng = Engine(model, max_positions=64, max_requests=3)
    for rid in ("x", "y", "z"):
        eng.admit(rid)
    eng.step([StepEntry("x", [1, 2, 3], [2]), StepEntry("y", [4, 5], [])])
    eng.check_status()                                   # all well
    eng.step([StepEntry("y", [6], [0])])
    eng.status[0] = 1
    with pytest.raises(gesso_b200.GessoError, match="without a cache page"):
        eng.check_status()
    with pytest.raises(gesso_b200.GessoError, match="cannot go on"):
        eng.step([StepEntry("y", [7], [0]), StepEntry("z", [1], [0])])
    assert eng.length("z") == 0                          # the refused step touched nobody
    out = eng.step([StepEntry("x", [4], [0]), StepEntry("z", [1, 2], [1])])      # x was not part of the bad step
    assert out.shape[0] == 2 and bool(torch.isfinite(out).all())
    eng.check_status()
    eng.release("y")
    eng.admit("y")                                       # a new request under the old name starts clean
    eng.step([StepEntry("y", [4, 5, 6], [2])])
    eng.check_status()
    # a step that raises inside the engine (the model's forward here) marks its requests too
    real = model.forward
    try:
        model.forward = lambda ctx, views: (_ for _ in ()).throw(RuntimeError("forward broke"))
        with pytest.raises(RuntimeError, match="forward broke"):
            eng.step([StepEntry("z", [3, 4], [1])])
    finally:
        model.forward = real
    with pytest.raises(gesso_b200.GessoError, match="cannot go on"):
        eng.step([StepEntry("z", [5], [0])])
    for rid in ("x", "y", "z"):
        eng.release(rid)
    eng.cache.check_invariants()
    assert eng.cache.pages_in_use() == [0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_run_out_preemption_keeps_the_tokens(dtype, models, plain_models):
    """A pool too small for everybody: requests are preempted and recomputed.  In float32 the ids are the
    plain model's.  In bfloat16 (model "c", head size 32: the tensor-core attention kernels) a recomputed
    prefix runs as a prompt portion where the first run decoded token by token, other kernels and other
    roundings, so every token must be a near-maximum of the plain logits."""
    import gesso_b200
    name = "a" if dtype == "float32" else "c"
    model = models(name, dtype)
    prompts = prompts_for(name, [30, 28, 25, 20], seed=8)
    s = gesso_b200.Session(model, context_length=64, page_size=16, num_pages=7, max_batch=4, prefill_chunk=16)
    res = s.run_batch([gesso_b200.BatchRequest(p, max_new_tokens=30) for p in prompts])
    assert s.stats()["preemptions"] >= 1
    for p, r in zip(prompts, res):
        assert r.status == "complete" and len(r.ids) == len(p) + 30
        if dtype == "float32":
            assert r.ids == plain_models[name].greedy(p, 30)
        else:
            near_max(plain_models[name], r.ids, len(p), TOL16)
    assert s.engine.cache.pages_in_use() == [0]


# ---- prefill / decode of a Session ----------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [("float32", TOL32), ("bfloat16", TOL16)])
def test_session_prefill_decode(dtype, tol, models, plain_models):
    import gesso_b200
    s = gesso_b200.Session(models("b", dtype), context_length=128, page_size=16)
    p = prompts_for("b", [21], seed=9)[0]
    logits = s.prefill(p)
    ref = plain_models["b"].logits(p).numpy()
    assert logits.shape == ref.shape and np.abs(logits - ref).max() <= tol * max(1, np.abs(ref).max())
    assert s.kv_len == len(p)
    ids = list(p)
    for step in range(5):
        tok = s.decode()
        ids.append(tok)
        assert s.kv_len == len(p) + step + 1                                # test/test_reference_generate.jl:39-46
    if dtype == "float32":
        assert ids == plain_models["b"].greedy(p, 5)
    with pytest.raises(gesso_b200.GessoError):
        gesso_b200.Session(models("b", dtype), context_length=128).decode()  # nothing prefilled


# ---- long decoding, first tokens ----------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [("float32", TOL32), ("bfloat16", TOL16)])
def test_long_decoding_token_by_token(dtype, tol, models, plain_models):
    """300 tokens, all but the first fed one by one (CUDA-graph steps), across many pages."""
    from gesso_b200.engine import Engine, StepEntry
    model = models("c", dtype)
    ids = prompts_for("c", [300], seed=4)[0]
    ref = plain_models["c"].logits(ids).numpy()
    eng = Engine(model, max_positions=320, page_size=16, num_pages=20, max_requests=1)
    eng.admit("r")
    scale = max(1.0, float(np.abs(ref).max()))
    for t, tok in enumerate(ids):
        row = eng.step([StepEntry("r", [tok], [0])])[0].cpu().numpy()
        err = float(np.abs(row - ref[t]).max())
        assert err <= tol * scale, f"position {t}: {err:.3e}"
    eng.check_status()


@pytest.mark.parametrize("dtype,tol", [("float32", TOL32), ("bfloat16", TOL16)])
def test_long_context(dtype, tol, model_dirs, plain_models):
    """5,000 tokens: the prompt in portions of 2,048, then 24 tokens one by one at positions near 5,000
    (hundreds of pages per request, many key splits, rotation angles at large positions), beside a short
    request that shares the steps."""
    import gesso_b200
    from gesso_b200.engine import Engine, StepEntry
    model = gesso_b200.load(model_dirs["a"], dtype=dtype, max_positions=5120)
    ids = prompts_for("a", [5000], seed=12)[0]
    other = prompts_for("a", [40], seed=13)[0]
    plain = plain_models["a"]
    ref = plain.logits(ids).numpy()
    ref_o = plain.logits(other).numpy()
    eng = Engine(model, max_positions=5120, page_size=16, num_pages=330, max_requests=2)
    eng.admit("long")
    eng.admit("short")
    scale, scale_o = max(1.0, float(np.abs(ref).max())), max(1.0, float(np.abs(ref_o).max()))
    head = len(ids) - 24
    for at in range(0, head, 2048):
        n = min(2048, head - at)
        out = eng.step([StepEntry("long", ids[at:at + n], [0, n - 1])]).cpu().numpy()
        assert float(np.abs(out[0] - ref[at]).max()) <= tol * scale, f"position {at}"
        assert float(np.abs(out[1] - ref[at + n - 1]).max()) <= tol * scale, f"position {at + n - 1}"
    eng.step([StepEntry("short", other[:16], [])])
    for k in range(24):
        out = eng.step([StepEntry("short", [other[16 + k]], [0]), StepEntry("long", [ids[head + k]], [0])]).cpu().numpy()
        assert float(np.abs(out[0] - ref_o[16 + k]).max()) <= tol * scale_o, f"short request, position {16 + k}"
        assert float(np.abs(out[1] - ref[head + k]).max()) <= tol * scale, f"position {head + k}"
    eng.check_status()


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_first_tokens_of_a_sequence(name, models, plain_models):
    """Prompts of 1, 2, 3 tokens, whole and token by token: the conv history is shorter than its
    kernel and the cache holds a single partly filled page."""
    from gesso_b200.engine import Engine, StepEntry
    model = models(name, "float32")
    for n in (1, 2, 3, 4):
        ids = prompts_for(name, [n], seed=20 + n)[0]
        ref = plain_models[name].logits(ids).numpy()
        for cuts in ([n], [1] * n):
            eng = Engine(model, max_positions=16, page_size=16, num_pages=1, max_requests=1)
            eng.admit("r")
            rows, p = [], 0
            for c in cuts:
                rows.append(eng.step([StepEntry("r", ids[p:p + c], list(range(c)))]).cpu().numpy().copy())
                p += c
            assert np.abs(np.concatenate(rows) - ref).max() <= TOL32 * max(1, np.abs(ref).max())


# ---- weights made so that faults show ----------------------------------------------------------------------
@pytest.fixture(scope="module")
def sharp_model_dir(model_dirs, tmp_path_factory):
    """Model 'a' with its q/k norm weights scaled by 4: attention scores spread over +-16, so single
    keys dominate and a wrong key, page or position changes the logits by far more than rounding."""
    from gesso_b200.weights import read_safetensors_file, write_safetensors_file
    d = str(tmp_path_factory.mktemp("model_a_sharp"))
    t = read_safetensors_file(os.path.join(model_dirs["a"], "model.safetensors"))
    for k in t:
        if k.endswith("q_layernorm.weight"):
            t[k] = t[k] * 4.0
    write_safetensors_file(os.path.join(d, "model.safetensors"), t)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(configs.TINY_A, f)
    return d


@pytest.mark.parametrize("dtype,tol", [("float32", TOL32), ("bfloat16", 2 * TOL16)])
def test_sharp_attention_far_keys_and_page_edges(dtype, tol, sharp_model_dir):
    """A 400-token request decoded across page edges beside another request whose pages were used before."""
    import gesso_b200
    from gesso_b200.engine import Engine, StepEntry
    from plain_lfm2 import PlainModel
    plain = PlainModel(sharp_model_dir)
    model = gesso_b200.load(sharp_model_dir, dtype=dtype, max_positions=512)
    g = torch.Generator().manual_seed(77)
    a = torch.randint(0, 256, (400,), generator=g).tolist()
    b = torch.randint(0, 256, (90,), generator=g).tolist()
    ref_a, ref_b = plain.logits(a).numpy(), plain.logits(b).numpy()
    # the plain attention is sharp: the largest probability of the last rows is well above uniform
    eng = Engine(model, max_positions=512, page_size=16, num_pages=32, max_requests=2)
    eng.admit("old")
    eng.step([StepEntry("old", b[:70], [])])          # fills pages that "b" will get again
    eng.release("old")
    eng.admit("a")
    eng.admit("b")
    got_a = [eng.step([StepEntry("a", a[:250], list(range(250)))]).cpu().numpy().copy()]
    pa, pb = 250, 0
    got_b = []
    while pa < len(a) or pb < len(b):
        entries = []
        if pa < len(a):
            n = 1 if pa >= 300 else min(31, len(a) - pa)
            entries.append(StepEntry("a", a[pa:pa + n], list(range(n))))
        if pb < len(b):
            m = min(7, len(b) - pb) if pb < 60 else 1
            entries.append(StepEntry("b", b[pb:pb + m], list(range(m))))
        out = eng.step(entries).cpu().numpy().copy()
        if pa < len(a):
            got_a.append(out[:n])
            out = out[n:]
            pa += n
        if pb < len(b):
            got_b.append(out)
            pb += m
    for got, ref, what in ((np.concatenate(got_a), ref_a, "a"), (np.concatenate(got_b), ref_b, "b")):
        err = np.abs(got - ref).max(axis=1)
        bad = np.nonzero(err > tol * max(1, np.abs(ref).max()))[0]
        assert bad.size == 0, f"request {what}: first wrong position {bad[0]} (error {err[bad[0]]:.3e})"
    eng.check_status()


# ---- the command line ---------------------------------------------------------------------------------
def test_command_line(model_dirs, plain_models, tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root)
    p = subprocess.run([sys.executable, "-m", "gesso_b200", "generate", "--model", model_dirs["a"], "--dtype", "float32",
                        "--prompt-ids", "5,6,7", "--prompt-ids", "9 8", "--max-new-tokens", "4", "--n-ctx", "64"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-1500:]
    lines = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")]
    assert [l["ids"] for l in lines] == [plain_models["a"].greedy([5, 6, 7], 4), plain_models["a"].greedy([9, 8], 4)]
    bad = subprocess.run([sys.executable, "-m", "gesso_b200", "generate", "--model", model_dirs["a"], "--no-such-flag"],
                         capture_output=True, text=True, env=env, timeout=120)
    assert bad.returncode == 2 and "usage" in bad.stderr.lower()
    # random-weights mode writes a model folder that loads
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(configs.TINY_C))
    out = tmp_path / "m"
    r = subprocess.run([sys.executable, "-m", "gesso_b200", "init-random", "--config", str(cfg), "--seed", "3", "--out", str(out)],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
    d = subprocess.run([sys.executable, "-m", "gesso_b200", "describe", "--model", str(out)], capture_output=True, text=True, env=env)
    assert d.returncode == 0 and "short_conv" in d.stdout
    # generate straight from a configuration and a seed, no folder in between
    g = subprocess.run([sys.executable, "-m", "gesso_b200", "generate", "--random-weights", "3", "--config", str(cfg),
                        "--prompt-ids", "5,6,7", "--max-new-tokens", "3", "--n-ctx", "64"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert g.returncode == 0, g.stderr[-1500:]
    line = json.loads([l for l in g.stdout.splitlines() if l.startswith("{")][0])
    assert line["status"] == "complete" and line["ids"][:3] == [5, 6, 7] and len(line["ids"]) == 6
    both = subprocess.run([sys.executable, "-m", "gesso_b200", "generate", "--model", str(out), "--random-weights", "3",
                           "--prompt-ids", "5"], capture_output=True, text=True, env=env, timeout=120)
    assert both.returncode == 2
    # replay as a sub-command: the same program as bin/trace_run
    steps = '{"step": 0, "entries": [{"id": "a", "tokens": [5, 6, 7], "want": [2]}], "end": ["a"]}\n'
    rp = subprocess.run([sys.executable, "-m", "gesso_b200", "replay", "--model", model_dirs["a"], "--dtype", "float32",
                         "--out", str(tmp_path / "rp"), "--max-tokens", "64"], input=steps, capture_output=True, text=True,
                        env=env, timeout=600)
    assert rp.returncode == 0 and "done 0" in rp.stdout, rp.stderr[-1500:]
    row = np.fromfile(tmp_path / "rp" / "0.f32", dtype="<f4")
    ref = plain_models["a"].logits([5, 6, 7])[2].numpy()
    assert row.shape == ref.shape and float(np.abs(row - ref).max()) <= TOL32 * max(1.0, float(np.abs(ref).max()))
    # bench as a sub-command hands its options to bench.py, which refuses more than one GPU with exit code 2
    bn = subprocess.run([sys.executable, "-m", "gesso_b200", "bench", "--gpus", "2"], capture_output=True, text=True, env=env,
                        timeout=120)
    assert bn.returncode == 2 and "one GPU" in bn.stdout
