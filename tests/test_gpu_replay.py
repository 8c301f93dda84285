"""Replay of the same requests under four ways of cutting and batching, in float32 and bfloat16,
against the plain implementation."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import configs
import trace_tools as tt

pytestmark = pytest.mark.gpu

# float32: the reference's device tolerance, 1e-4 * max(1, max|ref|) (test/test_lava_lfm25.jl:31-32).
TOL = {"float32": 1e-4,
       # bfloat16: every stored activation is rounded to 8 bits (unit roundoff u = 2^-9).  The plain
       # implementation with a bfloat16 rounding at each place where the engine stores an activation
       # (norm outputs, projection outputs, rotated q/k, attention, conv and SwiGLU outputs) differs
       # from the exact one by 0.036-0.040 of max|ref| on these models (rms 1.3-2.8 %), so the bound
       # is 32 u = 0.0625 of max(1, max|ref|).
       "bfloat16": 32 * 2.0 ** -9}

LENGTHS = {"a": [7, 13, 1, 70, 33, 97, 16, 65],
           "b": [40, 1, 23, 64, 81, 5, 17, 50],
           "c": [48, 3, 90, 31]}


@pytest.fixture(scope="module")
def loaded(model_dirs):
    import gesso_b200
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            cache[(name, dtype)] = gesso_b200.load(model_dirs[name], dtype=dtype, max_positions=1024)
        return cache[(name, dtype)]
    return get


@pytest.fixture(scope="module")
def plain_logits(plain_models):
    cache = {}

    def get(name):
        if name not in cache:
            vocab = configs.TINY[name][0]["vocab_size"]
            reqs = tt.make_requests(vocab, LENGTHS[name], seed=100 + len(name))
            cache[name] = (reqs, [plain_models[name].logits(t).numpy() for t in reqs])
        return cache[name]
    return get


SCHEDULES = {
    "whole": lambda reqs: tt.trace_whole(reqs),
    "tail_decode": lambda reqs: tt.trace_tail_decode(reqs),
    "portions": lambda reqs: tt.trace_portions(reqs),
    "mixed": lambda reqs: tt.trace_mixed(reqs, seed=7),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", list(SCHEDULES))
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_replay_matches_plain(name, schedule, dtype, loaded, plain_logits, tmp_path):
    reqs, ref = plain_logits(name)
    tb, max_tokens = SCHEDULES[schedule](reqs)
    model = loaded(name, dtype)
    tt.run_in_process(model, tb, max_tokens, str(tmp_path))
    rows = tt.read_rows(tb, str(tmp_path), model.vocab_size)
    worst = tt.compare_with_plain(rows, ref, TOL[dtype], f"{name}/{schedule}/{dtype}")
    print(f"worst relative error {name}/{schedule}/{dtype}: {worst:.3e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedules_agree_closely(dtype, loaded, plain_logits, tmp_path):
    """The logits at a position do not depend on the cutting or the batch beyond rounding: in float32
    the schedules agree to 2e-5 (the reference's decode-vs-prefill bound, test/test_lfm25.jl:185)."""
    reqs, _ = plain_logits("b")
    model = loaded("b", dtype)
    got = {}
    for sched, make in SCHEDULES.items():
        tb, max_tokens = make(reqs)
        d = tmp_path / sched
        tt.run_in_process(model, tb, max_tokens, str(d))
        got[sched] = tt.read_rows(tb, str(d), model.vocab_size)
    base = got["whole"]
    bound = 2e-5 if dtype == "float32" else TOL["bfloat16"]
    for sched, rows in got.items():
        for key, row in rows.items():
            scale = max(1.0, float(np.abs(base[key]).max()))
            err = float(np.abs(row - base[key]).max())
            assert err <= bound * scale, f"{sched} differs from whole at request/position {key}: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,schedule", [("a", "mixed"), ("b", "mixed"), ("c", "mixed"), ("c", "portions"),
                                           ("c", "tail_decode")])
def test_what_a_free_page_holds_never_reaches_a_request(name, schedule, dtype, loaded, plain_logits, tmp_path):
    """Pages and state slots go from request to request as they are.  Whatever the last owner left in
    them, non-finite values included (a request whose activations overflowed ends, its pages do not
    get cleaned), a new request starts from nothing and never sees another's rows
    (src/Inference/Inference.jl:147-148, src/Inference/generate_state.jl:188-192).  Every free page
    and slot is filled with NaN before the first step; the mixed replay uses pages again.  Model "c"
    has head size 32, so its bfloat16 runs take the tensor-core attention kernels."""
    reqs, ref = plain_logits(name)
    tb, max_tokens = SCHEDULES[schedule](reqs)
    model = loaded(name, dtype)
    tt.run_in_process(model, tb, max_tokens, str(tmp_path), prepare=tt.poison_free_memory)
    rows = tt.read_rows(tb, str(tmp_path), model.vocab_size)
    tt.compare_with_plain(rows, ref, TOL[dtype], f"poisoned pages {name}/{schedule}/{dtype}")


def test_trace_run_program(model_dirs, plain_logits, tmp_path):
    """The program itself, as a user runs it: a subprocess fed through standard input."""
    reqs, ref = plain_logits("a")
    tb, max_tokens = tt.trace_mixed(reqs, seed=3)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model_dirs["a"],
                        "--dtype", "float32", "--out", str(out), "--max-tokens", str(max_tokens)],
                       input=tb.text(), capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(tb.steps))]
    rows = tt.read_rows(tb, str(out), configs.TINY_A["vocab_size"])
    tt.compare_with_plain(rows, ref, TOL["float32"], "trace_run a/mixed/float32")


def test_replay_through_the_tcgen05_product(model_dirs, plain_logits, tmp_path, monkeypatch):
    """Steps of 17 tokens or more forced onto the tcgen05 matrix product (fused residual add and
    SwiGLU epilogues included), on the tiny models, against the plain implementation."""
    import gesso_b200
    from gesso_b200 import ops
    monkeypatch.setattr(ops, "TC_MIN_ROWS", 17)
    for name in ("a", "c"):
        reqs, ref = plain_logits(name)
        model = gesso_b200.load(model_dirs[name], dtype="bfloat16", max_positions=1024)
        for sched in ("whole", "mixed"):
            tb, max_tokens = SCHEDULES[sched](reqs)
            d = tmp_path / f"{name}_{sched}"
            tt.run_in_process(model, tb, max_tokens, str(d))
            tt.compare_with_plain(tt.read_rows(tb, str(d), model.vocab_size), ref, TOL["bfloat16"], f"tcgen05 {name}/{sched}")
        ops.check_tc_status()
