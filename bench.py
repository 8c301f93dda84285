#!/usr/bin/env python3
"""Decode and prefill throughput of the LFM2-1.2B-shaped model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096] [--layers 16]
    python bench.py --impl reference        # the reference arm (unavailable: a Julia project)

A "step" is one decode step of the whole batch.  The default run: the layer sizes of LFM2-1.2B
(16 layers, attention at 2,5,8,10,12,14, hidden 2048, 32 heads, 8 kv heads, head 64, ff 8192, vocab
65536, 3 conv taps, tied head), random weights (seed 0), batch 8, context 4096 with 16-token pages:
every request holds ``context - steps - warmup - 1`` tokens when the timed steps begin, so the last
timed step runs at the full context.

One JSON line is printed:

* ``value``: decoded tokens per second, K steps timed on the device with CUDA events (W warm-up steps
  before); inputs of a step are larger than L2 (all weights are read once per step);
* ``e2e``: the same through the Python entry point (``Session.open_batch`` + ``step()``): host token
  ids in, sampled ids out, every step's metadata copied from pinned host memory and its ids read back;
* ``prefill``: a prefill step of one request of 2,048 tokens, logits at its last position: the device time
  per step of five such steps in a row (the engine replays a captured graph for a portion of a length it
  has seen before); ``frac`` = flops / time / the bf16 peak;
* ``roofline``: bytes a decode step has to read (every weight once + the cache of the live requests)
  / its time, against the measured copy bandwidth;
* ``points``: decode tokens per second at batch 1 and 64 (context 4,096) and at batch 8 with contexts of
  512 and 2,048; ``rooflines``: the same fraction as ``roofline`` for every decode point;
* ``blocks``: the timed steps cut into 8 blocks by events on the stream (no host wait between them): the
  median and the extremes of their per-step times, beside the one bracket around all K steps that ``value``
  comes from (the reference's rule: warm up, report samples, benchmark/runbenchmarks.jl:5-10);
* ``cpu_baseline``: the plain float64 implementation of the tests (``tests/plain_lfm2.py``: whole
  sequences, no cache, CPU) generating greedily at the two tiny configurations, in tokens per second.

Other workloads, each printing one JSON line of its own:

    python bench.py --workload serve350m     # LFM2-350M sizes: 64 live requests, prompts of 128-2,048 tokens
                                             # in portions of 512 beside the decoding requests
    python bench.py --workload serve700m     # LFM2-700M sizes: 32 requests, prompts of 64-4,096 tokens,
                                             # 256 new tokens each, temperature 0.8

both through ``Session.run_batch`` (scheduler, cache manager, sampler), with the host and device time of
a step;

    python bench.py --workload timeline --batch 8      # the kernels of one decoding step, by name

a table (not JSON) of where a step's time goes, from the CUPTI activity trace.

Peaks come from ``MEASURED_PEAKS.json`` beside this file when the driver wrote it, else the
fallback of an earlier measurement on this pool (6.65 TB/s, 1.59 PFLOP/s).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}

LFM2_1_2B = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 65536, "hidden_size": 2048, "num_hidden_layers": 16,
    "num_attention_heads": 32, "num_key_value_heads": 8,
    "full_attn_idxs": [2, 5, 8, 10, 12, 14],
    "conv_L_cache": 3, "conv_bias": False, "block_ff_dim": 12288, "block_auto_adjust_ff_dim": True,
    "block_multiple_of": 256, "norm_eps": 1e-5, "rope_theta": 1000000.0, "tie_embedding": True,
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            out = {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
            if "bf16_tflops_sustained" in p:
                out["bf16_tflops_sustained"] = float(p["bf16_tflops_sustained"])
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid=None):
        super().__init__(daemon=True)
        self.samples, self.stop_flag = [], threading.Event()
        # the device this process computes on, by UUID: index 0 of nvidia-smi is another GPU when the
        # process sees one of several through CUDA_VISIBLE_DEVICES
        self.gpu = str(uuid) if uuid else "0"

    def run(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", self.gpu, f"--query-gpu={self.Q}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip().splitlines()
                if out:
                    self.samples.append([x.strip() for x in out[0].split(",")])
            except Exception:
                pass
            self.stop_flag.wait(0.05)

    def summary(self):
        self.stop_flag.set()
        self.join(timeout=6)
        mhz, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                mhz.append(float(s[0]))
                mx = float(s[1])
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz), "gpu": self.gpu}


def device_uuid():
    """``GPU-...`` of cuda:0 as nvidia-smi names it."""
    import torch
    try:
        u = str(torch.cuda.get_device_properties(0).uuid)
        return u if u.startswith("GPU-") else "GPU-" + u
    except Exception:
        return None


def model_flops_per_token(cfg_obj, n_layers_attn, n_layers_conv):
    H, F, V = cfg_obj.hidden_size, cfg_obj.ff_dim, cfg_obj.vocab_size
    kv = cfg_obj.num_key_value_heads * cfg_obj.head_dim
    conv = 3 * H * H + H * H + 3 * F * H
    attn = H * H + 2 * kv * H + H * H + 3 * F * H
    return 2 * (n_layers_conv * conv + n_layers_attn * attn), 2 * V * H


def decode_setup(gb, model, batch, context, steps, warmup, page_size, seed=1, margin=0):
    """A session with ``batch`` requests prefilled so that the timed steps end at the full context
    (``margin`` tokens short of it)."""
    import torch
    start_len = max(1, context - steps - warmup - 1 - margin)
    pages = batch * ((context + page_size - 1) // page_size)
    s = gb.Session(model, context_length=context, page_size=page_size, num_pages=pages, max_batch=batch,
                   max_tokens_per_step=4096, prefill_chunk=2048)
    g = torch.Generator().manual_seed(seed)
    prompts = [torch.randint(0, model.vocab_size, (start_len,), generator=g).tolist() for _ in range(batch)]
    return s, prompts, start_len


def time_decode(gb, model, batch, context, steps, warmup, page_size):
    """Device-timed decode: K steps of the engine's step function with greedy selection on the device."""
    import torch
    from gesso_b200.engine.batch import StepEntry
    from gesso_b200 import ops
    s, prompts, start_len = decode_setup(gb, model, batch, context, steps, warmup, page_size)
    eng = s.engine
    ids = [f"q{i}" for i in range(batch)]
    for rid, p in zip(ids, prompts):
        eng.admit(rid)
        for c in range(0, len(p), 2048):
            eng.step([StepEntry(rid, p[c:c + 2048], [])])
    g = torch.Generator().manual_seed(7)
    toks = torch.randint(0, model.vocab_size, (warmup + steps, batch), generator=g).tolist()

    def one(k):
        logits = eng.step([StepEntry(rid, [toks[k][i]], [0]) for i, rid in enumerate(ids)])
        ops.argmax_rows(logits)

    for k in range(warmup):
        one(k)
    torch.cuda.synchronize()
    launches0 = eng.launches
    # one bracket around all K steps, and events on the stream that cut them into blocks (no host wait)
    n_blocks = min(8, steps)
    cuts = [round(i * steps / n_blocks) for i in range(n_blocks + 1)]
    marks = [torch.cuda.Event(enable_timing=True) for _ in cuts]
    marks[0].record()
    nxt = 1
    for k in range(steps):
        one(warmup + k)
        if k + 1 == cuts[nxt]:
            marks[nxt].record()
            nxt += 1
    torch.cuda.synchronize()
    ms = marks[0].elapsed_time(marks[-1])
    per_block = sorted(marks[i].elapsed_time(marks[i + 1]) / (cuts[i + 1] - cuts[i]) for i in range(n_blocks))
    time_decode.blocks = {"n": n_blocks, "ms_per_step_median": round(per_block[n_blocks // 2], 4),
                          "ms_per_step_min": round(per_block[0], 4), "ms_per_step_max": round(per_block[-1], 4)}
    launches = eng.launches - launches0 + steps          # + the argmax launch of every step
    eng.check_status()
    kv_len_mid = start_len + warmup + steps // 2
    for rid in ids:
        eng.release(rid)
    return ms / steps, launches, kv_len_mid


def time_e2e(gb, model, batch, context, steps, warmup, page_size):
    """The same through the Python entry point: host ids in, sampled ids out, every step."""
    import torch
    # While the later prompts are still being prefilled the earlier requests already decode; the
    # margin keeps every request short of the context until the timed steps are over, so that the
    # batch stays whole (no request ends, and no step of another batch size falls into the timed region).
    margin = batch * (context // 4096 + 1) + 2
    s, prompts, start_len = decode_setup(gb, model, batch, context, steps, warmup, page_size, margin=margin)
    sched = s.open_batch([gb.BatchRequest(p, max_new_tokens=context - start_len) for p in prompts])
    while any(r.fed < len(r.prompt) for r in sched.running + sched.waiting):
        sched.step()                                       # prefill
    for _ in range(warmup):
        sched.step()
    torch.cuda.synchronize()
    h2d0 = s.engine.h2d_bytes
    t0 = time.perf_counter()
    emitted = 0
    for _ in range(steps):
        emitted += len(sched.step())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = (s.engine.h2d_bytes - h2d0) / steps
    d2h = 2 * 4 * batch + 2 * 4                             # ids + flags read back (int32 each) and the two status words
    return emitted / dt, h2d, d2h


def time_prefill(gb, model, tokens, page_size, reps=5):
    """Device time of one prefill step of ``tokens`` tokens (logits at the last position): ``reps`` requests are
    prefilled back to back behind a first, untimed one, with events on the stream around the timed ones.  The
    host prepares and launches a step while the device still runs the one before, as in a serving loop, so the
    time between the events is the device's; a single step timed from an idle device would also count the
    host's preparation and the launch of its graph (0.3 ms here), which steps in a row hide."""
    import torch
    from gesso_b200.engine.batch import StepEntry
    from gesso_b200.engine.engine import Engine
    n = reps + 1
    eng = Engine(model, max_positions=max(tokens, 64), page_size=page_size,
                 num_pages=n * ((tokens + page_size - 1) // page_size) + 1, max_requests=n)
    g = torch.Generator().manual_seed(3)
    p = torch.randint(0, model.vocab_size, (tokens,), generator=g).tolist()
    best = None
    for r in range(3):                       # the first rounds capture the step's graph
        for i in range(n):
            eng.admit(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        eng.step([StepEntry(0, p, [tokens - 1])])
        e0.record()
        for i in range(1, n):
            eng.step([StepEntry(i, p, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        eng.check_status()
        for i in range(n):
            eng.release(i)
        if r >= 1:
            best = ms if best is None else min(best, ms)
    return best


def cpu_baseline():
    """The timed CPU baseline: the plain implementation of the tests (float64, whole sequences, no cache, one
    function per part, ``tests/plain_lfm2.py``) generating greedily at the two tiny configurations with
    the prompts the configurations name.  It is a restatement of the reference's formulas, not the
    reference (a Julia project that cannot run here)."""
    import tempfile
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import configs
    from plain_lfm2 import PlainModel
    from gesso_b200.weights import write_random_model
    out = {"what": "tests/plain_lfm2.py (float64, no cache) on the CPU, greedy, tokens/s"}
    g = torch.Generator().manual_seed(0)
    for name, lengths, n_new in (("a", [7, 13, 1], 8), ("b", [1, 9, 17, 28, 40], 8)):
        cfg, seed, _ = configs.TINY[name]
        with tempfile.TemporaryDirectory() as d:
            write_random_model(d, cfg, seed)
            plain = PlainModel(d)
            prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]
            t0 = time.perf_counter()
            for p in prompts:
                plain.greedy(p, n_new)
            out[f"tiny_{name}"] = round(len(prompts) * n_new / (time.perf_counter() - t0), 1)
    return out


SERVE = {
    # BASELINE configuration 4: LFM2-350M layer sizes, a mixed batch of 64 decodes beside 512-token portions,
    # random prompts of 128 to 2,048 tokens
    "serve350m": dict(hidden=1024, heads=16, block_ff=6656, requests=96, max_batch=64, prompt=(128, 2048), new=64,
                      chunk=512, temperature=0.0, top_p=1.0, context=2304),
    # BASELINE configuration 5: LFM2-700M layer sizes, 32 concurrent requests, prompts of 64 to 4,096 tokens,
    # 256 new tokens each, temperature 0.8
    "serve700m": dict(hidden=1536, heads=24, block_ff=10240, requests=32, max_batch=32, prompt=(64, 4096), new=256,
                      chunk=512, temperature=0.8, top_p=0.95, context=4352),
}


def serve_workload(name: str) -> int:
    """One of the serving-like runs through ``Session.run_batch``; the second run of the workload is timed
    (the first captures the graphs a serving process would have long had)."""
    import torch
    import gesso_b200 as gb
    w = SERVE[name]
    cfg = dict(LFM2_1_2B, hidden_size=w["hidden"], num_attention_heads=w["heads"], block_ff_dim=w["block_ff"])
    model = gb.random_model(cfg, seed=0, dtype="bfloat16", max_positions=w["context"])
    pages = w["max_batch"] * ((w["context"] + 15) // 16)

    def run(seed):
        g = torch.Generator().manual_seed(seed)
        lens = torch.randint(w["prompt"][0], w["prompt"][1] + 1, (w["requests"],), generator=g).tolist()
        prompts = [torch.randint(0, model.vocab_size, (n,), generator=g).tolist() for n in lens]
        s = run.session
        reqs = [gb.BatchRequest(p, max_new_tokens=w["new"], temperature=w["temperature"], top_p=w["top_p"], seed=i)
                for i, p in enumerate(prompts)]
        steps0, tokens0 = s.engine.steps_run, s.engine.tokens_run
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        t0 = time.perf_counter()
        res = s.run_batch(reqs)
        e1.record()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        assert all(r.status == "complete" for r in res), [(r.status, r.error) for r in res if r.status != "complete"][:2]
        new = sum(len(r.ids) for r in res) - sum(lens)
        return {"seconds": dt, "steps": s.engine.steps_run - steps0, "tokens": s.engine.tokens_run - tokens0,
                "new_tokens": new, "device_ms": e0.elapsed_time(e1), "preemptions": s.stats()["preemptions"]}

    run.session = gb.Session(model, context_length=w["context"], page_size=16, num_pages=pages, max_batch=w["max_batch"],
                             max_tokens_per_step=4096, prefill_chunk=w["chunk"])
    sampler = ClockSampler(device_uuid())
    sampler.start()
    run(1)                      # the shapes of this workload's steps get their graphs
    r = run(1)                  # the same requests again, timed
    clocks = sampler.summary()
    # host time of a step: the wall time of the run minus the time the device was the one being waited for
    # cannot be read from outside; what can is the wall time per step beside the device-busy time per step
    busy_ms = device_busy_ms(run, 1)
    print(json.dumps({
        "workload": name, "metric": "tokens/s through Session.run_batch (prompt and new tokens; new tokens alone)",
        "value": round(r["tokens"] / r["seconds"], 1), "new_tokens_per_s": round(r["new_tokens"] / r["seconds"], 1),
        "unit": "tokens/s", "seconds": round(r["seconds"], 4), "steps": r["steps"],
        "wall_ms_per_step": round(1000 * r["seconds"] / r["steps"], 4),
        "device_busy_ms_per_step": round(busy_ms["busy_ms"] / busy_ms["steps"], 4),
        "host_ms_per_step": round(busy_ms["host_s"] * 1000 / busy_ms["steps"], 4),
        "preemptions": r["preemptions"], "dtype": "bf16", "data": "synthetic (uniform-random token ids, random weights seed 0)",
        "config": dict({k: v for k, v in w.items() if not isinstance(v, tuple)}, prompt_min=w["prompt"][0],
                       prompt_max=w["prompt"][1], layers=cfg["num_hidden_layers"], vocab=cfg["vocab_size"]),
        "clocks": clocks}))
    return 0


def device_busy_ms(run, seed):
    """Two more runs of the workload.  One under the CUPTI activity trace: the time covered by its kernels
    is the device's busy time.  One with ``Scheduler.step`` timed on the host, the device idle when each step
    begins (a synchronize before it, outside the timed part), so that the time of a step is the host's own
    work (planning, packing, launching, digesting the step before) and holds no waiting for a busy device
    beyond the read of the ids it is about to digest."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    from gesso_b200.engine import scheduler as sched_mod
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        run(seed)
        torch.cuda.synchronize()
    # the union of the kernels' intervals: kernels launched programmatically start while their predecessor
    # still runs, so the sum of their durations would count that time twice
    spans = sorted((e.time_range.start, e.time_range.end) for e in prof.events()
                   if e.device_type == torch.autograd.DeviceType.CUDA)
    busy, cur_end = 0.0, None
    for a, b in spans:
        if cur_end is None or a > cur_end:
            busy += b - a
            cur_end = b
        elif b > cur_end:
            busy += b - cur_end
            cur_end = b
    busy /= 1000.0
    host = {"s": 0.0, "steps": 0}
    real_step = sched_mod.Scheduler.step

    def timed_step(self):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = real_step(self)
        host["s"] += time.perf_counter() - t0
        host["steps"] += 1
        return out

    sched_mod.Scheduler.step = timed_step
    try:
        run(seed)
    finally:
        sched_mod.Scheduler.step = real_step
    return {"busy_ms": busy, "steps": max(host["steps"], 1), "host_s": host["s"]}


def kernel_timeline(batch: int, context: int, page_size: int, layers=None) -> int:
    """Where the time of one decoding step goes: the kernels of one graph-replayed step at ``batch`` and
    ``context`` from the CUPTI activity trace (through ``torch.profiler``), summed by kernel name.  Kernels of a
    step overlap (each is launched while its predecessor drains), so beside a kernel's own duration the table
    gives the time from its start to its successor's start, which adds up to the step."""
    import collections
    import torch
    import gesso_b200 as gb
    from gesso_b200 import ops
    from gesso_b200.engine.batch import StepEntry
    from torch.profiler import ProfilerActivity, profile
    cfg = dict(LFM2_1_2B)
    if layers is not None and layers < cfg["num_hidden_layers"]:
        cfg["num_hidden_layers"] = layers
        cfg["full_attn_idxs"] = [i for i in cfg["full_attn_idxs"] if i < layers]
    model = gb.random_model(cfg, seed=0, dtype="bfloat16", max_positions=context)
    s, prompts, _ = decode_setup(gb, model, batch, context, 16, 8, page_size)
    eng = s.engine
    ids = [f"q{i}" for i in range(batch)]
    for rid, p in zip(ids, prompts):
        eng.admit(rid)
        for c in range(0, len(p), 2048):
            eng.step([StepEntry(rid, p[c:c + 2048], [])])

    def one(k):
        ops.argmax_rows(eng.step([StepEntry(rid, [(7 * k + i) % 1000], [0]) for i, rid in enumerate(ids)]))

    for k in range(8):
        one(k)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for k in range(8, 12):
            one(k)
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
          and "Memcpy" not in e.name and "Memset" not in e.name]
    ev.sort(key=lambda e: e.time_range.start)
    first = [i for i, e in enumerate(ev) if "embed_gather" in e.name]
    step = ev[first[-2]:first[-1]]                      # the last whole step
    t0 = step[0].time_range.start
    agg = collections.OrderedDict()
    for i, e in enumerate(step):
        nxt = step[i + 1].time_range.start if i + 1 < len(step) else e.time_range.end
        a = agg.setdefault(e.name.split("(")[0][:72], [0.0, 0, 0.0])
        a[0] += e.time_range.end - e.time_range.start
        a[1] += 1
        a[2] += nxt - e.time_range.start
    print(f"one decoding step, batch {batch}, context {context}, {cfg['num_hidden_layers']} layers: "
          f"{step[-1].time_range.end - t0:.1f} us, {len(step)} kernels")
    print(f"{'start to next start, us':>24} {'launches':>8} {'each':>7} {'own duration each':>18}  kernel")
    for name, (dur, n, s2s) in sorted(agg.items(), key=lambda kv: -kv[1][2]):
        print(f"{s2s:24.1f} {n:8d} {s2s / n:7.2f} {dur / n:18.2f}  {name}")
    return 0


def reference_arm():
    """The reference is a Julia 1.12 project (Project.toml, no setup.py / pyproject.toml): pip cannot
    install it, no Julia toolchain exists here, and its CUDA extension has no short-convolution
    lowering for LFM2 (ext/GessoCUDAExt.jl:138-157)."""
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference is a Julia project: pip cannot install it offline, no Julia toolchain "
                      "is on this box, and its CUDA extension does not run LFM2"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--workload", default="decode", choices=["decode", "timeline"] + sorted(SERVE),
                    help="decode: the headline (default); serve350m / serve700m: serving-like runs through run_batch; "
                         "timeline: the kernels of one decoding step at --batch and --context")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.workload == "timeline":
        return kernel_timeline(args.batch, args.context, args.page_size, args.layers)
    if args.workload != "decode":
        return serve_workload(args.workload)
    warmup = max(args.warmup, 3)

    import torch
    import gesso_b200 as gb
    from gesso_b200.config import Lfm2Config

    cfg = dict(LFM2_1_2B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers is not None and args.layers < full_layers:
        cfg["num_hidden_layers"] = args.layers
        cfg["full_attn_idxs"] = [i for i in cfg["full_attn_idxs"] if i < args.layers]
    c = Lfm2Config.from_json(cfg)
    n_attn = sum(c.layer_is_attention)
    n_conv = c.num_hidden_layers - n_attn
    model = gb.random_model(cfg, seed=0, dtype="bfloat16", max_positions=args.context)
    pk = peaks()

    sampler = ClockSampler(device_uuid())
    sampler.start()
    ms_step, launches, kv_mid = time_decode(gb, model, args.batch, args.context, args.steps, warmup, args.page_size)
    clocks = sampler.summary()
    value = args.batch * 1000.0 / ms_step

    # bytes a decode step has to read: every weight it uses once + the cache of the live requests
    layer_flops, head_flops = model_flops_per_token(c, n_attn, n_conv)
    weight_bytes = (layer_flops // 2 + head_flops // 2) * 2                 # bf16

    def roofline_of(batch, kv_len, ms):
        kv_bytes = batch * kv_len * n_attn * 2 * c.num_key_value_heads * c.head_dim * 2
        state_bytes = batch * n_conv * (c.conv_L_cache - 1) * c.hidden_size * 4
        achieved = (weight_bytes + kv_bytes + state_bytes) / (ms * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"]}

    roofline = roofline_of(args.batch, kv_mid, ms_step)
    blocks = dict(time_decode.blocks)

    e2e_value, h2d, d2h = time_e2e(gb, model, args.batch, args.context, args.steps, warmup, args.page_size)
    e2e = {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
           "d2h_bytes_per_step": int(d2h)}

    out = {
        "metric": "decode tokens/s (LFM2-1.2B layer sizes, random weights)", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (uniform-random token ids, random weights seed 0)",
        "config": {"model": "LFM2-1.2B-shaped", "layers": c.num_hidden_layers, "layers_of_config": full_layers,
                   "hidden": c.hidden_size, "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
                   "head_dim": c.head_dim, "ff": c.ff_dim, "vocab": c.vocab_size, "conv_taps": c.conv_L_cache,
                   "attention_layers": n_attn, "global_batch": args.batch, "seq_len": args.context,
                   "page_size": args.page_size, "prefill_tokens": args.prefill_tokens,
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (all weights read every step)"},
        "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline, "clocks": clocks, "blocks": blocks,
    }
    if not args.no_points:
        # the other decoding points first, the prefill last: it is the one measurement that runs the device at
        # its power limit, and a decoding point timed right behind it came out 5 to 9 % lower than alone
        pts, roofs = {}, {f"decode_b{args.batch}": roofline}
        for b, ctx in ((1, args.context), (64, args.context), (args.batch, 512), (args.batch, 2048)):
            if ctx > args.context or (b, ctx) == (args.batch, args.context):
                continue
            ms_b, _, kv_b = time_decode(gb, model, b, ctx, min(args.steps, 64), warmup, args.page_size)
            name = f"decode_b{b}" if ctx == args.context else f"decode_b{b}_ctx{ctx}"
            pts[name] = round(b * 1000.0 / ms_b, 1)
            roofs[name] = roofline_of(b, kv_b, ms_b)
        ms_pf = time_prefill(gb, model, args.prefill_tokens, args.page_size)
        T = args.prefill_tokens
        attn_flops = n_attn * 4 * c.num_attention_heads * c.head_dim * (T * (T + 1) // 2)
        pf_flops = T * layer_flops + head_flops + attn_flops
        out["prefill"] = {"value": round(T * 1000.0 / ms_pf, 1), "tokens": T, "ms": round(ms_pf, 3),
                          "frac": round(pf_flops / (ms_pf * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        out["points"] = pts
        out["rooflines"] = {k: v["frac"] for k, v in roofs.items()}
        out["cpu_baseline"] = cpu_baseline()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
