"""Command line: ``python -m gesso_b200 <command> ...``.

The reference's launcher takes ``--gguf PATH --n-ctx N --check`` and refuses unknown flags
(scripts/gesso-serve.jl:61-84); its request fields are ``temperature``, ``top_p``, ``seed``,
``max_tokens``, ``stop`` (docs/serving.md:95-106).  The same names are used here where this engine
has the same thing; the model comes from a folder (``--model``) instead of a GGUF file.

    generate     --model DIR | --random-weights SEED --config FILE
                 --prompt-ids 1,2,3 [--max-new-tokens N] [--temperature T] [--top-p P]
                 [--seed S] [--stop-ids ..] [--eos-ids ..] [--dtype bfloat16|float32] [--n-ctx N]
                 [--page-size 16] [--num-pages N] [--max-batch B] [--prefill-chunk C]
    init-random  --config FILE --seed S --out DIR      write a model folder with random weights
    describe     --model DIR                           print the typed configuration and the layers
    replay       --model DIR --dtype D --out DIR --max-tokens N   steps from standard input (bin/trace_run)
    bench        [options of bench.py]                 the throughput measurements (bench.py at the root of the tree)
    check                                              build the kernels and run a tiny generation
"""
from __future__ import annotations

import argparse
import json
import sys


def _ids(text: str):
    return [int(x) for x in text.replace(",", " ").split()]


def _parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="gesso_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="generate tokens for one or more prompts")
    g.add_argument("--model", help="folder with config.json and model.safetensors")
    g.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                   help="instead of --model: random weights drawn from this seed for the configuration of --config")
    g.add_argument("--config", help="config.json for --random-weights")
    g.add_argument("--prompt-ids", action="append", default=[], help="token ids, comma or space separated; repeatable")
    g.add_argument("--prompt-file", help="one prompt of token ids per line")
    g.add_argument("--max-new-tokens", type=int, default=8)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--stop-ids", default="")
    g.add_argument("--eos-ids", default=None)
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--n-ctx", type=int, default=4096)
    g.add_argument("--page-size", type=int, default=16)
    g.add_argument("--num-pages", type=int, default=None)
    g.add_argument("--max-batch", type=int, default=8)
    g.add_argument("--prefill-chunk", type=int, default=512)
    r = sub.add_parser("init-random", help="write a model folder with random weights")
    r.add_argument("--config", required=True)
    r.add_argument("--seed", type=int, required=True)
    r.add_argument("--out", required=True)
    r.add_argument("--weights-dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.add_argument("--std", type=float, default=0.02)
    d = sub.add_parser("describe", help="print the typed configuration")
    d.add_argument("--model", required=True)
    t = sub.add_parser("replay", help="feed given token ids step by step and write logits (steps on standard input)")
    t.add_argument("--model", required=True)
    t.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    t.add_argument("--out", required=True)
    t.add_argument("--max-tokens", type=int, required=True)
    t.add_argument("--page-size", type=int, default=16)
    sub.add_parser("bench", help="run bench.py with the options that follow", add_help=False)
    sub.add_parser("check", help="build the kernels and run a tiny generation on cuda:0")
    return ap


def _replay(args) -> int:
    """The same as ``bin/trace_run``: the engine's own step function fed from standard input."""
    import gesso_b200
    from .engine import trace
    unit = max(trace.PAGE_ROUND, args.page_size)
    max_tokens = unit * ((args.max_tokens + unit - 1) // unit)
    model = gesso_b200.load(args.model, dtype=args.dtype, max_positions=max_tokens)
    trace.replay(trace.make_engine(model, max_tokens, page_size=args.page_size), sys.stdin, args.out)
    return 0


def _bench(argv) -> int:
    import os
    import subprocess
    script = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py")
    if not os.path.isfile(script):
        print(f"bench: {script} not found (bench.py lives at the root of the source tree)", file=sys.stderr)
        return 2
    return subprocess.call([sys.executable, script] + list(argv))


def _check() -> int:
    """Build the kernel library and the host library, then generate with a small random model in float32
    and bfloat16 and hold the engine to itself: the greedy ids that came out token by token must be the
    most likely ones (bfloat16: within rounding of them) when the whole sequence is run again in one step,
    as the reference checks its decoding against a re-run prefill (test/test_lfm25.jl:172-187)."""
    import tempfile
    import numpy as np
    import gesso_b200
    from .csrc import build as kernel_build, hostlib
    from .weights.random_init import write_random_model
    kernel_build.build(verbose=True)
    hostlib.build()
    cfg = {"architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2", "vocab_size": 320, "hidden_size": 128,
           "num_hidden_layers": 3, "num_attention_heads": 4, "num_key_value_heads": 2, "full_attn_idxs": [1],
           "conv_L_cache": 3, "conv_bias": False, "block_ff_dim": 256, "block_auto_adjust_ff_dim": False,
           "norm_eps": 1e-5, "rope_theta": 10000.0, "tie_embedding": True}
    prompts = [[5, 17, 3, 250, 9, 77, 41], [1] * 19, [300]]
    with tempfile.TemporaryDirectory() as d:
        write_random_model(d, cfg, 0, style="fan_in")
        for dtype, slack in (("float32", 1e-4), ("bfloat16", 0.0625)):
            model = gesso_b200.load(d, dtype=dtype, max_positions=64)
            s = gesso_b200.Session(model, context_length=64, max_batch=4)
            res = s.run_batch([gesso_b200.BatchRequest(p, max_new_tokens=6) for p in prompts])
            for p, r in zip(prompts, res):
                if r.status != "complete":
                    print(f"check: {dtype}: request ended as {r.status}: {r.error}", file=sys.stderr)
                    return 1
                whole = s.prefill(r.ids[:-1])
                for k in range(len(p), len(r.ids)):
                    row = whole[k - 1]
                    if float(row.max() - row[r.ids[k]]) > slack * max(1.0, float(np.abs(row).max())):
                        print(f"check: {dtype}: token {k} of {r.ids} is not the most likely one of a whole run",
                              file=sys.stderr)
                        return 1
            print(f"check: {dtype} ok")
    print("ok")
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "bench":
        return _bench(argv[1:])            # bench.py parses (and refuses) its own options
    args = _parser().parse_args(argv)      # an unknown flag prints the usage and exits with 2
    if args.command == "replay":
        return _replay(args)
    if args.command == "init-random":
        from .config.registry import parse_strict_json
        from .weights.random_init import write_random_model
        with open(args.config) as f:
            cfg = parse_strict_json(f.read(), args.config)
        write_random_model(args.out, cfg, args.seed, dtype=args.weights_dtype, std=args.std)
        print(args.out)
        return 0
    if args.command == "describe":
        from .config.registry import spec_from_dir
        spec = spec_from_dir(args.model)
        print(json.dumps({"architecture": spec.architecture, "config": getattr(spec.source, "__dict__", None),
                          "layers": [b.mixer.kind for b in spec.blocks]}, indent=1, default=str))
        return 0
    if args.command == "check":
        return _check()
    # generate
    import gesso_b200
    from .engine.session import BatchRequest, Session
    prompts = [_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [_ids(line) for line in f if line.strip()]
    if not prompts:
        print("generate: no prompt given (--prompt-ids or --prompt-file)", file=sys.stderr)
        return 2
    if (args.model is None) == (args.random_weights is None):
        print("generate: give either --model DIR or --random-weights SEED --config FILE", file=sys.stderr)
        return 2
    if args.model is not None:
        model = gesso_b200.load(args.model, dtype=args.dtype, max_positions=args.n_ctx)
    else:
        if not args.config:
            print("generate: --random-weights needs --config FILE", file=sys.stderr)
            return 2
        from .config.registry import parse_strict_json
        with open(args.config) as f:
            cfg = parse_strict_json(f.read(), args.config)
        model = gesso_b200.random_model(cfg, seed=args.random_weights, dtype=args.dtype, max_positions=args.n_ctx)
    s = Session(model, context_length=args.n_ctx, page_size=args.page_size, num_pages=args.num_pages,
                max_batch=args.max_batch, prefill_chunk=args.prefill_chunk)
    eos = None if args.eos_ids is None else _ids(args.eos_ids)
    res = s.run_batch([BatchRequest(p, args.max_new_tokens, args.temperature, args.top_p, args.seed + i,
                                    _ids(args.stop_ids), eos) for i, p in enumerate(prompts)])
    for r in res:
        print(json.dumps({"ids": r.ids, "status": r.status, "error": None if r.error is None else str(r.error)}))
    return 0 if all(r.status != "failed" for r in res) else 1


if __name__ == "__main__":
    sys.exit(main())
