"""Replay at the layer widths of LFM2-1.2B (hidden 2048, 32 heads / 8 kv heads of 64, feed-forward
8192), LFM2-350M (1024, 16 / 8, 4608) and LFM2-700M (1536, 24 / 8, 6912), vocabulary 65536, 3 taps;
three layers each: conv, attention, conv; against the plain implementation.

The tiny configurations never reach the kernels that serve these widths: the tensor-memory matrix
product and flash attention of steps with a thousand tokens and more, the skinny product with its
inner size split over blocks (8192), the 32-way argmax scan.  One long request is replayed whole,
with its last 32 tokens one by one, in portions, and beside other requests that come and go."""
import numpy as np
import pytest

import trace_tools as tt

pytestmark = pytest.mark.gpu

def wide_config(hidden, heads, block_ff):
    return {
        "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
        "vocab_size": 65536, "hidden_size": hidden, "num_hidden_layers": 3,
        "num_attention_heads": heads, "num_key_value_heads": 8, "full_attn_idxs": [1],
        "conv_L_cache": 3, "conv_bias": False, "block_ff_dim": block_ff, "block_auto_adjust_ff_dim": True,
        "block_multiple_of": 256, "norm_eps": 1e-5, "rope_theta": 1000000.0, "tie_embedding": True,
    }


WIDE = {"1.2B": wide_config(2048, 32, 12288), "350M": wide_config(1024, 16, 6656), "700M": wide_config(1536, 24, 10240)}
VOCAB = 65536
TOL = {"float32": 1e-4, "bfloat16": 32 * 2.0 ** -9}
LONG, SIDE, LATE = 1100, 300, 256
# places of the long request whose logits are compared: the first tokens, borders of pages, of
# 64-token tiles and of 128-key blocks, the thousand-token border, and the last 32
PLACES = sorted(set([0, 1, 2, 15, 16, 63, 64, 127, 128, 129, 511, 512, 699, 700, 701, 1023, 1024, 1034]
                    + list(range(LONG - 32, LONG))))


@pytest.fixture(scope="module", params=["1.2B", "350M", "700M"])
def wide(request, tmp_path_factory):
    from gesso_b200.weights import write_random_model
    from plain_lfm2 import PlainModel
    d = str(tmp_path_factory.mktemp("model_wide"))
    write_random_model(d, WIDE[request.param], 5, dtype="bfloat16", style="fan_in")
    reqs = tt.make_requests(VOCAB, [LONG, SIDE, LATE], seed=77)
    plain = PlainModel(d)
    side_places = [0, 149, 150, 151, SIDE - 1]
    late_places = [0, 99, 100, LATE - 1]
    ref = {0: dict(zip(PLACES, plain.logits(reqs[0], PLACES).numpy())),
           1: dict(zip(side_places, plain.logits(reqs[1], side_places).numpy())),
           2: dict(zip(late_places, plain.logits(reqs[2], late_places).numpy()))}
    del plain
    return d, reqs, ref


@pytest.fixture(scope="module")
def loaded(wide):
    import gesso_b200
    cache = {}

    def get(dtype):
        if dtype not in cache:
            cache.clear()                       # one copy of the weights on the device at a time
            cache[dtype] = gesso_b200.load(wide[0], dtype=dtype, max_positions=1280)
        return cache[dtype]
    return get


def pieces(tb, rid, tokens, start, sizes, want_of):
    """Steps of one request alone: portions of the given sizes from ``start``."""
    p = start
    for n in sizes:
        tb.add_step([(rid, tokens[p:p + n], p, want_of(p, n))])
        p += n
    return p


def wanted(places):
    s = set(places)
    return lambda p, n: [i for i in range(n) if p + i in s]


def build(schedule, reqs):
    A, B, C = reqs
    tb = tt.TraceBuilder()
    wa = wanted(PLACES)
    if schedule == "whole":
        tb.add_step([(0, A, 0, wa(0, LONG))], end=[0])
        return tb, tt.round_up(LONG)
    if schedule == "tail_decode":
        pieces(tb, 0, A, 0, [LONG - 32] + [1] * 32, wa)
        tb.steps[-1]["end"] = ["r0"]
        return tb, tt.round_up(LONG)
    if schedule == "portions":
        pieces(tb, 0, A, 0, [700, 2, 333, 33, 2, 30], wa)
        tb.steps[-1]["end"] = ["r0"]
        return tb, tt.round_up(LONG)
    # mixed: portions of the long request beside the side request's portions and single tokens; the
    # side request ends, a late one takes over its pages while the long one decodes
    wb, wc = wanted([0, 149, 150, 151, SIDE - 1]), wanted([0, 99, 100, LATE - 1])
    tb.add_step([(0, A[:600], 0, wa(0, 600)), (1, B[:150], 0, wb(0, 150))])
    tb.add_step([(1, B[150:152], 150, wb(150, 2)), (0, A[600:1050], 600, wa(600, 450))])
    tb.add_step([(0, A[1050:1051], 1050, wa(1050, 1)), (1, B[152:], 152, wb(152, SIDE - 152))], end=[1])
    tb.add_step([(2, C[:100], 0, wc(0, 100)), (0, A[1051:1052], 1051, wa(1051, 1))])
    p, q = 1052, 100
    while p < LONG:
        entries, end = [(0, A[p:p + 1], p, wa(p, 1))], []
        if q < LATE:
            n = min(7 if p % 2 else 1, LATE - q)
            entries.insert(p % 2, (2, C[q:q + n], q, wc(q, n)))
            q += n
            if q == LATE:
                end.append(2)
        p += 1
        if p == LONG:
            end.append(0)
        tb.add_step(entries, end=end)
    assert q == LATE
    return tb, tt.round_up(LONG) + tt.round_up(SIDE)      # the late request fits only in the side one's pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", ["whole", "tail_decode", "portions", "mixed"])
def test_full_width_replay(schedule, dtype, wide, loaded, tmp_path):
    d, reqs, ref = wide
    tb, max_tokens = build(schedule, reqs)
    eng = tt.run_in_process(loaded(dtype), tb, max_tokens, str(tmp_path))
    rows = tt.read_rows(tb, str(tmp_path), VOCAB)
    want = {(rid, pos) for rid in ((0, 1, 2) if schedule == "mixed" else (0,)) for pos in ref[rid]}
    assert set(rows) == want
    worst = 0.0
    for (rid, pos), got in sorted(rows.items()):
        r = ref[rid][pos]
        scale = max(1.0, float(np.abs(r).max()))
        err = float(np.abs(got.astype(np.float64) - r).max())
        assert np.isfinite(got).all() and err <= TOL[dtype] * scale, \
            f"{schedule}/{dtype}: request {rid} position {pos}: max error {err:.3e} > {TOL[dtype]:.1e} * {scale:.2f}"
        worst = max(worst, err / scale)
    print(f"full width {schedule}/{dtype}: worst {worst:.3e}")


@pytest.mark.parametrize("schedule", ["portions", "mixed"])
def test_full_width_replay_few_row_product(schedule, wide, loaded, tmp_path, monkeypatch):
    """The same replays with the optional few-row tcgen05 product serving every matrix of the steps of
    17 .. 128 tokens (portions of 33, 30 and 100 tokens, 150 + ... mixed steps)."""
    from gesso_b200 import ops
    monkeypatch.setattr(ops, "TC_FEW", True)
    monkeypatch.setattr(ops, "TC_FEW_MIN_BYTES", 0)
    test_full_width_replay(schedule, "bfloat16", wide, loaded, tmp_path)
    ops.check_tc_status()
