"""Replay of seeded random LFM2 configurations (head sizes 16..128 in steps of 16, any number of heads
and groups, widths and vocabularies that are no power of two, 2..5 taps, attention layers anywhere) under
the four schedules, in both run types, against the plain implementation.  The wide ones reach the paths
a block takes when it walks several tiles of a matrix."""
import random
import shutil

import pytest

import trace_tools as tt

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-4, "bfloat16": 32 * 2.0 ** -9}


def random_config(seed, wide):
    rng = random.Random(seed)
    if wide:
        hd = rng.choice([64, 128])
        H = rng.choice([1024, 1280, 1536, 1792, 2048, 2560, 3072])
        nh = H // hd
        nkv = rng.choice([d for d in (1, 2, 4, 8) if nh % d == 0])
        L, n_layers, attn = rng.choice([2, 3, 4]), 2, [rng.choice([0, 1])]
        ff, V = rng.choice([2560, 3072, 4608, 6912, 8192]), rng.choice([8192, 32000, 65536])
        lengths = [rng.choice([5, 17, 40]) for _ in range(3)]
    else:
        hd = rng.choice([16, 32, 48, 64, 80, 96, 112, 128])
        nkv = rng.choice([1, 2, 3, 4])
        nh = nkv * rng.choice([1, 2, 3, 4, 5, 8])
        if nh * hd > 1536:
            nkv, nh = 1, rng.choice([1, 2, 4])
        H = nh * hd
        L, n_layers = rng.choice([2, 3, 4, 5]), rng.choice([2, 3, 4, 5])
        attn = sorted(rng.sample(range(n_layers), rng.randint(1, n_layers)))
        ff, V = rng.choice([40, 72, 136, 200, 264, 384, 520, 1000]), rng.choice([97, 256, 503, 1000, 4099, 9001])
        lengths = [rng.choice([1, 5, 17, 33, 64, 65, 70, 97, 130]) for _ in range(4)]
    cfg = {"architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2", "vocab_size": V, "hidden_size": H,
           "num_hidden_layers": n_layers, "num_attention_heads": nh, "num_key_value_heads": nkv,
           "full_attn_idxs": attn, "conv_L_cache": L, "conv_bias": rng.random() < 0.3, "block_ff_dim": ff,
           "block_auto_adjust_ff_dim": False, "norm_eps": rng.choice([1e-5, 1e-6]),
           "rope_theta": rng.choice([1e4, 1e6]), "tie_embedding": rng.random() < 0.5}
    return cfg, lengths


@pytest.mark.parametrize("seed,wide", [(0, False), (9, False), (16, False), (19, False), (21, False), (29, False),
                                       (104, True), (111, True), (112, True)])
def test_random_configuration_replays_like_plain(seed, wide, tmp_path):
    import gesso_b200
    from gesso_b200.weights import write_random_model
    from plain_lfm2 import PlainModel
    cfg, lengths = random_config(seed, wide)
    d = str(tmp_path / "model")
    write_random_model(d, cfg, seed, dtype="bfloat16", style="fan_in")
    reqs = tt.make_requests(cfg["vocab_size"], lengths, seed=seed)
    plain = PlainModel(d)
    ref = [plain.logits(t).numpy() for t in reqs]
    del plain
    schedules = {"whole": tt.trace_whole, "tail_decode": tt.trace_tail_decode, "portions": tt.trace_portions,
                 "mixed": lambda r: tt.trace_mixed(r, seed=seed)}
    for dtype in ("float32", "bfloat16"):
        model = gesso_b200.load(d, dtype=dtype, max_positions=256)
        for name, make in schedules.items():
            tb, max_tokens = make(reqs)
            out = str(tmp_path / f"{dtype}_{name}")
            tt.run_in_process(model, tb, max_tokens, out)
            tt.compare_with_plain(tt.read_rows(tb, out, cfg["vocab_size"]), ref, TOL[dtype],
                                  f"seed {seed} {cfg} / {name} / {dtype}")
            shutil.rmtree(out, ignore_errors=True)
        del model
