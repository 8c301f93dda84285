"""Configuration and registry (CPU)."""
import copy

import pytest

import configs
from gesso_b200.config import (Lfm2Config, PartSpec, effective_ff_dim, known_architectures,
                               parse_strict_json, register_architecture, spec_from_config,
                               unregister_architecture)
from gesso_b200.errors import ErrorCode, GessoError


def test_ff_dim_rule():
    # the sizes the model family publishes: 2/3 rule, then rounding up to a multiple
    assert effective_ff_dim(12288, True, 256, None) == 8192
    assert effective_ff_dim(6656, True, 256, None) == 4608
    assert effective_ff_dim(10240, True, 256, None) == 6912
    assert effective_ff_dim(384, True, 32, None) == 256
    assert effective_ff_dim(128, False, 256, None) == 128
    assert effective_ff_dim(12288, True, 256, 1.0) == 8192


def test_tiny_configs_parse_and_differ():
    a, b, c = (Lfm2Config.from_json(x) for x in (configs.TINY_A, configs.TINY_B, configs.TINY_C))
    assert a.layer_is_attention == (False, True, False, True)
    assert b.layer_is_attention == (True, False, True, False, False, True)
    assert (a.head_dim, b.head_dim, c.head_dim) == (16, 24, 32)
    assert (a.ff_dim, b.ff_dim, c.ff_dim) == (128, 256, 200)
    assert (a.tie_embedding, b.tie_embedding, c.tie_embedding) == (True, False, True)
    for f in ("vocab_size", "hidden_size", "num_hidden_layers", "num_key_value_heads", "conv_L_cache",
              "rope_theta", "ff_dim"):
        assert len({getattr(x, f) for x in (a, b, c)}) == 3, f
    assert a.norm_eps != b.norm_eps and a.conv_bias != b.conv_bias


def test_spec_names_layers_by_part():
    spec = spec_from_config(configs.TINY_B)
    kinds = [b.mixer.kind for b in spec.blocks]
    assert kinds == ["gqa_attention", "short_conv", "gqa_attention", "short_conv", "short_conv", "gqa_attention"]
    assert spec.blocks[0].mixer["n_kv_heads"] == 1 and spec.blocks[1].mixer["kernel"] == 4
    assert [e.layer for e in spec.schedule] == list(range(6))
    assert spec.external_names("layers.1.mixer.conv.weight")[0] == "model.layers.1.conv.conv.weight"
    assert "blk.1.shortconv.conv.weight" in spec.external_names("layers.1.mixer.conv.weight")


def _bad(mutate, needle):
    cfg = copy.deepcopy(configs.TINY_A)
    mutate(cfg)
    with pytest.raises(GessoError) as e:
        Lfm2Config.from_json(cfg)
    assert e.value.code == ErrorCode.INVALID_PLAN
    assert needle in str(e.value), str(e.value)


def test_refusals_name_the_key():
    _bad(lambda c: c.update(sliding_window=128), "sliding_window")            # unknown key
    _bad(lambda c: c.pop("vocab_size"), "vocab_size")                         # missing key
    _bad(lambda c: c.update(layer_types=["conv"] * 3), "layer_types")         # wrong length
    _bad(lambda c: c.update(layer_types=["conv", "attn", "conv", "conv"]), "layer_types[1]")
    _bad(lambda c: c.update(conv_L_cache=1), "conv_L_cache")                  # one tap keeps no history
    _bad(lambda c: c.update(head_dim=32), "head_dim")                         # nh*hd != hidden
    _bad(lambda c: c.update(num_key_value_heads=3), "num_key_value_heads")
    _bad(lambda c: c.update(full_attn_idxs=[0, 2]), "disagree")
    _bad(lambda c: c.update(intermediate_size=64), "intermediate_size")
    _bad(lambda c: c.update(norm_eps=0), "norm_eps")
    _bad(lambda c: c.update(tie_embedding=True, tie_word_embeddings=False), "disagree")
    _bad(lambda c: (c.pop("layer_types")), "layer_types")


def test_full_attn_idxs_equals_layer_types():
    cfg = copy.deepcopy(configs.TINY_A)
    cfg.pop("layer_types")
    cfg["full_attn_idxs"] = [1, 3]
    assert Lfm2Config.from_json(cfg) == Lfm2Config.from_json(configs.TINY_A)


def test_to_json_round_trip():
    for cfg in (configs.TINY_A, configs.TINY_B, configs.TINY_C):
        c = Lfm2Config.from_json(cfg)
        assert Lfm2Config.from_json(c.to_json()) == c


def test_registry():
    assert "Lfm2ForCausalLM" in known_architectures()
    with pytest.raises(GessoError) as e:
        spec_from_config({"architectures": ["NoSuchModel"]})
    assert "Lfm2ForCausalLM" in str(e.value)          # the refusal lists what is known
    assert spec_from_config({k: v for k, v in configs.TINY_A.items() if k != "architectures"}).architecture \
        == "Lfm2ForCausalLM"                          # model_type is the fallback key
    with pytest.raises(GessoError):
        spec_from_config({"hidden_size": 4})
    marker = object()
    register_architecture("ToyArch", lambda cfg: marker)
    try:
        assert spec_from_config({"architectures": ["ToyArch"]}) is marker
        with pytest.raises(GessoError):
            register_architecture("ToyArch", lambda cfg: None)
    finally:
        unregister_architecture("ToyArch")


def test_strict_json_rejects_duplicates():
    with pytest.raises(GessoError):
        parse_strict_json('{"a": 1, "a": 2}')
    with pytest.raises(GessoError):
        parse_strict_json('[1, 2]')
    assert parse_strict_json('{"a": {"b": 1}}') == {"a": {"b": 1}}
