"""Weight container, by-name binding and the random-weights mode (CPU)."""
import json
import os
import struct

import pytest
import torch

import configs
from gesso_b200.config import spec_from_config
from gesso_b200.errors import GessoError
from gesso_b200.weights import (bind_tensors, load_model_tensors, model_param_decls, random_tensors,
                                read_model_tensors, read_safetensors_file, write_random_model,
                                write_safetensors_file)


def test_round_trip_keeps_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
         "d": torch.randn(2, 2).to(torch.float16)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors_file(p, t)
    back = read_safetensors_file(p)
    assert set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k])


def _write_raw(path, header: dict, payload: bytes, hdr_len=None):
    text = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text) if hdr_len is None else hdr_len))
        f.write(text)
        f.write(payload)


@pytest.mark.parametrize("case", ["truncated", "dtype", "span", "overlap", "trailing", "gap", "dup", "hdrlen"])
def test_malformed_files_are_refused(tmp_path, case):
    p = str(tmp_path / "m.safetensors")
    ok = {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}
    if case == "truncated":
        open(p, "wb").write(b"\x01\x02")
    elif case == "dtype":
        _write_raw(p, {"a": dict(ok, dtype="F8_E4M3")}, b"\0" * 8)
    elif case == "span":
        _write_raw(p, {"a": dict(ok, shape=[3])}, b"\0" * 8)
    elif case == "overlap":
        _write_raw(p, {"a": ok, "b": dict(ok, data_offsets=[4, 12])}, b"\0" * 12)
    elif case == "trailing":
        _write_raw(p, {"a": ok}, b"\0" * 12)
    elif case == "gap":
        _write_raw(p, {"a": ok, "b": dict(ok, data_offsets=[12, 20])}, b"\0" * 20)
    elif case == "dup":
        text = b'{"a": {"dtype":"F32","shape":[2],"data_offsets":[0,8]}, "a": {"dtype":"F32","shape":[2],"data_offsets":[0,8]}}'
        with open(p, "wb") as f:
            f.write(struct.pack("<Q", len(text)) + text + b"\0" * 8)
    elif case == "hdrlen":
        _write_raw(p, {"a": ok}, b"\0" * 8, hdr_len=10 ** 9)
    with pytest.raises(GessoError):
        read_safetensors_file(p)


def test_random_model_folder_loads(tmp_path):
    d = str(tmp_path / "m")
    spec = write_random_model(d, configs.TINY_B, seed=1)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    tensors, decls = load_model_tensors(d, spec)
    assert set(tensors) == set(decls)
    assert tensors["embedding.weight"].dtype == torch.bfloat16            # matrices are kept in bfloat16
    assert tensors["final_norm.weight"].dtype == torch.float32            # a tensor stored in 32 bit stays so
    assert tensors["layers.1.mixer.conv.weight"].shape == (96, 4)
    assert "lm_head.weight" in tensors and "layers.1.mixer.in_proj.bias" in tensors
    # same seed, same weights; another seed, other weights
    again = random_tensors(spec, 1)
    assert all(torch.equal(again[k], tensors[k]) for k in tensors)
    assert not torch.equal(random_tensors(spec, 2)["embedding.weight"], tensors["embedding.weight"])
    # N(0, 0.02) and norm weights 1
    w = tensors["layers.0.mixer.q_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.004 and torch.all(tensors["final_norm.weight"] == 1)


def test_one_error_lists_missing_unexpected_and_misshaped():
    spec = spec_from_config(configs.TINY_A)
    t = {spec.external_names(k)[0]: v for k, v in random_tensors(spec, 0).items()}
    del t["model.layers.0.conv.in_proj.weight"]
    del t["model.embedding_norm.weight"]
    t["model.layers.9.bogus.weight"] = torch.zeros(1)
    t["model.layers.1.self_attn.q_proj.weight"] = torch.zeros(64, 32, dtype=torch.bfloat16)
    with pytest.raises(GessoError) as e:
        bind_tensors(spec, t)
    msg = str(e.value)
    assert "model.layers.0.conv.in_proj.weight" in msg and "model.embedding_norm.weight" in msg
    assert "model.layers.9.bogus.weight" in msg
    assert "model.layers.1.self_attn.q_proj.weight: expected (64, 64), found (64, 32)" in msg


def test_aliases_ignorable_and_tied_head():
    spec = spec_from_config(configs.TINY_A)
    tensors = random_tensors(spec, 0)
    # the reference's GGUF-style names are accepted as aliases
    t = {spec.external_names(k)[-1]: v for k, v in tensors.items()}
    assert "blk.0.shortconv.conv.weight" in t and "token_embd_norm.weight" in t
    bound = bind_tensors(spec, t)
    assert torch.equal(bound["layers.0.mixer.conv.weight"], tensors["layers.0.mixer.conv.weight"])
    # conv taps may carry the unit axis of a depthwise convolution
    t2 = dict(t)
    t2["blk.0.shortconv.conv.weight"] = tensors["layers.0.mixer.conv.weight"].reshape(64, 1, 3)
    assert bind_tensors(spec, t2)["layers.0.mixer.conv.weight"].shape == (64, 3)
    # rotary inv_freq buffers are ignored; a tied head that equals the embedding is accepted
    t3 = dict(t)
    t3["model.layers.1.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    t3["output.weight"] = tensors["embedding.weight"].clone()
    bind_tensors(spec, t3)
    t3["output.weight"] = tensors["embedding.weight"] + 1
    with pytest.raises(GessoError) as e:
        bind_tensors(spec, t3)
    assert "tied" in str(e.value)


def test_untied_model_needs_its_head():
    spec = spec_from_config(configs.TINY_B)
    t = {spec.external_names(k)[0]: v for k, v in random_tensors(spec, 0).items()}
    del t["lm_head.weight"]
    with pytest.raises(GessoError) as e:
        bind_tensors(spec, t)
    assert "lm_head.weight" in str(e.value)


def test_sharded_folder(tmp_path):
    spec = spec_from_config(configs.TINY_A)
    t = {spec.external_names(k)[0]: v for k, v in random_tensors(spec, 0).items()}
    names = sorted(t)
    half = len(names) // 2
    write_safetensors_file(str(tmp_path / "s1.safetensors"), {n: t[n] for n in names[:half]})
    write_safetensors_file(str(tmp_path / "s2.safetensors"), {n: t[n] for n in names[half:]})
    idx = {"weight_map": {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(idx))
    back = read_model_tensors(str(tmp_path))
    assert set(back) == set(t) and all(torch.equal(back[n], t[n]) for n in t)
    assert len(model_param_decls(spec)) == len(t)
