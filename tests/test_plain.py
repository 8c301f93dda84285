"""The plain implementation checked against identities restated from the reference's own tests,
with negative controls (CPU)."""
import math

import numpy as np
import pytest
import torch

import plain_lfm2 as P

F64 = torch.float64


def test_conv_tap_order_analytic():
    """Ones input, in/out projections of ones, taps [2, -1, 3], norm weight 1, eps 1e-5 gives
    [3, 2, 4, 4] / (1 + 1e-5)^1.5 (test/test_lfm25.jl:79-90)."""
    H = 1
    x = torch.ones(4, H, dtype=F64)
    xn = P.rmsnorm(x, torch.ones(H, dtype=F64), 1e-5)
    out = P.short_conv_mixer(xn, torch.ones(3 * H, H, dtype=F64), torch.tensor([[2.0, -1.0, 3.0]], dtype=F64),
                             torch.ones(H, H, dtype=F64))
    want = torch.tensor([3.0, 2.0, 4.0, 4.0], dtype=F64) / (1 + 1e-5) ** 1.5
    assert torch.allclose(out.flatten(), want, atol=1e-14, rtol=0)
    rev = P.short_conv_mixer(xn, torch.ones(3 * H, H, dtype=F64), torch.tensor([[3.0, -1.0, 2.0]], dtype=F64),
                             torch.ones(H, H, dtype=F64))
    assert float((rev - out).abs().max()) > 1e-3          # reversed taps must show


def test_fir_equals_causal_convolution():
    g = torch.Generator().manual_seed(0)
    T, H, L = 23, 7, 4
    bcx = torch.randn(T, 3 * H, generator=g, dtype=F64)
    taps = torch.randn(H, L, generator=g, dtype=F64)
    got = P.short_conv_fir(bcx, taps)
    bx = bcx[:, :H] * bcx[:, 2 * H:]
    pad = torch.cat([torch.zeros(L - 1, H, dtype=F64), bx])
    want = torch.stack([sum(pad[t + p] * taps[:, p] for p in range(L)) for t in range(T)]) * bcx[:, H:2 * H]
    assert torch.allclose(got, want, atol=1e-12)
    # swapping the B/C/X thirds is not the same function
    swapped = torch.cat([bcx[:, H:2 * H], bcx[:, :H], bcx[:, 2 * H:]], dim=1)
    assert float((P.short_conv_fir(swapped, taps) - got).abs().max()) > 1e-3


def test_rmsnorm_formula():
    x = torch.tensor([[3.0, 4.0]], dtype=F64)
    w = torch.tensor([2.0, 0.5], dtype=F64)
    r = math.sqrt((9 + 16) / 2 + 1e-6)
    assert torch.allclose(P.rmsnorm(x, w, 1e-6), torch.tensor([[3 / r * 2, 4 / r * 0.5]], dtype=F64), atol=1e-14)


def test_rope_half_split_and_relative():
    d, theta = 8, 10000.0
    x = torch.randn(5, 2, d, dtype=F64)
    y = P.rope(x, [0, 1, 2, 3, 4], theta)
    assert torch.allclose(y[0], x[0])                                  # position 0 is the identity
    # pair (i, i + d/2) rotates by pos * theta^(-2i/d)
    i, pos = 1, 3
    ang = pos * theta ** (-2 * i / d)
    a, b = x[pos, 0, i], x[pos, 0, i + d // 2]
    assert abs(float(y[pos, 0, i]) - float(a * math.cos(ang) - b * math.sin(ang))) < 1e-12
    assert abs(float(y[pos, 0, i + d // 2]) - float(a * math.sin(ang) + b * math.cos(ang))) < 1e-12
    # scores depend on the distance only
    q, k = torch.randn(1, 1, d, dtype=F64), torch.randn(1, 1, d, dtype=F64)
    s1 = (P.rope(q, [7], theta) * P.rope(k, [4], theta)).sum()
    s2 = (P.rope(q, [13], theta) * P.rope(k, [10], theta)).sum()
    assert abs(float(s1 - s2)) < 1e-12
    # the interleaved layout would differ
    inter = x.clone().reshape(5, 2, d // 2, 2).transpose(-1, -2).reshape(5, 2, d)
    assert float((P.rope(inter, [0, 1, 2, 3, 4], theta) - y).abs().max()) > 1e-3


def test_attention_causal_gqa_window():
    g = torch.Generator().manual_seed(1)
    T, nh, nkv, d = 9, 4, 2, 6
    q, k, v = (torch.randn(T, n, d, generator=g, dtype=F64) for n in (nh, nkv, nkv))
    o = P.causal_attention(q, k, v)
    assert torch.allclose(o[0, 0], v[0, 0]) and torch.allclose(o[0, 3], v[0, 1])     # first row sees one key; head 3 -> kv 1
    # by hand for one (row, head)
    t, h = 5, 2
    s = torch.tensor([float(q[t, h] @ k[u, 1]) / math.sqrt(d) for u in range(t + 1)], dtype=F64)
    p = torch.softmax(s, 0)
    assert torch.allclose(o[t, h], (p[:, None] * v[:t + 1, 1]).sum(0), atol=1e-12)
    # future keys do not matter; a window of 3 reads exactly keys t-2..t
    k2 = k.clone()
    k2[6:] += 5.0
    assert torch.allclose(P.causal_attention(q, k2, v)[:6], o[:6])
    ow = P.causal_attention(q, k, v, window=3)
    s = torch.tensor([float(q[t, h] @ k[u, 1]) / math.sqrt(d) for u in range(t - 2, t + 1)], dtype=F64)
    assert torch.allclose(ow[t, h], (torch.softmax(s, 0)[:, None] * v[t - 2:t + 1, 1]).sum(0), atol=1e-12)
    assert torch.allclose(ow[:3], o[:3])


def test_swiglu_formula():
    x = torch.tensor([[1.0, -2.0]], dtype=F64)
    wg = torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=F64)
    wu = torch.tensor([[2.0, 0.0], [0.0, 3.0]], dtype=F64)
    wd = torch.tensor([[1.0, 1.0]], dtype=F64)
    g = x @ wg.T
    want = ((g / (1 + torch.exp(-g))) * (x @ wu.T)) @ wd.T
    assert torch.allclose(P.swiglu_ffn(x, wg, wu, wd), want)
    assert abs(float(want) - (1 / (1 + math.exp(-1)) * 2 + (-2 / (1 + math.exp(2))) * -6)) < 1e-12


def test_model_is_causal_and_deterministic(plain_models):
    pm = plain_models["b"]
    ids = [3, 99, 250, 7, 7, 401, 12, 88, 5, 300, 2]
    full = pm.logits(ids)
    assert full.shape == (len(ids), 503) and torch.isfinite(full).all()
    assert torch.allclose(pm.logits(ids[:6]), full[:6], atol=1e-12)     # a prefix gives the same logits
    assert torch.equal(pm.logits(ids), full)
    out = pm.greedy(ids[:4], 3)
    assert out[:4] == ids[:4] and out[4] == int(torch.argmax(pm.logits(ids[:4])[-1]))


def test_model_negative_controls(plain_models, model_dirs):
    """Faults the engine could make must move the plain logits by far more than any tolerance."""
    pm = plain_models["a"]
    ids = list(range(40, 60))
    base = pm.logits(ids)
    w = pm.w
    name = "model.layers.0.conv.conv.weight"
    keep = w[name].clone()
    w[name] = keep.flip(-1)                              # reversed taps (test/test_lfm25.jl:188-194)
    assert float((pm.logits(ids) - base).abs().max()) > 1e-3
    w[name] = keep
    name = "model.layers.1.self_attn.q_layernorm.weight"
    keep = w[name].clone()
    w[name] = keep.flip(0)                               # q-norm weight applied to the wrong features
    assert float((pm.logits(ids) - base).abs().max()) > 1e-3
    w[name] = keep
    theta = pm.theta
    pm.theta = theta * 2                                 # wrong rotary base
    assert float((pm.logits(ids) - base).abs().max()) > 1e-3
    pm.theta = theta
    assert torch.equal(pm.logits(ids), base)


def test_effective_ff_and_layers():
    assert P.effective_ff({"block_ff_dim": 12288, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256}) == 8192
    assert P.effective_ff({"block_ff_dim": 384, "block_auto_adjust_ff_dim": True, "block_multiple_of": 32}) == 256
    assert P.effective_ff({"block_ff_dim": 128}) == 128
    assert P.layer_is_attention({"num_hidden_layers": 4, "full_attn_idxs": [1, 3]}) == [False, True, False, True]


def test_plain_sampler_rules():
    s1, s2 = P.PlainSampler(0.8, 0.9, 5), P.PlainSampler(0.8, 0.9, 5)
    row = torch.randn(300, generator=torch.Generator().manual_seed(2)).tolist()
    assert [s1.sample(row) for _ in range(20)] == [s2.sample(row) for _ in range(20)]     # same seed, same ids
    assert P.PlainSampler(1e-3, 1.0, 0).sample(row) == int(np.argmax(row))              # low temperature -> argmax
    # nucleus keeps exactly the top set (test/test_sampling.jl:64-69)
    row = [-30.0] * 50
    row[4], row[9], row[30] = 2.0, 1.5, 1.0
    seen = {P.PlainSampler(1.0, 0.7, s).sample(row) for s in range(60)}
    assert seen == {4, 9}
    # the first unit float of seed 0 of splitmix64
    assert abs(P.PlainSampler(1.0, 1.0, 0).unit() - 0xE220A8397B1DCDAF / 2.0 ** 64) < 2.0 ** -52
