"""A plain, slow LFM2: whole sequences, no cache, one function per part, float64 on the CPU.

This is the oracle of the test-suite.  It shares no code with ``gesso_b200``: it reads
``config.json`` and ``model.safetensors`` itself and restates every formula from the reference's
source.  The reference is a Julia project and no Julia toolchain exists on the machines these
tests run on, so the reference's own model code cannot be imported or compiled here: this file
rests on the reference's formulas (cited per function as file:line of the reference tree), plus
the analytic identity of its conv test (test/test_lfm25.jl:79-90) that ``test_plain.py`` checks.

Arithmetic: weights are taken as stored (bfloat16/float32 values) and everything is computed in
float64, which is at least as wide as the reference's mix of storage-type products and Float64
statistics (src/Operators/cpu.jl:296-300, 359-369; src/Inference/Inference.jl:1419-1425).
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch

F64 = torch.float64


# ---- reading the model folder (own reader, no engine code) -------------------------------------
def read_safetensors(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b0, b1 = meta["data_offsets"]
        raw = np.frombuffer(data, dtype=np.uint8, count=b1 - b0, offset=b0).copy()
        dt = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32}[meta["dtype"]]
        out[name] = torch.from_numpy(raw).view(dt).reshape(meta["shape"]).to(F64)
    return out


def effective_ff(cfg):
    """The feed-forward width a config.json gives (2/3 rule, multiplier, round up)."""
    ff = cfg["block_ff_dim"] if "block_ff_dim" in cfg else cfg["intermediate_size"]
    if cfg.get("block_auto_adjust_ff_dim", False):
        ff = (2 * ff) // 3
        if cfg.get("block_ffn_dim_multiplier") is not None:
            ff = int(cfg["block_ffn_dim_multiplier"] * ff)
        m = cfg.get("block_multiple_of", 256)
        ff = m * ((ff + m - 1) // m)
    return ff


def layer_is_attention(cfg):
    n = cfg["num_hidden_layers"]
    if "layer_types" in cfg:
        return [t == "full_attention" for t in cfg["layer_types"]]
    idx = set(cfg["full_attn_idxs"])
    return [i in idx for i in range(n)]


class PlainModel:
    def __init__(self, model_dir):
        with open(os.path.join(model_dir, "config.json")) as f:
            self.cfg = json.load(f)
        self.w = read_safetensors(os.path.join(model_dir, "model.safetensors"))
        c = self.cfg
        self.H = c["hidden_size"]
        self.nh = c["num_attention_heads"]
        self.nkv = c["num_key_value_heads"]
        self.hd = self.H // self.nh
        self.L = c.get("conv_L_cache", 3)
        self.eps = c.get("norm_eps", 1e-5)
        self.theta = c.get("rope_theta", 1e6)
        self.bias = c.get("conv_bias", False)
        self.tied = c.get("tie_embedding", c.get("tie_word_embeddings", True))
        self.is_attn = layer_is_attention(c)
        self.window = None   # LFM2 has no sliding window (src/Inference/lfm2.jl:73-76)

    # ---- whole model ---------------------------------------------------------------------------
    def logits(self, token_ids, rows=None):
        """All logits [T, V] of one whole sequence (src/Inference/Inference.jl:179-391); with ``rows``
        only those positions go through the head (wide vocabularies)."""
        w = self.w
        h = embedding(w["model.embed_tokens.weight"], token_ids)
        for i, attn in enumerate(self.is_attn):
            p = f"model.layers.{i}."
            xn = rmsnorm(h, w[p + "operator_norm.weight"], self.eps)
            if attn:
                m = attention_mixer(
                    xn, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"],
                    w[p + "self_attn.v_proj.weight"], w[p + "self_attn.out_proj.weight"],
                    w[p + "self_attn.q_layernorm.weight"], w[p + "self_attn.k_layernorm.weight"],
                    self.nh, self.nkv, self.hd, self.eps, self.theta, self.window)
            else:
                m = short_conv_mixer(
                    xn, w[p + "conv.in_proj.weight"], w[p + "conv.conv.weight"], w[p + "conv.out_proj.weight"],
                    w.get(p + "conv.in_proj.bias"), w.get(p + "conv.conv.bias"), w.get(p + "conv.out_proj.bias"))
            h = h + m                                              # Inference.jl:2372, 2511
            h = h + swiglu_ffn(rmsnorm(h, w[p + "ffn_norm.weight"], self.eps),
                               w[p + "feed_forward.w1.weight"], w[p + "feed_forward.w3.weight"],
                               w[p + "feed_forward.w2.weight"])    # Inference.jl:2514-2517
        if rows is not None:
            h = h[list(rows)]
        hn = rmsnorm(h, w["model.embedding_norm.weight"], self.eps)   # the final norm, lfm2.jl:173
        head = w["model.embed_tokens.weight"] if self.tied else w["lm_head.weight"]
        return hn @ head.T                                          # Inference.jl:2747-2800

    def greedy(self, prompt, n_new):
        """Prompt + n_new greedy tokens, re-running the whole sequence for every token."""
        ids = list(prompt)
        for _ in range(n_new):
            ids.append(int(torch.argmax(self.logits(ids)[-1])))
        return ids


# ---- parts ------------------------------------------------------------------------------------------
def embedding(table, token_ids):
    """h[t,:] = E[id_t,:], no scaling (src/Operators/cpu.jl:85-90; Inference.jl:222-224)."""
    return table[torch.as_tensor(list(token_ids), dtype=torch.long)].clone()


def rmsnorm(x, weight, eps):
    """y = (x / sqrt(mean(x^2) + eps)) * w over the last axis (src/Operators/cpu.jl:293-311)."""
    r = torch.sqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return (x / r) * weight.reshape(-1)


def rope(x, positions, theta):
    """Half-split rotary on [T, heads, d]: pairs (i, i+d/2), angle pos*theta^(-2i/d)
    (src/Operators/cpu.jl:357-371)."""
    T, nheads, d = x.shape
    half = d // 2
    i = torch.arange(half, dtype=F64)
    ang = torch.as_tensor(positions, dtype=F64)[:, None] * torch.pow(torch.tensor(theta, dtype=F64), -2.0 * i / d)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1)


def causal_attention(q, k, v, window=None):
    """q [T,nh,d], k/v [T,nkv,d] -> [T,nh,d].  scores q.k/sqrt(d) (Inference.jl:1201-1205), query t
    sees keys lo..t with lo = max(0, t-window+1) (:1206-1207), softmax (:1414-1430), GQA map
    h -> h // (nh/nkv) (:1398), values in ascending key order (:1449-1457)."""
    T, nh, d = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    out = torch.zeros_like(q)
    for h in range(nh):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].T) / math.sqrt(d)
        t_idx = torch.arange(T)
        mask = t_idx[None, :] > t_idx[:, None]
        if window is not None:
            mask = mask | (t_idx[None, :] < (t_idx[:, None] - window + 1))
        s = s.masked_fill(mask, float("-inf"))
        p = torch.exp(s - s.max(dim=-1, keepdim=True).values)
        p = p / p.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, g, :]
    return out


def attention_mixer(xn, wq, wk, wv, wo, q_norm_w, k_norm_w, nh, nkv, hd, eps, theta, window=None):
    """Projections, head split (head-major features, Inference.jl:1573-1583), per-head q/k RMSNorm
    before the rotation (:2401-2416), attention, merge and output projection (:2494, 2508)."""
    T = xn.shape[0]
    q = (xn @ wq.T).reshape(T, nh, hd)
    k = (xn @ wk.T).reshape(T, nkv, hd)
    v = (xn @ wv.T).reshape(T, nkv, hd)
    q = rmsnorm(q, q_norm_w, eps)
    k = rmsnorm(k, k_norm_w, eps)
    pos = list(range(T))
    q, k = rope(q, pos, theta), rope(k, pos, theta)
    o = causal_attention(q, k, v, window)
    return o.reshape(T, nh * hd) @ wo.T


def short_conv_fir(bcx, taps, conv_bias=None):
    """The gated FIR between the projections, token by token with an explicit history, exactly as
    the reference's loop (src/Inference/lfm2.jl:253-271): bx = B*X; y = sum_p hist[p]*w[p] +
    bx*w[L-1]; out = C*y; history shifts and takes bx.  Zero history at the start."""
    T, H3 = bcx.shape
    H = H3 // 3
    taps = taps.reshape(H, -1)
    L = taps.shape[1]
    hist = torch.zeros((H, L - 1), dtype=F64)
    out = torch.zeros((T, H), dtype=F64)
    for t in range(T):
        bx = bcx[t, :H] * bcx[t, 2 * H:]
        y = torch.zeros(H, dtype=F64)
        for p in range(L - 1):
            y = y + hist[:, p] * taps[:, p]
        y = y + bx * taps[:, L - 1]
        if conv_bias is not None:
            y = y + conv_bias
        out[t] = bcx[t, H:2 * H] * y
        hist = torch.cat([hist[:, 1:], bx[:, None]], dim=1)
    return out


def short_conv_mixer(xn, w_in, taps, w_out, b_in=None, b_conv=None, b_out=None):
    """in_proj -> gated FIR -> out_proj (src/Inference/lfm2.jl:192-204).  The biases are this
    engine's own option (the reference has no bias tensors, lfm2.jl:171-172)."""
    bcx = xn @ w_in.T
    if b_in is not None:
        bcx = bcx + b_in
    y = short_conv_fir(bcx, taps, b_conv) @ w_out.T
    if b_out is not None:
        y = y + b_out
    return y


def swiglu_ffn(xn, w_gate, w_up, w_down):
    """d = ((g / (1 + exp(-g))) * u) Wd^T (Inference.jl:869-882; cpu.jl:482-488)."""
    g, u = xn @ w_gate.T, xn @ w_up.T
    return ((g / (1.0 + torch.exp(-g))) * u) @ w_down.T


# ---- sampling (src/Inference/sampling.jl:13-74, plain full-sort form) --------------------------------
class PlainSampler:
    def __init__(self, temperature, top_p=1.0, seed=0):
        assert temperature > 0 and 0 < top_p <= 1 and seed >= 0
        self.temperature, self.top_p, self.state = float(temperature), float(top_p), int(seed)

    def unit(self):
        """splitmix64 step, 53-bit unit float (sampling.jl:32-39)."""
        M = (1 << 64) - 1
        self.state = (self.state + 0x9E3779B97F4A7C15) & M
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        z = z ^ (z >> 31)
        return float(z >> 11) * 2.0 ** -53

    def sample(self, logits_row):
        l = [float(x) for x in logits_row]
        hi = max(l)
        w = [math.exp((x - hi) / self.temperature) for x in l]
        total = 0.0
        for x in w:
            total += x
        if self.top_p >= 1:
            r = self.unit() * total
            acc = 0.0
            for i, x in enumerate(w):
                acc += x
                if r < acc:
                    return i
            return len(w) - 1
        order = sorted(range(len(w)), key=lambda i: (-w[i], i))   # stable: ties by lower id
        target = self.top_p * total
        acc, keep = 0.0, len(w)
        for k, i in enumerate(order):
            acc += w[i]
            if acc >= target:
                keep = k + 1
                break
        cut = 0.0
        for i in order[:keep]:
            cut += w[i]
        r = self.unit() * cut
        acc = 0.0
        for i in order[:keep]:
            acc += w[i]
            if r < acc:
                return i
        return order[keep - 1]
