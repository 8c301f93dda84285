"""Grouped-query attention over the paged cache, with per-head q/k RMSNorm and a position part.

``q = x Wq^T`` (nh heads), ``k, v = x Wk^T, x Wv^T`` (nkv heads), features head-major
(src/Inference/Inference.jl:1573-1583).  q and k are normed per head over ``head_dim``
before the rotation (:2401-2416); the cache holds normed, rotated K and raw V (:2417-2421).
Scores are ``q.k / sqrt(head_dim)`` (:1201-1205), causal, optionally limited to the last
``window`` positions (:1206-1207); query head h reads kv head ``h // (nh/nkv)`` (:1398).
``out = merge(heads) Wo^T`` (:2494, 2508).

Parameters (all from the part spec): hidden_size, n_heads, n_kv_heads, head_dim,
qk_norm_eps (``None``: no q/k norm), window (``None``: all keys), position (a position
part spec).  The three projections are fused into one matrix at bind time.
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from .. import ops
from ..errors import invalid
from .base import Mixer, PagedNeed, ParamDecl
from .registry import build_position, register_mixer


class GQAttention(Mixer):
    accepts_lazy_norm = True
    fuses_residual = True

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["n_heads"])
        self.nkv = int(spec["n_kv_heads"])
        self.hd = int(spec["head_dim"])
        self.eps = spec.get("qk_norm_eps")
        self.window = spec.get("window")
        if self.nh < 1 or self.nkv < 1 or self.nh % self.nkv != 0:
            raise invalid(f"attention: {self.nh} heads are not a multiple of {self.nkv} kv heads")
        if self.hd < 2 or self.hd % 2 != 0 or self.hd > 256:
            raise invalid(f"attention: head_dim {self.hd} must be even and at most 256")
        if self.window is not None and int(self.window) < 1:
            raise invalid("attention: window must be >= 1")
        self.position = build_position(spec["position"])
        self.position.check_head_dim(self.hd)
        # 1/sqrt(hd) rounded once from float64 (exact when sqrt(hd) is a power of two,
        # src/Inference/Inference.jl:1209-1232)
        self.scale = 1.0 / math.sqrt(self.hd)

    def param_decls(self) -> Dict[str, ParamDecl]:
        q, kv = self.nh * self.hd, self.nkv * self.hd
        d = {
            "q_proj.weight": ParamDecl((q, self.hidden), fan_in=self.hidden),
            "k_proj.weight": ParamDecl((kv, self.hidden), fan_in=self.hidden),
            "v_proj.weight": ParamDecl((kv, self.hidden), fan_in=self.hidden),
            "o_proj.weight": ParamDecl((self.hidden, q), fan_in=q),
        }
        if self.eps is not None:
            d["q_norm.weight"] = ParamDecl((self.hd,), role="vector", init="ones")
            d["k_norm.weight"] = ParamDecl((self.hd,), role="vector", init="ones")
        return d

    def cache_need(self):
        return PagedNeed(self.nkv, self.hd, None if self.window is None else int(self.window))

    def bind(self, tensors, rt) -> None:
        ws = [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]]
        common = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_q = ws[0].to(common).contiguous()
        self.w_qkv = torch.cat([w.to(common) for w in ws], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"]
        self.q_norm = tensors.get("q_norm.weight")
        self.k_norm = tensors.get("k_norm.weight")
        self.position.bind({}, rt)
        self.rt = rt

    def fold_input_scale(self, scale) -> bool:
        self.w_q = ops.fold_norm_weight(self.w_q, scale)
        self.w_qkv = ops.fold_norm_weight(self.w_qkv, scale)
        return True

    def forward(self, x, ctx, cache, residual=None):
        writes = cache.writes
        qkv = ops.linear(x, self.w_qkv if writes else self.w_q, out_dtype=x.dtype)
        cos, sin = self.position.tables()
        # a position part without layout() rotates the whole head by halves
        rot_dim, interleaved = self.position.layout() if hasattr(self.position, "layout") else (self.hd, False)
        q = ops.qk_norm_rope_store(qkv, self.q_norm, self.k_norm, self.eps if self.eps is not None else 0.0,
                                   cos, sin, ctx.positions, ctx.seg_of_token, cache.block_table,
                                   cache.k_pages, cache.v_pages, self.nh, self.nkv, self.hd, writes, ctx.status,
                                   tiles=None if ctx.decode_only else (ctx.seg_start, ctx.seg_pos0, ctx.tile_seg,
                                                                       ctx.tile_q0),
                                   rot_dim=rot_dim or None, interleaved=interleaved)
        o = self.rt.attention(q, cache, ctx, self.window, self.scale)
        if residual is not None:
            return ops.linear_residual(o, self.w_o, residual, None), None
        return ops.linear(o, self.w_o, out_dtype=x.dtype), None


register_mixer("gqa_attention", GQAttention, replace=True)
