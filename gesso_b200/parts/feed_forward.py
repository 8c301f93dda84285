"""SwiGLU feed-forward: ``down( silu(gate(x)) * up(x) )``, no biases.

``g = x Wg^T``, ``u = x Wu^T``, ``a = (g / (1 + exp(-g))) * u``, ``d = a Wd^T``
(src/Inference/Inference.jl:869-882, src/Operators/cpu.jl:482-488).  Gate and up are fused
into one matrix at bind time.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from .base import FeedForward, ParamDecl
from .registry import register_feed_forward


class SwiGLU(FeedForward):
    accepts_lazy_norm = True
    fuses_residual = True

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec["hidden_size"])
        self.ff = int(spec["ff_dim"])

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {
            "gate_proj.weight": ParamDecl((self.ff, self.hidden), fan_in=self.hidden),
            "up_proj.weight": ParamDecl((self.ff, self.hidden), fan_in=self.hidden),
            "down_proj.weight": ParamDecl((self.hidden, self.ff), fan_in=self.ff),
        }

    def bind(self, tensors, rt) -> None:
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        common = torch.float32 if (g.dtype == torch.float32 or u.dtype == torch.float32) else g.dtype
        # groups of 8 gate rows followed by their 8 up rows when the width allows it (the layout
        # whose activation the skinny matrix product applies in its epilogue), else gate rows first
        self.packed = self.ff % 8 == 0
        if self.packed:
            self.w_gate_up = ops.pack_gate_up(g.to(common), u.to(common))
        else:
            self.w_gate_up = torch.cat([g.to(common), u.to(common)], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"]

    def fold_input_scale(self, scale) -> bool:
        self.w_gate_up = ops.fold_norm_weight(self.w_gate_up, scale)
        return True

    def forward(self, x, ctx, residual=None):
        a = ops.linear_swiglu(x, self.w_gate_up, self.packed)
        if residual is not None:
            return ops.linear_residual(a, self.w_down, residual, None), None
        return ops.linear(a, self.w_down, out_dtype=a.dtype), None


register_feed_forward("swiglu", SwiGLU, replace=True)
