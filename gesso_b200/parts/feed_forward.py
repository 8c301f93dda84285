"""SwiGLU feed-forward: ``down( silu(gate(x)) * up(x) )``, no biases.

``g = x Wg^T``, ``u = x Wu^T``, ``a = (g / (1 + exp(-g))) * u``, ``d = a Wd^T``
(src/Inference/Inference.jl:869-882, src/Operators/cpu.jl:482-488).  Gate and up are fused
into one matrix at bind time (gate rows first).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from .base import FeedForward, ParamDecl
from .registry import register_feed_forward


class SwiGLU(FeedForward):
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
        self.w_gate_up = torch.cat([g.to(common), u.to(common)], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"]

    def forward(self, x, ctx):
        gu = ops.linear(x, self.w_gate_up, out_dtype=x.dtype)
        a = ops.swiglu(gu)
        return ops.linear(a, self.w_down, out_dtype=x.dtype), None


register_feed_forward("swiglu", SwiGLU, replace=True)
