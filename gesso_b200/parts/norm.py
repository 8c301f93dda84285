"""RMSNorm with the residual add folded in.

``y = (x / sqrt(mean(x^2) + eps)) * w`` over the last axis, divide first, scale
second (src/Operators/cpu.jl:293-311).  The residual stream is float32; the sum
and the statistics are float32, the output is rounded to the run dtype.

With ``lazy=True`` and nothing to add, the norm is not run: a
:class:`~gesso_b200.ops.LazyNorm` is returned, which the consumer's first matrix
product applies in its prologue for steps of few tokens (or materialises).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from .base import Norm, ParamDecl
from .registry import register_norm


class RMSNorm(Norm):
    supports_lazy = True

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = None
        self.out_dtype = None
        self.folded = False      # True once the consumer's matrix carries this norm's weight

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {"weight": ParamDecl((self.size,), role="vector", init="ones")}

    def bind(self, tensors, rt) -> None:
        self.weight = tensors["weight"]
        self.out_dtype = rt.dtype

    def fold_into(self, consumer) -> bool:
        """Let ``consumer`` (a part with ``fold_input_scale``) absorb the weight into its first matrix.
        Only in bfloat16 runs: the 32-bit path keeps the reference's order of operations."""
        if self.folded or self.out_dtype != torch.bfloat16:
            return self.folded
        fold = getattr(consumer, "fold_input_scale", None)
        if fold is not None and fold(self.weight):
            self.folded = True
        return self.folded

    def add_norm(self, h, delta, delta_bias, rows=None, lazy=False):
        weight = None if self.folded else self.weight
        if lazy and delta is None and rows is None:
            return ops.LazyNorm(h, weight, self.eps, self.out_dtype)
        return ops.add_rmsnorm(h, delta, delta_bias, weight, self.eps, self.out_dtype, rows)


register_norm("rmsnorm", RMSNorm, replace=True)
