"""The double-gated short convolution mixer.

``bcx = x W_in^T`` gives B, C and X side by side; ``bx = B * X``; a causal depthwise FIR of
``kernel`` taps runs over ``bx`` (taps oldest to newest, the newest on the current token);
``y = C * fir``; ``out = y W_out^T`` (src/Inference/lfm2.jl:192-204, 253-271).  The last
``kernel - 1`` values of ``bx`` per channel are the request's state (float32, zero at the start
of a request, src/Inference/Inference.jl:147-148).  There is no activation function.

With ``bias`` the two projections and the FIR each add a bias vector; the reference's tensor
map has no bias tensors (src/Inference/lfm2.jl:171-172), so that option is this engine's own
definition, shared with the plain implementation of the tests.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..errors import invalid
from .base import Mixer, ParamDecl, StateNeed
from .registry import register_mixer


class ShortConv(Mixer):
    accepts_lazy_norm = True
    fuses_residual = True

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec["hidden_size"])
        self.kernel = int(spec["kernel"])
        self.bias = bool(spec.get("bias", False))
        if self.kernel < 2:
            raise invalid("short_conv: kernel must be >= 2 (one tap keeps no history)")
        if self.kernel > 8:
            raise invalid("short_conv: kernels longer than 8 taps are not supported")

    def param_decls(self) -> Dict[str, ParamDecl]:
        H, L = self.hidden, self.kernel
        d = {
            "in_proj.weight": ParamDecl((3 * H, H), fan_in=H),
            "conv.weight": ParamDecl((H, L), role="vector", alt_shapes=((H, 1, L),), fan_in=L),
            "out_proj.weight": ParamDecl((H, H), fan_in=H),
        }
        if self.bias:
            d["in_proj.bias"] = ParamDecl((3 * H,), role="vector")
            d["conv.bias"] = ParamDecl((H,), role="vector")
            d["out_proj.bias"] = ParamDecl((H,), role="vector")
        return d

    def cache_need(self):
        return StateNeed((self.kernel - 1, self.hidden))

    def bind(self, tensors, rt) -> None:
        self.w_in = tensors["in_proj.weight"]
        self.w_out = tensors["out_proj.weight"]
        self.taps = tensors["conv.weight"].reshape(self.hidden, self.kernel).contiguous()
        self.b_in = tensors.get("in_proj.bias")
        self.b_conv = tensors.get("conv.bias")
        self.b_out = tensors.get("out_proj.bias")
        # bfloat16 runs keep the input projection in groups of 24 rows (B, C, X of 8 channels): decoding
        # steps then run the convolution in the projection's epilogue, and longer steps read the
        # projection's output in the same grouping
        self.packed = self.w_in.dtype == torch.bfloat16 and self.hidden % 8 == 0
        if self.packed:
            self.w_in = ops.pack_bcx(self.w_in)

    def fold_input_scale(self, scale) -> bool:
        self.w_in = ops.fold_norm_weight(self.w_in, scale)
        return True

    def forward(self, x, ctx, cache, residual=None):
        if self.packed and ctx.decode_only and ops.skinny_conv_takes(x.shape[0], self.w_in, x.dtype, self.kernel):
            y = ops.linear_conv(x, self.w_in, self.b_in, self.taps, self.b_conv, cache.state, ctx.seg_pos0,
                                cache.slots)
        else:
            bcx = ops.linear(x, self.w_in, out_dtype=x.dtype)
            y = ops.short_conv(bcx, self.b_in, self.taps, self.b_conv, cache.state, ctx.seg_of_token,
                               ctx.seg_start, ctx.seg_pos0, cache.slots, ctx.n_segs, ctx.max_seg_len,
                               packed=self.packed)
        if residual is not None:
            d = ops.linear_residual(y, self.w_out, residual, self.b_out)
            return (None, None) if d is None else (d, self.b_out)
        return ops.linear(y, self.w_out, out_dtype=x.dtype), self.b_out


register_mixer("short_conv", ShortConv, replace=True)
