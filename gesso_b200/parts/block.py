"""Block arrangements: how a layer's parts and residuals are ordered.

``prenorm`` (src/Inference/Inference.jl:278-363, 3322-3378)::

    h = h + Mixer(Norm_m(h))
    h = h + FeedForward(Norm_f(h))

The residual stream ``h`` is float32 and is updated in place.  A sublayer's output is not
added at once: it travels as ``pending = (delta, bias)`` to the next norm, which adds it into
``h`` and norms the sum in one kernel (the reference fuses the same add+norm on its decode
path, src/Inference/Inference.jl:3239-3247).
"""
from __future__ import annotations

from typing import Dict

from .base import ParamDecl
from .registry import (build_feed_forward, build_mixer, build_norm, register_block)


class PreNormBlock:
    def __init__(self, block_spec):
        self.spec = block_spec
        self.mixer = build_mixer(block_spec.mixer)
        self.feed_forward = build_feed_forward(block_spec.feed_forward)
        self.mixer_norm = build_norm(block_spec.mixer_norm)
        self.ff_norm = build_norm(block_spec.ff_norm)

    def parts(self):
        return (("mixer_norm.", self.mixer_norm), ("mixer.", self.mixer),
                ("ff_norm.", self.ff_norm), ("feed_forward.", self.feed_forward))

    def param_decls(self) -> Dict[str, ParamDecl]:
        out = {}
        for prefix, part in self.parts():
            for name, decl in part.param_decls().items():
                out[prefix + name] = decl
        return out

    def cache_need(self):
        return self.mixer.cache_need()

    def bind(self, tensors, rt) -> None:
        for prefix, part in self.parts():
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}, rt)
        # a norm's weight may move into the first matrix of the part it feeds (bfloat16 runs): the
        # norm then only divides by the root mean square, which the consumer's skinny matrix product
        # gathers on the fly
        for norm, consumer in ((self.mixer_norm, self.mixer), (self.ff_norm, self.feed_forward)):
            fold = getattr(norm, "fold_into", None)
            if fold is not None:
                fold(consumer)

    def forward(self, h, pending, ctx, cache):
        """``pending`` is the previous sublayer's (delta, bias) not yet added to ``h`` (or Nones).

        Parts that set ``accepts_lazy_norm`` may be handed a norm that has not run yet; parts that
        set ``fuses_residual`` are given ``residual=h`` and may add their output into it themselves
        (they then return ``(None, None)``)."""
        x = self._norm(self.mixer_norm, self.mixer, h, pending)
        if getattr(self.mixer, "fuses_residual", False):
            m = self.mixer.forward(x, ctx, cache, residual=h)
        else:
            m = self.mixer.forward(x, ctx, cache)
        x = self._norm(self.ff_norm, self.feed_forward, h, m)
        if getattr(self.feed_forward, "fuses_residual", False):
            return self.feed_forward.forward(x, ctx, residual=h)
        return self.feed_forward.forward(x, ctx)

    @staticmethod
    def _norm(norm, consumer, h, pending):
        if getattr(consumer, "accepts_lazy_norm", False) and getattr(norm, "supports_lazy", False):
            return norm.add_norm(h, pending[0], pending[1], lazy=True)
        return norm.add_norm(h, pending[0], pending[1])


register_block("prenorm", PreNormBlock, replace=True)
