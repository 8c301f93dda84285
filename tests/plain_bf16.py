"""The plain LFM2 with a bfloat16 rounding wherever the engine's bfloat16 run stores an activation.

``plain_lfm2.PlainModel`` is exact (float64 throughout), so a bfloat16 engine can only be held to it at
a bound as wide as bfloat16's own noise (a few percent of the largest logit), which hides small faults.
This model computes the same formulas in float64 but rounds to bfloat16 at the places where the engine
keeps a bfloat16 tensor, so that what is left between it and the engine is accumulation order and
flips of a rounding that sat on the fence.  It shares no code with ``gesso_b200``; what it has to know about the
engine is listed here and nowhere else.

Where the engine rounds depends on the kernels a step takes, which depend on the step, not on the
token alone.  Every token therefore carries the *kind* of the step it ran in:

``S``  a step of single tokens, at most 16 of them (decoding): norm weights folded into the matrix
       that follows, the matrix product fed ``bf16(h)`` and scaled by ``1/rms(h)`` afterwards, the
       sublayer's result added to the float32 stream unrounded, SwiGLU from unrounded gate and up
       (for the matrices whose sizes the small-step product takes; the others go the way of ``L``);
``P``  any other step of at most 16 tokens: the same matrix products, attention as a portion;
``L``  a step of 17 to 1023 tokens: ``bf16(h / rms(h))`` computed first, every product stored in
       bfloat16 (gate and up too) and the sublayer's result added to the stream from its bfloat16 copy;
``T``  a step of 1024 tokens or more: as ``L``, but SwiGLU from unrounded gate and up (the epilogue of
       the matrix product).

Keys are stored normed, rotated and rounded, values rounded, whatever the kind, so a token's attention
reads the same cache in every schedule.  ``p_rounded`` says whether the attention kernels round the
probabilities to bfloat16 before they meet the values (the tensor-core kernels do: head sizes 32, 64,
96, 128 on pages of 16 slots and multiples; the general kernel does not).
"""
from __future__ import annotations

import math

import torch

import plain_lfm2 as P

F64 = torch.float64


def r(x):
    """Round to bfloat16 (nearest even), keep computing in float64."""
    return x.to(torch.bfloat16).to(F64)


def kinds_of_steps(steps, wide: bool = False):
    """``steps``: for one request, a list of (tokens this request brings, tokens of the whole step, whether the
    step holds single tokens only) in feeding order -> one kind per token.  ``wide``: the model's fused
    gate/up matrix is wide enough for the tensor-memory product of steps of 1024 tokens and more (its tile
    waves fill the device; narrow test models stay with the library product there, kind ``L``)."""
    out = []
    for n, total, single in steps:
        kind = ("S" if single else "P") if total <= 16 else ("T" if total >= 1024 and wide else "L")
        out += [kind] * n
    return out


class RoundedPlain(P.PlainModel):
    def __init__(self, model_dir, p_rounded: bool):
        super().__init__(model_dir)
        self.p_rounded = p_rounded
        w = self.w
        # the norm weight moves into the columns of the matrix that follows, rounded once
        self.folded = {}
        for i, attn in enumerate(self.is_attn):
            p = f"model.layers.{i}."
            wn = w[p + "operator_norm.weight"]
            if attn:
                for name in ("q_proj", "k_proj", "v_proj"):
                    self.folded[p + name] = r(w[p + f"self_attn.{name}.weight"] * wn)
            else:
                self.folded[p + "in_proj"] = r(w[p + "conv.in_proj.weight"] * wn)
            wf = w[p + "ffn_norm.weight"]
            self.folded[p + "w1"] = r(w[p + "feed_forward.w1.weight"] * wf)
            self.folded[p + "w3"] = r(w[p + "feed_forward.w3.weight"] * wf)

    # ---- the parts, with the engine's roundings ---------------------------------------------------
    @staticmethod
    def few_rows_product_takes(n_out: int, n_in: int) -> bool:
        """The matrix product of steps of at most 16 tokens takes output widths that are multiples of 16
        and inner sizes that are multiples of 32; other matrices go to the library product even in small
        steps, which stores its result in bfloat16."""
        return n_out >= 16 and n_out % 16 == 0 and n_in >= 32 and n_in % 32 == 0

    def _rinv(self, h):
        return 1.0 / torch.sqrt((h * h).sum(-1, keepdim=True) / h.shape[-1] + self.eps)

    def _first_product(self, h, w_folded, few):
        """``rmsnorm(h) W'^T`` unrounded: for the tokens of ``few`` with ``bf16(h)`` into the product and the
        scale by ``1/rms(h)`` afterwards (the norm rides in the product of a small step when nothing is
        waiting to be added to the stream), else from the norm kernel's bfloat16 output."""
        rinv = self._rinv(h)
        return torch.where(few[:, None], (r(h) @ w_folded.T) * rinv, r(h * rinv) @ w_folded.T)

    def _add(self, h, product, fused, bias=None):
        """The sublayer's result joins the float32 stream: unrounded where the product's epilogue adds it
        (``fused``), from its bfloat16 copy else; a bias joins in float32 beside it."""
        h = h + torch.where(fused[:, None], product, r(product))
        return h if bias is None else h + bias

    def logits(self, token_ids, rows=None, kinds=None):
        T = len(token_ids)
        kinds = kinds or ["L"] * T
        assert len(kinds) == T
        small = torch.tensor([k in "SP" for k in kinds])
        tensor_memory = torch.tensor([k == "T" for k in kinds])
        none = torch.zeros(T, dtype=torch.bool)
        takes = self.few_rows_product_takes
        H, F = self.H, P.effective_ff(self.cfg)
        qkv_width = (self.nh + 2 * self.nkv) * self.hd
        w = self.w
        h = P.embedding(w["model.embed_tokens.weight"], token_ids)
        lazy = small.clone()        # nothing waits to be added to the stream: the next norm need not run on its own
        for i, attn in enumerate(self.is_attn):
            p = f"model.layers.{i}."
            if attn:
                few = lazy if takes(qkv_width, H) else none
                fused = small if takes(H, self.nh * self.hd) else none
                h = self._add(h, self._attention(h, p, few), fused)
            else:
                few = lazy if takes(3 * H, H) else none
                fused = small if takes(H, H) else none
                h = self._add(h, self._conv(h, p, few), fused, w.get(p + "conv.out_proj.bias"))
            lazy = fused
            in_small_product = small if takes(2 * F, H) else none
            few = lazy & in_small_product
            g = self._first_product(h, self.folded[p + "w1"], few)
            u = self._first_product(h, self.folded[p + "w3"], few)
            # gate and up meet the activation unrounded in the epilogue of the small-step product and of the
            # tensor-memory product; the library product stores them in bfloat16 first
            unrounded = in_small_product | tensor_memory
            g = torch.where(unrounded[:, None], g, r(g))
            u = torch.where(unrounded[:, None], u, r(u))
            a = r((g / (1.0 + torch.exp(-g))) * u)
            fused = small if takes(H, F) else none
            h = self._add(h, a @ w[p + "feed_forward.w2.weight"].T, fused)
            lazy = fused
        if rows is not None:
            h = h[list(rows)]
        hn = r((h * self._rinv(h)) * w["model.embedding_norm.weight"])      # the final norm is not folded
        head = w["model.embed_tokens.weight"] if self.tied else w["lm_head.weight"]
        return hn @ head.T

    def _conv(self, h, p, few):
        w = self.w
        bcx = r(self._first_product(h, self.folded[p + "in_proj"], few))
        b_in, b_conv = w.get(p + "conv.in_proj.bias"), w.get(p + "conv.conv.bias")
        if b_in is not None:
            bcx = bcx + b_in
        y = r(P.short_conv_fir(bcx, w[p + "conv.conv.weight"], b_conv))       # the history holds unrounded B*X
        return y @ w[p + "conv.out_proj.weight"].T

    def _attention(self, h, p, few):
        w = self.w
        T = h.shape[0]
        q = r(self._first_product(h, self.folded[p + "q_proj"], few)).reshape(T, self.nh, self.hd)
        k = r(self._first_product(h, self.folded[p + "k_proj"], few)).reshape(T, self.nkv, self.hd)
        v = r(self._first_product(h, self.folded[p + "v_proj"], few)).reshape(T, self.nkv, self.hd)
        pos = list(range(T))
        q = r(P.rope(P.rmsnorm(q, w[p + "self_attn.q_layernorm.weight"], self.eps), pos, self.theta))
        k = r(P.rope(P.rmsnorm(k, w[p + "self_attn.k_layernorm.weight"], self.eps), pos, self.theta))
        group = self.nh // self.nkv
        o = torch.zeros(T, self.nh, self.hd, dtype=F64)
        idx = torch.arange(T)
        mask = idx[None, :] > idx[:, None]
        for hh in range(self.nh):
            g = hh // group
            s = (q[:, hh] @ k[:, g].T) / math.sqrt(self.hd)
            s = s.masked_fill(mask, float("-inf"))
            if self.p_rounded:
                # the tensor-core kernels work in base 2 against the row's maximum rounded up to a whole
                # number, and round the probabilities to bfloat16 for their product with the values (the
                # sum of the probabilities stays unrounded)
                s2 = s * math.log2(math.e)
                pr = torch.exp2(s2 - torch.ceil(s2.max(dim=-1, keepdim=True).values))
                num = r(pr) @ v[:, g]
            else:
                pr = torch.exp(s - s.max(dim=-1, keepdim=True).values)
                num = pr @ v[:, g]
            o[:, hh] = num / pr.sum(dim=-1, keepdim=True)
        return r(o.reshape(T, self.nh * self.hd)) @ w[p + "self_attn.out_proj.weight"].T
