"""Which attention kernel a step's queries run on.

float32 runs always take the FP32 kernel.  bfloat16 runs take the tensor-core kernels
when the head size fits them (a multiple of 16 up to 128): the flash prefill kernel for steps
with portions, the split-KV kernel for steps of single tokens; other head sizes take the FP32
arithmetic kernel on bfloat16 data.  Every branch is one of this library's own kernels.
"""
from __future__ import annotations

import torch

from .. import ops


def paged_attention(rt, q, cache, ctx, window, scale):
    fast = getattr(ops, "paged_attention_fast", None)
    if fast is not None and q.dtype == torch.bfloat16 and ops.fast_attention_takes(q.shape[2]):
        return fast(q, cache.k_pages, cache.v_pages, cache.block_table, ctx, window, scale)
    return ops.paged_attention_generic(q, cache.k_pages, cache.v_pages, cache.block_table,
                                       ctx.positions, ctx.seg_of_token, window, scale)
