"""Which attention kernel a step's queries run on.

float32 runs always take the FP32-arithmetic kernel.  bfloat16 runs take the tensor-core kernels
when the sizes fit them (head 32/64/96/128, pages in multiples of 16 slots): the split-KV kernel
for steps of single tokens; for steps with portions the tcgen05 flash kernel (head 64, 2 to 16 query
heads per kv head) or else the mma.sync flash kernel; other sizes take the FP32-arithmetic kernel
on bfloat16 data.  Every branch is one of this library's own kernels.
"""
from __future__ import annotations

import torch

from .. import ops


def paged_attention(rt, q, cache, ctx, window, scale):
    N, nh, hd = q.shape
    nkv, page_size = cache.k_pages.shape[1], cache.k_pages.shape[2]
    if q.dtype == torch.bfloat16 and ops.fast_attention_takes(hd, page_size, nh, nkv):
        if ctx.decode_only:
            splits = ops.decode_splits(ctx.n_segs, nkv, ctx.max_kv_len, uneven=True)
            ws = None
            if splits > 1:
                key = ("decode_attention_workspace", ctx.n_segs, nh, nkv, hd, splits)
                ws = rt.shared.get(key)
                if ws is None:
                    dev = q.device
                    ws = (torch.empty((ctx.n_segs * nh * splits * hd,), dtype=torch.float32, device=dev),
                          torch.empty((ctx.n_segs * nh * splits * 2,), dtype=torch.float32, device=dev),
                          torch.zeros((ctx.n_segs * nkv,), dtype=torch.int32, device=dev))
                    rt.shared[key] = ws
            return ops.decode_attention(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.positions,
                                        window, scale, splits, ws, ctx.kv_span)
        if ops.attention_tcgen05_takes(hd, page_size, nh, nkv):
            # head 64 with 2..16 query heads per kv head: S and P in tensor memory, pages by TMA
            return ops.prefill_attention_tcgen05(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.seg_start,
                                                 ctx.seg_pos0, ctx.tile_seg, ctx.tile_q0, window, scale)
        return ops.prefill_attention(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.seg_start,
                                     ctx.seg_pos0, ctx.tile_seg, ctx.tile_q0, window, scale)
    return ops.paged_attention_generic(q, cache.k_pages, cache.v_pages, cache.block_table,
                                       ctx.positions, ctx.seg_of_token, window, scale)
