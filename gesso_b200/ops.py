"""Tensor-level wrappers of the kernel library.

Each function checks device, dtype, layout and sizes of its ``torch`` tensors,
launches one kernel (or a short fixed sequence) on the current CUDA stream and
returns the output tensor.  Nothing here computes on the CPU and nothing falls
back to a library implementation of the same operation; the only library call
is the dense bfloat16 matrix product (cuBLAS through ``torch.mm``) for steps of
17 to 1023 tokens, where the reference also calls a BLAS
(src/Operators/cpu.jl:629-630); fewer tokens take the skinny kernel, more take
the tcgen05 kernel.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .csrc import lib as _lib
from .errors import ErrorCode, GessoError

F32, BF16 = 0, 1


def _library_mm(x: torch.Tensor, w_t: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """The library matrix product with float32 accumulation from start to end: no bfloat16 intermediate
    sums (split-K partials rounded to 16 bits cost about a digit of accuracy).  The process-wide switch
    is set for the call only and put back."""
    flag = torch.backends.cuda.matmul
    was = flag.allow_bf16_reduced_precision_reduction
    flag.allow_bf16_reduced_precision_reduction = False
    try:
        return torch.mm(x, w_t) if out_dtype is None else torch.mm(x, w_t, out_dtype=out_dtype)
    finally:
        flag.allow_bf16_reduced_precision_reduction = was


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise GessoError(ErrorCode.LAUNCH, f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    # the raw handle of the current stream of the current device (the public accessor builds a Stream
    # object and resolves the device by name: ten times the cost, paid once per kernel launch)
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise GessoError(ErrorCode.LAUNCH, msg)


def _cuda_contig(t: torch.Tensor, name: str, dtype=None) -> None:
    if t.is_cuda and t.is_contiguous() and (dtype is None or t.dtype == dtype):
        return
    _need(t.is_cuda, f"{name} must be a CUDA tensor")
    _need(t.is_contiguous(), f"{name} must be contiguous")
    _need(t.dtype == dtype, f"{name} must be {dtype}, got {t.dtype}")


# ---- embedding / norms ---------------------------------------------------------------------
def embed_gather(tokens: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    _cuda_contig(tokens, "tokens", torch.int32)
    _cuda_contig(table, "table")
    n, (V, H) = tokens.numel(), table.shape
    h = torch.empty((n, H), dtype=torch.float32, device=table.device)
    _lib.check(_lib.library().gesso_embed_gather(_p(tokens), _p(table), _dt(table), _p(h), n, H, V,
                                                 float(scale), _stream()), "embed_gather")
    return h


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], delta_bias: Optional[torch.Tensor],
                weight: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``h += delta (+ bias)`` in place (float32), returns ``rmsnorm(h) * weight`` in ``out_dtype``.

    With ``rows`` only those rows are summed and normed, and ``h`` is left as it was.  ``weight`` may
    be ``None`` (no scaling: the weight was folded into the matrix that consumes the result).
    """
    _cuda_contig(h, "h", torch.float32)
    N, H = h.shape
    if weight is not None:
        _cuda_contig(weight, "weight", torch.float32)
        _need(weight.numel() == H, "norm weight size differs from the row width")
    if delta is not None:
        _cuda_contig(delta, "delta")
        _need(tuple(delta.shape) == (N, H), "delta shape differs from h")
    if delta_bias is not None:
        _cuda_contig(delta_bias, "delta_bias", torch.float32)
        _need(delta is not None and delta_bias.numel() == H, "delta_bias needs a delta of the same width")
    if rows is not None:
        _cuda_contig(rows, "rows", torch.int32)
    n_out = N if rows is None else rows.numel()
    out = torch.empty((n_out, H), dtype=out_dtype, device=h.device)
    _lib.check(_lib.library().gesso_add_rmsnorm(
        _p(h), _p(delta), _dt(delta) if delta is not None else F32, _p(delta_bias), _p(weight),
        float(eps), _p(out), _dt(out), _p(rows), n_out, H, _stream()), "add_rmsnorm")
    return out


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    _cuda_contig(x, "x")
    _cuda_contig(weight, "weight", torch.float32)
    D = x.shape[-1]
    _need(weight.numel() == D, "norm weight size differs from the last axis")
    out = torch.empty_like(x)
    _lib.check(_lib.library().gesso_rmsnorm_rows(_p(x), _p(weight), float(eps), _p(out), _dt(x),
                                                 x.numel() // D, D, _stream()), "rmsnorm_rows")
    return out


# ---- short convolution -----------------------------------------------------------------------
def short_conv(bcx: torch.Tensor, in_bias: Optional[torch.Tensor], taps: torch.Tensor,
               conv_bias: Optional[torch.Tensor], state: torch.Tensor, seg_of_token: torch.Tensor,
               seg_start: torch.Tensor, seg_pos0: torch.Tensor, slots: torch.Tensor,
               n_segs: int, max_seg_len: int, packed: bool = False) -> torch.Tensor:
    """Gated FIR over ``bcx`` [N, 3H]; ``state`` is this layer's view [slots, L-1, H] (float32).
    ``packed``: the columns of ``bcx`` come in groups of 24 (see :func:`pack_bcx`)."""
    _cuda_contig(bcx, "bcx")
    _cuda_contig(taps, "taps", torch.float32)
    N, H3 = bcx.shape
    H, L = taps.shape
    _need(H3 == 3 * H, "bcx width must be three times the tap count")
    _need(state.dtype == torch.float32 and state.is_cuda, "conv state must be float32 on the device")
    _need(state.dim() == 3 and state.shape[1] == L - 1 and state.shape[2] == H
          and state.stride(2) == 1 and state.stride(1) == H, "conv state must be [slots, L-1, H] with dense rows")
    for name, t in (("seg_of_token", seg_of_token), ("seg_start", seg_start), ("seg_pos0", seg_pos0),
                    ("slots", slots)):
        _cuda_contig(t, name, torch.int32)
    out = torch.empty((N, H), dtype=bcx.dtype, device=bcx.device)
    _lib.check(_lib.library().gesso_short_conv(
        _p(bcx), _dt(bcx), _p(in_bias), _p(taps), _p(conv_bias), _p(state), state.stride(0),
        _p(seg_of_token), _p(seg_start), _p(seg_pos0), _p(slots), _p(out), N, n_segs, max_seg_len,
        H, L, 1 if packed else 0, _stream()), "short_conv")
    return out


def pack_bcx(w_in: torch.Tensor) -> torch.Tensor:
    """The short convolution's input projection [3H, K] (rows B, then C, then X) in groups of 24 rows:
    B, C and X of 8 channels (the layout whose convolution the skinny matrix product can run in its
    epilogue).  H % 8 == 0."""
    H3, K = w_in.shape
    H = H3 // 3
    return w_in.reshape(3, H // 8, 8, K).permute(1, 0, 2, 3).reshape(H3, K).contiguous()


def skinny_conv_takes(M: int, w_in: torch.Tensor, x_dtype, L: int) -> bool:
    H3, K = w_in.shape
    return (w_in.dtype == torch.bfloat16 and x_dtype == torch.bfloat16 and w_in.is_contiguous()
            and 1 <= M <= SKINNY_MAX_ROWS and H3 % 24 == 0 and K % 32 == 0 and 2 <= L <= 8)


def linear_conv(x, w_in_packed: torch.Tensor, in_bias: Optional[torch.Tensor], taps: torch.Tensor,
                conv_bias: Optional[torch.Tensor], state: torch.Tensor, seg_pos0: torch.Tensor,
                slots: torch.Tensor) -> torch.Tensor:
    """Input projection and gated FIR in one kernel for a step of single tokens (token i is request i):
    ``x`` is a bfloat16 tensor or a :class:`LazyNorm` of at most 16 rows, ``w_in_packed`` from
    :func:`pack_bcx`; returns y [M, H] and shifts bx into ``state`` [slots, L-1, H]."""
    H3, K = w_in_packed.shape
    H, L = taps.shape
    _need(H3 == 3 * H, "packed input projection must have three rows per channel")
    _need(state.dtype == torch.float32 and state.is_cuda and state.dim() == 3 and state.shape[1] == L - 1
          and state.shape[2] == H and state.stride(2) == 1 and state.stride(1) == H,
          "conv state must be [slots, L-1, H] float32 with dense rows")
    _cuda_contig(taps, "taps", torch.float32)
    _cuda_contig(seg_pos0, "seg_pos0", torch.int32)
    _cuda_contig(slots, "slots", torch.int32)
    x = _skinny_input(x)
    M = x.shape[0]
    _need(slots.numel() >= M and seg_pos0.numel() >= M, "one slot and one position per token")
    if isinstance(x, LazyNorm):
        _cuda_contig(x.h, "h", torch.float32)
        args = (None, _p(x.h), _p(x.weight), x.eps)
    else:
        _cuda_contig(x, "x", torch.bfloat16)
        args = (_p(x), None, None, 0.0)
    y = torch.empty((M, H), dtype=torch.bfloat16, device=w_in_packed.device)
    _lib.check(_lib.library().gesso_skinny_gemm_conv(
        *args, _p(w_in_packed), _p(y), M, H, K, _p(taps), _p(conv_bias), _p(in_bias), _p(state), state.stride(0),
        _p(slots), _p(seg_pos0), L, _stream()), "skinny_gemm_conv")
    return y


# ---- attention ---------------------------------------------------------------------------------
def qk_norm_rope_store(qkv: torch.Tensor, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor],
                       eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                       positions: torch.Tensor, seg_of_token: torch.Tensor, block_table: torch.Tensor,
                       k_pages: torch.Tensor, v_pages: torch.Tensor, nh: int, nkv: int, hd: int,
                       write_kv: bool, status: torch.Tensor, tiles=None, rot_dim: Optional[int] = None,
                       interleaved: bool = False) -> torch.Tensor:
    """Norm + rotate q and k, write k and v into their pages; returns q as [N, nh, hd].  ``tiles`` =
    (seg_start, seg_pos0, tile_seg, tile_q0) of a step with prompt portions lets bfloat16 runs take the
    kernel that works by 64-token tiles (wide loads, v written along the slots of its transposed page).
    ``rot_dim`` (default: the head size) is how many leading features of a head the tables rotate, the
    rest pass through normed; ``interleaved`` pairs neighbours (2i, 2i+1) instead of the two halves."""
    _cuda_contig(qkv, "qkv")
    N = qkv.shape[0]
    heads = nh + 2 * nkv if write_kv else nh
    _need(qkv.shape[1] == heads * hd, "fused projection width differs from the head layout")
    _need(k_pages.dtype == qkv.dtype and v_pages.dtype == qkv.dtype, "cache pages must have the run dtype")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous(), "cache pages must be contiguous")
    _need(k_pages.dim() == 4 and k_pages.shape[1] == nkv and k_pages.shape[3] == hd,
          "K pages must be [pages, kv heads, page size, head size]")
    _need(tuple(v_pages.shape) == (k_pages.shape[0], nkv, hd, k_pages.shape[2]),
          "V pages must be [pages, kv heads, head size, page size]")
    page_size = k_pages.shape[2]
    _cuda_contig(block_table, "block_table", torch.int32)
    _cuda_contig(positions, "positions", torch.int32)
    if cos is not None:
        _cuda_contig(cos, "cos", torch.float32)
        _cuda_contig(sin, "sin", torch.float32)
        rot_dim = hd if rot_dim is None else int(rot_dim)
        _need(2 <= rot_dim <= hd and rot_dim % 2 == 0, "rotary size must be even and at most the head size")
        _need(cos.shape[1] == rot_dim // 2 and sin.shape[1] == rot_dim // 2,
              "rotary table width must be half the rotary size")
    else:
        rot_dim = 0
    q_out = torch.empty((N, nh, hd), dtype=qkv.dtype, device=qkv.device)
    full_half_split = cos is None or (rot_dim == hd and not interleaved)
    if (tiles is not None and write_kv and qkv.dtype == torch.bfloat16 and tiles[2].numel() > 0 and full_half_split
            and _lib.library().gesso_qk_rope_store_tiles_takes(hd, page_size, nh, nkv)):
        seg_start, seg_pos0, tile_seg, tile_q0 = tiles
        _lib.check(_lib.library().gesso_qk_norm_rope_store_tiles(
            _p(qkv), _p(q_w), _p(k_w), float(eps), _p(cos), _p(sin), _p(seg_start), _p(seg_pos0), _p(tile_seg),
            _p(tile_q0), tile_seg.numel(), _p(block_table), block_table.shape[1], page_size, _p(q_out),
            _p(k_pages), _p(v_pages), nh, nkv, hd, _p(status), _stream()), "qk_norm_rope_store_tiles")
        return q_out
    _lib.check(_lib.library().gesso_qk_norm_rope_store(
        _p(qkv), _dt(qkv), _p(q_w), _p(k_w), float(eps), _p(cos), _p(sin), _p(positions),
        _p(seg_of_token), _p(block_table), block_table.shape[1], page_size, _p(q_out), _p(k_pages),
        _p(v_pages), N, nh, nkv, hd, 1 if write_kv else 0, int(rot_dim), 1 if interleaved else 0, _p(status),
        _stream()), "qk_norm_rope_store")
    return q_out


def paged_attention_generic(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                            block_table: torch.Tensor, positions: torch.Tensor,
                            seg_of_token: torch.Tensor, window: Optional[int], scale: float) -> torch.Tensor:
    _cuda_contig(q, "q")
    N, nh, hd = q.shape
    nkv, page_size = k_pages.shape[1], k_pages.shape[2]
    _need(k_pages.dtype == q.dtype, "cache pages must have the dtype of q")
    out = torch.empty((N, nh * hd), dtype=q.dtype, device=q.device)
    _lib.check(_lib.library().gesso_paged_attention_generic(
        _p(q), _p(k_pages), _p(v_pages), _dt(q), _p(block_table), block_table.shape[1], page_size,
        _p(positions), _p(seg_of_token), _p(out), N, nh, nkv, hd, int(window or 0), float(scale),
        _stream()), "paged_attention_generic")
    return out


# ---- feed-forward ------------------------------------------------------------------------------
def swiglu(gu: torch.Tensor, packed: bool = False) -> torch.Tensor:
    """``silu(gate) * up`` on the fused projection [N, 2F].  Plain layout: gate columns first, then
    up columns.  ``packed``: groups of 16 columns hold 8 gate and then the matching 8 up columns."""
    _cuda_contig(gu, "gate_up")
    N, F2 = gu.shape
    _need(F2 % 2 == 0, "fused gate/up width must be even")
    _need(not packed or F2 % 16 == 0, "the packed gate/up layout needs a width that is a multiple of 16")
    out = torch.empty((N, F2 // 2), dtype=gu.dtype, device=gu.device)
    _lib.check(_lib.library().gesso_swiglu(_p(gu), _p(out), _dt(gu), N, F2 // 2, 1 if packed else 0, _stream()),
               "swiglu")
    return out


def fold_norm_weight(w: torch.Tensor, norm_weight: torch.Tensor) -> torch.Tensor:
    """``w[n, k] * norm_weight[k]``: a matrix that takes ``x / rms(x)`` instead of ``rmsnorm(x) * weight``.
    The product is formed in float32 and rounded once to the matrix's own type."""
    return (w.float() * norm_weight.float()[None, :]).to(w.dtype).contiguous()


def pack_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Fused gate/up matrix [2F, H] in groups of 16 rows: 8 gate rows, then the matching 8 up rows
    (the layout whose SwiGLU the skinny matrix product can apply in its epilogue).  F % 8 == 0."""
    F, H = gate.shape
    return torch.stack([gate.reshape(F // 8, 8, H), up.reshape(F // 8, 8, H)], dim=1).reshape(2 * F, H).contiguous()


# ---- matrix products ---------------------------------------------------------------------------
def gemm_f32(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a [M,K] @ w[N,K]^T`` with FP32 FMAs; returns float32."""
    _cuda_contig(a, "a")
    _cuda_contig(w, "w")
    M, K = a.shape
    N, K2 = w.shape
    _need(K == K2, f"inner sizes differ: {K} vs {K2}")
    if bias is not None:
        _cuda_contig(bias, "bias", torch.float32)
    c = torch.empty((M, N), dtype=torch.float32, device=a.device)
    _lib.check(_lib.library().gesso_gemm_f32(_p(a), _dt(a), _p(w), _dt(w), _p(bias), _p(c), M, N, K,
                                             _stream()), "gemm_f32")
    return c


class LazyNorm:
    """A norm that has not run yet: ``rmsnorm(h) * weight`` of the float32 residual stream.

    The skinny matrix product can apply it in its prologue; every other consumer calls
    :meth:`materialize`, which runs the norm kernel.  ``weight`` is ``None`` when the consumer's
    matrix already carries the norm's weight (see :func:`fold_norm_weight`)."""

    def __init__(self, h: torch.Tensor, weight: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype):
        self.h, self.weight, self.eps, self.dtype = h, weight, float(eps), out_dtype
        self.shape = h.shape

    def materialize(self) -> torch.Tensor:
        return add_rmsnorm(self.h, None, None, self.weight, self.eps, self.dtype)


EPI_BF16, EPI_F32, EPI_RESID, EPI_SWIGLU = 0, 1, 2, 3
SKINNY_MAX_ROWS = 16
SKINNY_NORM_MAX_ROWS = 16


def skinny_takes(M: int, w: torch.Tensor, x_dtype) -> bool:
    """Whether the skinny (few-token) matrix product takes this product: bfloat16 operands, at most
    16 rows, an output width that is a multiple of 16 and an inner size that is a multiple of 32."""
    N, K = w.shape
    return (w.dtype == torch.bfloat16 and x_dtype == torch.bfloat16 and w.is_contiguous() and 1 <= M <= SKINNY_MAX_ROWS
            and N >= 16 and N % 16 == 0 and K >= 32 and K % 32 == 0)


# Steps of at least this many tokens take this library's tcgen05 matrix product (TMA-fed, accumulators
# in tensor memory, residual add / SwiGLU in its epilogue); between the skinny kernel's rows and this
# the library product is used, whose small-tile and split-K variants are faster there.
TC_MIN_ROWS = int(os.environ.get("GESSO_TC_MIN_ROWS", "1024"))


def tc_takes(M: int, w: torch.Tensor, x_dtype) -> bool:
    """Whether the tcgen05 matrix product takes this product: bfloat16 operands, at least TC_MIN_ROWS
    rows, inner and output sizes that are multiples of 8 (16-byte rows for TMA and vector stores)."""
    N, K = w.shape
    return (w.dtype == torch.bfloat16 and x_dtype == torch.bfloat16 and w.is_contiguous() and M >= TC_MIN_ROWS
            and N >= 8 and N % 8 == 0 and K >= 8 and K % 8 == 0 and w.data_ptr() % 16 == 0
            and _tc_wave_efficiency(M, N) >= TC_MIN_WAVE_EFFICIENCY)


# The tcgen05 kernels walk whole tiles, one wave of (pairs of) SMs after the other; where the last wave is
# mostly empty (few tokens times a narrow output) the library's smaller tiles and split-K variants win.
TC_MIN_WAVE_EFFICIENCY = 0.8


def _tc_wave_efficiency(M: int, N: int) -> float:
    if M >= 256 and N >= 256:
        tiles, slots = -(-M // 256) * -(-N // 256), sm_count() // 2        # pairs of blocks, 256 x 256 tiles
    else:
        tiles, slots = -(-M // 128) * -(-N // 256), sm_count()
    return tiles / (-(-tiles // slots) * slots)


_skinny_ws = {}
SKINNY_WS_BYTES = 16 * 1024 + 4 * 1024 * 1024


def _device_index(device) -> int:
    """``cuda`` and ``cuda:0`` name the same device: workspaces are kept by index."""
    d = torch.device(device)
    return d.index if d.index is not None else torch.cuda.current_device()


def _skinny_workspace(device) -> torch.Tensor:
    """Tickets and partial tiles for skinny products that are split along K: one zeroed buffer per
    device and stream (launches on one stream run in order, so they can share it)."""
    idx = _device_index(device)
    key = (idx, torch._C._cuda_getCurrentRawStream(idx))
    ws = _skinny_ws.get(key)
    if ws is None:
        ws = _skinny_ws[key] = torch.zeros((SKINNY_WS_BYTES,), dtype=torch.uint8, device=device)
    return ws


def ensure_workspaces(device, stream) -> None:
    """Create the zeroed workspace of the skinny matrix product for ``stream`` now (on the current stream),
    so that a graph captured on ``stream`` does not record its allocation and zero fill."""
    with torch.cuda.stream(stream):
        _skinny_workspace(device)
    torch.cuda.current_stream(device).wait_stream(stream)


def _skinny(x, w, out, bias, epi):
    """x: bfloat16 tensor or LazyNorm with at most SKINNY_NORM_MAX_ROWS rows."""
    N, K = w.shape
    if isinstance(x, LazyNorm):
        M = x.shape[0]
        _cuda_contig(x.h, "h", torch.float32)
        args = (None, _p(x.h), _p(x.weight), x.eps)
    else:
        M = x.shape[0]
        _cuda_contig(x, "x", torch.bfloat16)
        args = (_p(x), None, None, 0.0)
    ws = _skinny_workspace(w.device)
    _lib.check(_lib.library().gesso_skinny_gemm(*args, _p(w), _p(out), _p(bias), M, N, K, epi, _p(ws), ws.numel(),
                                                _stream()), "skinny_gemm")


def _as_tensor(x):
    return x.materialize() if isinstance(x, LazyNorm) else x


def _skinny_input(x):
    if isinstance(x, LazyNorm) and x.shape[0] > SKINNY_NORM_MAX_ROWS:
        return x.materialize()
    return x


def linear(x, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x @ w^T`` for a weight stored (out, in); ``x`` is a tensor or a :class:`LazyNorm`.

    bfloat16 activations with a bfloat16 weight use the tensor cores with float32 accumulation
    (this library's skinny kernel for steps of few tokens, the library matrix product otherwise);
    any float32 operand (the 32-bit path, or a matrix that was stored in 32 bit) uses the FP32 FMA
    kernel, so no reduced-precision mode is ever applied to 32-bit data.
    """
    out_dtype = out_dtype or x.dtype
    M = x.shape[0]
    if skinny_takes(M, w, x.dtype) and out_dtype in (torch.bfloat16, torch.float32):
        out = torch.empty((M, w.shape[0]), dtype=out_dtype, device=w.device)
        _skinny(_skinny_input(x), w, out, None, EPI_BF16 if out_dtype == torch.bfloat16 else EPI_F32)
        return out
    x = _as_tensor(x)
    if few_takes(M, w, x.dtype) and out_dtype in (torch.bfloat16, torch.float32):
        return gemm_tcgen05_few(x, w, EPI_BF16 if out_dtype == torch.bfloat16 else EPI_F32)
    if tc_takes(M, w, x.dtype) and out_dtype in (torch.bfloat16, torch.float32):
        return gemm_tcgen05(x, w, EPI_BF16 if out_dtype == torch.bfloat16 else EPI_F32)
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        _cuda_contig(x, "x")
        if out_dtype == torch.bfloat16:
            return _library_mm(x, w.t())
        return _library_mm(x, w.t(), torch.float32)
    c = gemm_f32(x, w)
    return c if out_dtype == torch.float32 else c.to(out_dtype)


def linear_residual(x, w: torch.Tensor, h: torch.Tensor, bias: Optional[torch.Tensor]):
    """``h += x @ w^T (+ bias)`` when the skinny kernel can add in its epilogue (returns ``None``);
    otherwise returns the product for the caller to pass on as a pending residual."""
    M = x.shape[0]
    if skinny_takes(M, w, x.dtype) and tuple(h.shape) == (M, w.shape[0]):
        _cuda_contig(h, "h", torch.float32)
        _skinny(_as_tensor(x), w, h, bias, EPI_RESID)
        return None
    if few_takes(M, w, x.dtype) and tuple(h.shape) == (M, w.shape[0]):
        gemm_tcgen05_few(_as_tensor(x), w, EPI_RESID, out=h, bias=bias)
        return None
    # Steps of many tokens hand the product on as a pending bfloat16 delta: the next norm kernel adds
    # it while it reads the residual stream anyway, which moves fewer bytes than a read-modify-write
    # of the float32 stream in the product's epilogue (measured: 15.7 vs 38.7 us at 2040 x 2048 x 2048).
    return linear(x, w, out_dtype=x.dtype)


def linear_swiglu(x, w_gate_up: torch.Tensor, packed: bool) -> torch.Tensor:
    """``silu(gate(x)) * up(x)`` for the fused gate/up matrix (see :func:`pack_gate_up`)."""
    M = x.shape[0]
    if packed and skinny_takes(M, w_gate_up, x.dtype):
        out = torch.empty((M, w_gate_up.shape[0] // 2), dtype=torch.bfloat16, device=w_gate_up.device)
        _skinny(_skinny_input(x), w_gate_up, out, None, EPI_SWIGLU)
        return out
    if packed and few_takes(M, w_gate_up, x.dtype) and w_gate_up.shape[0] % 16 == 0:
        return gemm_tcgen05_few(_as_tensor(x), w_gate_up, EPI_SWIGLU)
    if packed and tc_takes(M, w_gate_up, x.dtype) and w_gate_up.shape[0] % 16 == 0:
        return gemm_tcgen05(_as_tensor(x), w_gate_up, EPI_SWIGLU)
    return swiglu(linear(x, w_gate_up, out_dtype=x.dtype), packed)


_lib.declare("gesso_logit_transform", [_lib.P, _lib.LL, _lib.F, _lib.F])


def logit_transform(logits: torch.Tensor, scale: float = 1.0, softcap: Optional[float] = None) -> torch.Tensor:
    """``softcap * tanh(scale * logits / softcap)`` (``scale * logits`` without a cap), in place on float32 logits."""
    _cuda_contig(logits, "logits", torch.float32)
    _need(softcap is None or softcap > 0, "the soft cap must be positive")
    _lib.check(_lib.library().gesso_logit_transform(_p(logits), logits.numel(), float(scale), float(softcap or 0.0),
                                                   _stream()), "logit_transform")
    return logits


# ---- sampling ----------------------------------------------------------------------------------
def argmax_rows(logits: torch.Tensor, host_out: Optional[torch.Tensor] = None):
    """Greedy ids and non-finite flags of every row.  ``host_out``: pinned host int32 ``[2, R]`` that the
    kernel writes the same two rows into (no copy of its own is needed then; valid once the stream has
    passed the kernel)."""
    _cuda_contig(logits, "logits", torch.float32)
    R, V = logits.shape
    if host_out is not None:
        _need(host_out.dtype == torch.int32 and host_out.is_pinned() and host_out.is_contiguous()
              and tuple(host_out.shape) == (2, R), "argmax host output must be pinned int32 [2, rows]")
    both = torch.empty((2, R), dtype=torch.int32, device=logits.device)   # one buffer: one copy to the host
    ids, bad = both[0], both[1]
    sv = si = None
    if V >= 8192:      # wide rows are scanned by 32 blocks each; their partial results need scratch
        sv = torch.empty((R * 32,), dtype=torch.float32, device=logits.device)
        si = torch.empty((R * 64,), dtype=torch.int32, device=logits.device)
    _lib.check(_lib.library().gesso_argmax_rows(_p(logits), R, V, _p(ids), _p(bad), _p(sv), _p(si),
                                                host_out.data_ptr() if host_out is not None else None, _stream()),
               "argmax_rows")
    return ids, bad


KERNEL_COPIES = os.environ.get("GESSO_KERNEL_COPIES", "1") != "0"
KERNEL_COPY_MAX_WORDS = 1 << 18      # above 1 MB the copy engine is the better mover


def copy_words(segments) -> None:
    """Copy 32-bit words between device memory and pinned host memory with one kernel launch on the current
    stream: ``segments`` is a list of up to six ``(dst, src, n_words)``, ``dst`` / ``src`` being ``(tensor,
    first word)`` pairs (int32 tensors, contiguous; a host tensor must be pinned).  The segments of one call
    must not overlap.  Between decoding steps this replaces memcpy operations, each of which costs a change
    between the compute and the copy engines."""
    n = len(segments)
    _need(1 <= n <= 6, "copy_words takes one to six segments")
    dst, src, cnt = (ctypes.c_void_p * n)(), (ctypes.c_void_p * n)(), (ctypes.c_longlong * n)()
    for k, ((dt, d0), (st, s0), words) in enumerate(segments):
        for t, at in ((dt, d0), (st, s0)):
            _need(t.dtype == torch.int32 and t.is_contiguous() and (t.is_cuda or t.is_pinned()),
                  "copy_words takes contiguous int32 tensors on the device or in pinned host memory")
            _need(0 <= at and at + words <= t.numel() and words >= 0, "copy_words: a segment leaves its tensor")
        dst[k], src[k], cnt[k] = dt.data_ptr() + 4 * d0, st.data_ptr() + 4 * s0, words
    _lib.check(_lib.library().gesso_copy_words(n, dst, src, cnt, _stream()), "copy_words")


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, u: torch.Tensor):
    _cuda_contig(logits, "logits", torch.float32)
    _cuda_contig(temperature, "temperature", torch.float64)
    _cuda_contig(top_p, "top_p", torch.float64)
    _cuda_contig(u, "u", torch.float64)
    R, V = logits.shape
    _need(temperature.numel() == R and top_p.numel() == R and u.numel() == R, "one parameter per row")
    ids = torch.empty((R,), dtype=torch.int32, device=logits.device)
    bad = torch.empty((R,), dtype=torch.int32, device=logits.device)
    # the weights of a row are computed once into this scratch and read back by the later passes
    wcache = torch.empty((R, V), dtype=torch.float64, device=logits.device) if R * V <= (1 << 27) else None
    _lib.check(_lib.library().gesso_sample_rows(_p(logits), R, V, _p(temperature), _p(top_p), _p(u),
                                                _p(ids), _p(bad), _p(wcache), _stream()), "sample_rows")
    return ids, bad


_lib.declare("gesso_qk_rope_store_tiles_takes", [_lib.I, _lib.I, _lib.I, _lib.I])
_lib.declare("gesso_qk_norm_rope_store_tiles", [_lib.P, _lib.P, _lib.P, _lib.F, _lib.P, _lib.P, _lib.P, _lib.P, _lib.P,
                                                _lib.P, _lib.I, _lib.P, _lib.I, _lib.I, _lib.P, _lib.P, _lib.P, _lib.I,
                                                _lib.I, _lib.I, _lib.P, _lib.P])

# ---- tensor-core attention (bfloat16) ------------------------------------------------------------
_lib.declare("gesso_attention_tc_takes", [_lib.I, _lib.I, _lib.I, _lib.I])
_lib.declare("gesso_decode_attention", [_lib.P, _lib.P, _lib.P, _lib.P, _lib.I, _lib.I, _lib.P, _lib.P,
                                        _lib.I, _lib.I, _lib.I, _lib.I, _lib.I, _lib.F, _lib.I, _lib.P, _lib.P,
                                        _lib.P, _lib.P, _lib.P])
_lib.declare("gesso_prefill_attention", [_lib.P, _lib.P, _lib.P, _lib.P, _lib.I, _lib.I, _lib.P, _lib.P, _lib.P,
                                         _lib.P, _lib.I, _lib.P, _lib.I, _lib.I, _lib.I, _lib.I, _lib.F, _lib.P])

_lib.declare("gesso_sm_count", [])
_sm_count = 0


def sm_count() -> int:
    """Streaming multiprocessors of the current device (148 on a B200), asked of the device once."""
    global _sm_count
    if _sm_count == 0:
        _sm_count = int(_lib.library().gesso_sm_count())
        _need(_sm_count > 0, "cannot read the device's multiprocessor count")
    return _sm_count


def fast_attention_takes(hd: int, page_size: int, nh: int, nkv: int) -> bool:
    """Sizes the tensor-core attention kernels take: head 32/64/96/128, pages in multiples of 16
    slots, at most 16 query heads per kv head for single-token steps."""
    return bool(_lib.library().gesso_attention_tc_takes(hd, page_size, nh, nkv)) and nh // nkv <= 16


DECODE_BLOCKS_PER_SM = int(os.environ.get("GESSO_DECODE_BLOCKS_PER_SM", "2"))


DECODE_UNEVEN_SPLITS = int(os.environ.get("GESSO_DECODE_UNEVEN_SPLITS", "4"))


def decode_splits(n_segs: int, nkv: int, max_kv_len: int, uneven: bool = False) -> int:
    """The most pieces the keys of a request are cut into: so many that about DECODE_BLOCKS_PER_SM blocks
    per SM are busy; with ``uneven`` (the kernel is told the step's lengths and cuts a request that is long
    among short ones even where the batch alone fills the device) at least DECODE_UNEVEN_SPLITS for more
    than one request."""
    blocks = (max_kv_len + 15) // 16
    want = (DECODE_BLOCKS_PER_SM * sm_count()) // (n_segs * nkv)      # rounded down: all blocks resident at once
    if uneven and n_segs > 1:
        want = max(want, DECODE_UNEVEN_SPLITS)
    # at least 16 blocks (256 keys) per split: finer splits cost more in their set-up and in the merge of
    # the parts than they win (one request at 4,096 keys: 1,393 tokens/s with 16 splits, 1,226 with 37)
    return max(1, min(want, (blocks + 15) // 16))


def decode_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     block_table: torch.Tensor, positions: torch.Tensor,
                     window: Optional[int], scale: float, n_splits: int,
                     workspace=None, kv_span: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Split-KV attention for a step of single tokens (token i is request i).  ``workspace`` = (part_o, part_ml, tickets) of
    sizes [segs*nh*splits*hd], [segs*nh*splits*2] float32 and [segs*nkv] int32 (zeroed once).  ``kv_span``: int32 [2]
    on the device, the longest sequence of the step and the average one: a request then uses as many of the
    ``n_splits`` pieces as the step's lengths call for (without it, all of them)."""
    _cuda_contig(q, "q", torch.bfloat16)
    S, nh, hd = q.shape
    nkv, page_size = k_pages.shape[1], k_pages.shape[2]
    _need(k_pages.dtype == torch.bfloat16 and v_pages.dtype == torch.bfloat16, "cache pages must be bfloat16")
    if kv_span is not None:
        _cuda_contig(kv_span, "kv_span", torch.int32)
        _need(kv_span.numel() == 2, "kv_span holds two numbers")
    out = torch.empty((S, nh * hd), dtype=q.dtype, device=q.device)
    if n_splits > 1:
        if workspace is None:
            workspace = (torch.empty((S * nh * n_splits * hd,), dtype=torch.float32, device=q.device),
                         torch.empty((S * nh * n_splits * 2,), dtype=torch.float32, device=q.device),
                         torch.zeros((S * nkv,), dtype=torch.int32, device=q.device))
        part_o, part_ml, tickets = workspace
        _need(part_o.numel() >= S * nh * n_splits * hd and part_ml.numel() >= S * nh * n_splits * 2
              and tickets.numel() >= S * nkv, "split-KV workspace is too small")
    else:
        part_o = part_ml = tickets = None
    _lib.check(_lib.library().gesso_decode_attention(
        _p(q), _p(k_pages), _p(v_pages), _p(block_table), block_table.shape[1], page_size, _p(positions),
        _p(out), S, nh, nkv, hd, int(window or 0), float(scale), int(n_splits), _p(part_o),
        _p(part_ml), _p(tickets), _p(kv_span), _stream()), "decode_attention")
    return out


def prefill_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      block_table: torch.Tensor, seg_start: torch.Tensor, seg_pos0: torch.Tensor,
                      tile_seg: torch.Tensor, tile_q0: torch.Tensor, window: Optional[int],
                      scale: float) -> torch.Tensor:
    _cuda_contig(q, "q", torch.bfloat16)
    N, nh, hd = q.shape
    nkv, page_size = k_pages.shape[1], k_pages.shape[2]
    out = torch.empty((N, nh * hd), dtype=q.dtype, device=q.device)
    _lib.check(_lib.library().gesso_prefill_attention(
        _p(q), _p(k_pages), _p(v_pages), _p(block_table), block_table.shape[1], page_size, _p(seg_start),
        _p(seg_pos0), _p(tile_seg), _p(tile_q0), tile_seg.numel(), _p(out), nh, nkv, hd, int(window or 0),
        float(scale), _stream()), "prefill_attention")
    return out


# ---- tcgen05 matrix product (steps of many tokens) ---------------------------------------------------
_lib.declare("gesso_gemm_tcgen05_takes", [_lib.I, _lib.I, _lib.I])
_lib.declare("gesso_gemm_tcgen05", [_lib.P, _lib.P, _lib.P, _lib.P, _lib.I, _lib.I, _lib.I, _lib.I, _lib.P, _lib.P])

_tc_status = {}
_tc_status_scope: list = []


def tc_status_tensor(device) -> torch.Tensor:
    """The int32 word that a tcgen05 kernel writes when one of its bounded waits runs out: the word of
    the innermost :class:`tc_status_scope` (an engine's own, so that a step's failure is seen by the
    engine that ran it), else one word per device."""
    if _tc_status_scope:
        return _tc_status_scope[-1]
    key = _device_index(device)
    if key not in _tc_status:
        _tc_status[key] = torch.zeros((1,), dtype=torch.int32, device=device)
    return _tc_status[key]


class tc_status_scope:
    """``with tc_status_scope(word):`` every tcgen05 kernel launched (or captured into a graph) inside
    reports an exhausted wait to ``word`` (int32 [1] on the device)."""

    def __init__(self, word: torch.Tensor):
        self.word = word

    def __enter__(self):
        _tc_status_scope.append(self.word)
        return self.word

    def __exit__(self, *exc):
        _tc_status_scope.pop()
        return False


def tc_wait_error(code: int) -> GessoError:
    return GessoError(ErrorCode.RUNTIME, f"a tcgen05 kernel gave up on a pipeline wait (role code {code}); "
                      "what it computed is not valid")


def check_tc_status(device="cuda") -> None:
    """Raise if a tcgen05 kernel gave up on a wait since the last check (synchronises).  Kernels
    launched by an engine's steps report to the engine instead (``Engine.check_status``)."""
    st = tc_status_tensor(device)
    code = int(st.item())
    if code != 0:
        st.zero_()
        raise tc_wait_error(code)


_lib.declare("gesso_gemm_tcgen05_pair_takes", [_lib.I, _lib.I, _lib.I])
_lib.declare("gesso_gemm_tcgen05_pair", [_lib.P, _lib.P, _lib.P, _lib.P, _lib.I, _lib.I, _lib.I, _lib.I, _lib.P, _lib.P])
TC_PAIR = os.environ.get("GESSO_TC_PAIR", "1") != "0"


_lib.declare("gesso_gemm_tcgen05_few_takes", [_lib.I, _lib.I, _lib.I])
_lib.declare("gesso_gemm_tcgen05_few", [_lib.P, _lib.P, _lib.P, _lib.P, _lib.I, _lib.I, _lib.I, _lib.I, _lib.I, _lib.P,
                                        _lib.P])
FEW_MAX_ROWS = 128
# The few-row tcgen05 product (17 .. 128 tokens; W streamed once, SwiGLU or the residual add in the
# epilogue) is an option, GESSO_TC_FEW=1, for matrices of TC_FEW_MIN_BYTES or more.  Alone it ties with
# the library at 64 rows (14.9 us against 12.8 + 3.5 for the SwiGLU kernel at 16384 x 2048, 48 against
# 53 us at 65536 x 2048, 13.1 against 13.0 at 2048 x 8192; smaller matrices lose: 11.5 against 6.7 us at
# 6144 x 2048, a cluster's exchange through shared memory costs about 3 us), but inside a decoding step
# of 64 requests the library's kernels came out 1 to 3 % ahead (their start overlaps the preceding
# kernel; a block of this one holds a whole SM), so they are the default.
TC_FEW = os.environ.get("GESSO_TC_FEW", "0") == "1"
TC_FEW_MIN_BYTES = int(float(os.environ.get("GESSO_TC_FEW_MIN_MB", "32")) * (1 << 20))


def few_takes(M: int, w: torch.Tensor, x_dtype) -> bool:
    """Whether the few-row tcgen05 matrix product takes this product: bfloat16 operands, 17 .. 128 rows,
    an inner size that is a multiple of 8 (16-byte rows for TMA), a matrix of TC_FEW_MIN_BYTES or more."""
    N, K = w.shape
    return (TC_FEW and w.dtype == torch.bfloat16 and x_dtype == torch.bfloat16 and w.is_contiguous()
            and SKINNY_MAX_ROWS < M <= FEW_MAX_ROWS and N >= 8 and K >= 8 and K % 8 == 0 and w.data_ptr() % 16 == 0
            and N * K * 2 >= TC_FEW_MIN_BYTES)


def gemm_tcgen05_few(x: torch.Tensor, w: torch.Tensor, epi: int = EPI_BF16, out: Optional[torch.Tensor] = None,
                     bias: Optional[torch.Tensor] = None, cluster: int = 0) -> torch.Tensor:
    """``x [M,K] @ w [N,K]^T`` for at most 128 rows on the tcgen05 tensor cores with the operands swapped
    (128 rows of ``w`` per MMA, the tokens on its N side); ``epi`` and ``out`` as in :func:`gemm_tcgen05`.
    ``cluster``: blocks that share a tile along K (0: the kernel chooses; 1, 2, 4, 8: where that fits)."""
    _cuda_contig(x, "x", torch.bfloat16)
    _cuda_contig(w, "w", torch.bfloat16)
    M, K = x.shape
    N, K2 = w.shape
    _need(K == K2, f"inner sizes differ: {K} vs {K2}")
    if epi == EPI_RESID:
        _need(out is not None and out.dtype == torch.float32 and tuple(out.shape) == (M, N), "residual must be float32 [M,N]")
        _cuda_contig(out, "out")
    elif epi == EPI_SWIGLU:
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    else:
        out = torch.empty((M, N), dtype=torch.bfloat16 if epi == EPI_BF16 else torch.float32, device=x.device)
    _lib.check(_lib.library().gesso_gemm_tcgen05_few(_p(x), _p(w), _p(out), _p(bias), M, N, K, epi, int(cluster),
                                                     _p(tc_status_tensor(x.device)), _stream()), "gemm_tcgen05_few")
    return out


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, epi: int = EPI_BF16, out: Optional[torch.Tensor] = None,
                 bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x [M,K] @ w [N,K]^T`` on the tcgen05 tensor cores (TMA-fed, accumulators in tensor memory).

    ``epi``: EPI_BF16 / EPI_F32 give a new tensor; EPI_RESID adds into ``out`` (float32 [M,N], with
    ``bias``); EPI_SWIGLU gives ``silu(gate) * up`` [M, N/2] for packed gate/up rows of ``w``."""
    _cuda_contig(x, "x", torch.bfloat16)
    _cuda_contig(w, "w", torch.bfloat16)
    M, K = x.shape
    N, K2 = w.shape
    _need(K == K2, f"inner sizes differ: {K} vs {K2}")
    if epi == EPI_RESID:
        _need(out is not None and out.dtype == torch.float32 and tuple(out.shape) == (M, N), "residual must be float32 [M,N]")
        _cuda_contig(out, "out")
    elif epi == EPI_SWIGLU:
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    else:
        out = torch.empty((M, N), dtype=torch.bfloat16 if epi == EPI_BF16 else torch.float32, device=x.device)
    lib = _lib.library()
    # from 256 rows and columns on, two blocks share a 256 x 256 tile (a third less operand traffic per SM)
    if TC_PAIR and lib.gesso_gemm_tcgen05_pair_takes(M, N, K):
        _lib.check(lib.gesso_gemm_tcgen05_pair(_p(x), _p(w), _p(out), _p(bias), M, N, K, epi,
                                               _p(tc_status_tensor(x.device)), _stream()), "gemm_tcgen05_pair")
    else:
        _lib.check(lib.gesso_gemm_tcgen05(_p(x), _p(w), _p(out), _p(bias), M, N, K, epi,
                                          _p(tc_status_tensor(x.device)), _stream()), "gemm_tcgen05")
    return out


# ---- tcgen05 flash prefill attention -----------------------------------------------------------------
_lib.declare("gesso_attention_tcgen05_takes", [_lib.I, _lib.I, _lib.I, _lib.I])
_lib.declare("gesso_prefill_attention_tcgen05", [_lib.P, _lib.P, _lib.P, _lib.I, _lib.P, _lib.I, _lib.I, _lib.P, _lib.P,
                                                 _lib.P, _lib.P, _lib.I, _lib.I, _lib.P, _lib.I, _lib.I, _lib.I, _lib.F,
                                                 _lib.P, _lib.P])


def attention_tcgen05_takes(hd: int, page_size: int, nh: int, nkv: int) -> bool:
    """Head size 64, pages in multiples of 16 slots, 2 to 16 query heads per kv head."""
    return bool(_lib.library().gesso_attention_tcgen05_takes(hd, page_size, nh, nkv))


def prefill_attention_tcgen05(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                              block_table: torch.Tensor, seg_start: torch.Tensor, seg_pos0: torch.Tensor,
                              tile_seg: torch.Tensor, tile_q0: torch.Tensor, window: Optional[int],
                              scale: float) -> torch.Tensor:
    """Flash prefill attention on tcgen05 (S and P in tensor memory, K/V pages by TMA)."""
    _cuda_contig(q, "q", torch.bfloat16)
    N, nh, hd = q.shape
    nkv, page_size = k_pages.shape[1], k_pages.shape[2]
    _need(k_pages.is_contiguous() and v_pages.is_contiguous(), "cache pages must be contiguous")
    out = torch.empty((N, nh * hd), dtype=q.dtype, device=q.device)
    _lib.check(_lib.library().gesso_prefill_attention_tcgen05(
        _p(q), _p(k_pages), _p(v_pages), k_pages.shape[0], _p(block_table), block_table.shape[1], page_size,
        _p(seg_start), _p(seg_pos0), _p(tile_seg), _p(tile_q0), tile_seg.numel(), N, _p(out), nh, nkv,
        int(window or 0), float(scale), _p(tc_status_tensor(q.device)), _stream()), "prefill_attention_tcgen05")
    return out
