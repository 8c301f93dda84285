"""Loads the kernel library and declares its C entry points.

The library is opened with ``ctypes``; every entry point takes raw device
pointers, sizes and a CUDA stream handle.  Loading fails loudly: there is no
fallback path that could stand in for a missing library.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_double, c_float, c_int, c_longlong, c_void_p

from ..errors import ErrorCode, GessoError
from . import build as _build

_lock = threading.Lock()
_lib = None

P = c_void_p
I = c_int
F = c_float
LL = c_longlong

# name -> argtypes (the CUDA stream is always the last argument)
_SIGNATURES = {
    "gesso_embed_gather": [P, P, I, P, I, I, I, F, P],
    "gesso_add_rmsnorm": [P, P, I, P, P, F, P, I, P, I, I, P],
    "gesso_rmsnorm_rows": [P, P, F, P, I, I, I, P],
    "gesso_short_conv": [P, I, P, P, P, P, LL, P, P, P, P, P, I, I, I, I, I, I, P],
    "gesso_skinny_conv_takes": [I, I, I, I],
    "gesso_skinny_gemm_conv": [P, P, P, F, P, P, I, I, I, P, P, P, P, LL, P, P, I, P],
    "gesso_qk_norm_rope_store": [P, I, P, P, F, P, P, P, P, P, I, I, P, P, P, I, I, I, I, I, I, I, P, P],
    "gesso_paged_attention_generic": [P, P, P, I, P, I, I, P, P, P, I, I, I, I, I, F, P],
    "gesso_swiglu": [P, P, I, I, I, I, P],
    "gesso_skinny_gemm_takes": [I, I, I],
    "gesso_skinny_gemm": [P, P, P, F, P, P, P, I, I, I, I, P, LL, P],
    "gesso_gemm_f32": [P, I, P, I, P, P, I, I, I, P],
    "gesso_argmax_rows": [P, I, I, P, P, P, P, P, P],
    "gesso_copy_words": [I, P, P, P, P],
    "gesso_sample_rows": [P, I, I, P, P, P, P, P, P, P],
}

_REFUSALS = {-2: "unsupported dtype", -3: "a size this kernel does not take",
             -4: "unsupported configuration"}


def library():
    """The loaded library (built at the first call if it is stale or missing)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _build.build(verbose=True)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise GessoError(ErrorCode.COMPILE, f"cannot load {path}: {e}") from None
        for name, argtypes in _SIGNATURES.items():
            try:
                fn = getattr(lib, name)
            except AttributeError:
                continue   # optional entry points are declared where they are used
            fn.argtypes = argtypes
            fn.restype = c_int
        if hasattr(lib, "gesso_set_pdl"):
            lib.gesso_set_pdl.argtypes = [c_int]
            lib.gesso_set_pdl.restype = c_int
            # GESSO_PDL=0 launches the kernels of decoding steps without programmatic dependent launch
            lib.gesso_set_pdl(0 if os.environ.get("GESSO_PDL", "1") == "0" else 1)
        _lib = lib
        return lib


def declare(name: str, argtypes) -> None:
    """Declare one more entry point (kernels added in their own files register here)."""
    _SIGNATURES[name] = list(argtypes)
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.argtypes = list(argtypes)
        fn.restype = c_int


_launches = 0


def launch_count() -> int:
    """How many kernel launchers of this library have been called so far (by this process)."""
    return _launches


def check(status: int, what: str) -> None:
    global _launches
    _launches += 1
    if status == 0:
        return
    if status < 0:
        raise GessoError(ErrorCode.LAUNCH, f"{what}: refused: {_REFUSALS.get(status, status)}")
    raise GessoError(ErrorCode.LAUNCH, f"{what}: CUDA error {status} at launch")


__all__ = ["library", "check", "declare", "launch_count", "c_double", "P", "I", "F", "LL"]
