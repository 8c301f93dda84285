"""Loading a model folder (or drawing random weights) into a bound :class:`Model`."""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from .config.registry import spec_from_config, spec_from_dir
from .engine.model import Model
from .errors import ErrorCode, GessoError, invalid
from .weights.loader import load_model_tensors
from .weights.random_init import random_tensors

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, "f32": torch.float32}


def run_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name in (torch.bfloat16, torch.float32):
            return name
    elif str(name) in _DTYPES:
        return _DTYPES[str(name)]
    raise invalid(f"dtype must be bfloat16 or float32, got {name!r}")


def require_cuda(device="cuda") -> torch.device:
    """The engine runs on a CUDA device only; there is no CPU path."""
    if not torch.cuda.is_available():
        raise GessoError(ErrorCode.COMPILE, "no CUDA device: this engine runs on an NVIDIA B200 "
                         "(sm_100a) and has no CPU fallback")
    return torch.device(device)


def load(model_dir: str, dtype="bfloat16", device="cuda", max_positions: Optional[int] = None) -> Model:
    """Model folder (config.json + model.safetensors) -> bound model on the device."""
    dev = require_cuda(device)
    spec = spec_from_dir(model_dir)
    tensors, _ = load_model_tensors(model_dir, spec)
    return Model(spec, tensors, run_dtype(dtype), dev, max_positions or spec.max_position or 4096)


def random_model(config: Mapping, seed: int = 0, dtype="bfloat16", device="cuda",
                 max_positions: Optional[int] = None, std: float = 0.02, style: str = "normal",
                 weights_dtype: str = "bfloat16") -> Model:
    """Random weights drawn on the device from ``config`` and ``seed`` (no folder is written)."""
    dev = require_cuda(device)
    spec = spec_from_config(config)
    tensors = random_tensors(spec, seed, dtype=weights_dtype, std=std, style=style, device=str(dev))
    return Model(spec, tensors, run_dtype(dtype), dev, max_positions or spec.max_position or 4096)
