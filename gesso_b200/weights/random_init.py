"""Random-weights mode: a model folder from a configuration and a seed.

Matrices, conv taps and biases are N(0, std) (``std`` 0.02 by default; ``style="fan_in"``
draws N(0, 1/fan_in) and norm weights 1 + 0.1 N(0,1), as the reference's toy fixtures do,
test/lfm25_toy.jl:28-41); norm weights are 1.  Tensors are drawn in the order of their
sorted internal names from one seeded generator, in float32, then rounded to the storage
type: matrices to ``dtype`` (bfloat16 by default), small vectors stay float32.  The folder
holds ``config.json`` and ``model.safetensors`` under the checkpoint's canonical names.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Mapping, Optional

import torch

from ..config.registry import spec_from_config
from ..config.spec import ModelSpec
from ..errors import invalid
from .loader import model_param_decls
from .safetensors_io import write_safetensors_file

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def random_tensors(spec: ModelSpec, seed: int, dtype: str = "bfloat16", std: float = 0.02,
                   style: str = "normal", device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Internal name -> tensor, drawn as the module docstring says."""
    if dtype not in _STORE:
        raise invalid(f"random weights: dtype must be one of {sorted(_STORE)}")
    if style not in ("normal", "fan_in"):
        raise invalid("random weights: style must be 'normal' or 'fan_in'")
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}
    decls = model_param_decls(spec)
    for name in sorted(decls):
        d = decls[name]
        if d.role == "table":
            out[name] = torch.zeros(d.shape, dtype=torch.int32, device=device)
            continue
        if d.init == "ones":
            t = torch.ones(d.shape, dtype=torch.float32, device=device)
            if style == "fan_in":
                t = t + 0.1 * torch.randn(d.shape, generator=gen, dtype=torch.float32, device=device)
        elif d.init == "zeros":
            t = torch.zeros(d.shape, dtype=torch.float32, device=device)
        else:
            t = torch.randn(d.shape, generator=gen, dtype=torch.float32, device=device)
            if style == "fan_in":
                fan = d.fan_in or (d.shape[-1] if len(d.shape) > 1 else 1)
                t = t / float(fan) ** 0.5 if len(d.shape) > 1 else t * 0.1
            else:
                t = t * std
        out[name] = t.to(_STORE[dtype]) if d.role == "matrix" else t
    return out


def write_random_model(model_dir: str, config: Mapping, seed: int, dtype: str = "bfloat16",
                       std: float = 0.02, style: str = "normal",
                       spec: Optional[ModelSpec] = None) -> ModelSpec:
    """Write ``config.json`` and ``model.safetensors`` into ``model_dir`` (created if absent)."""
    spec = spec or spec_from_config(config)
    os.makedirs(model_dir, exist_ok=True)
    tensors = random_tensors(spec, seed, dtype=dtype, std=std, style=style)
    named = {spec.external_names(k)[0]: v for k, v in tensors.items()}
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(dict(config), f, indent=1)
    write_safetensors_file(os.path.join(model_dir, "model.safetensors"), named,
                           metadata={"format": "pt", "seed": str(seed), "init": style})
    return spec
