"""Binding of checkpoint tensors to the tensors a model declares, by name.

The model's parts declare what they need (internal names, shapes, roles); the
architecture adapter says which checkpoint names an internal name may carry.
Everything that is wrong with a checkpoint is reported in ONE error that lists
missing tensors, unexpected tensors and wrong shapes, each by name (the
reference's binder raises on the first of them, naming the tensor:
src/Inference/materialize_architecture.jl:217-222, 344-349, 369-384).  A tied
output head may be present only if it equals the embedding (:272-276); an
untied model without a head is a missing tensor (:284-289).
"""
from __future__ import annotations

import re
from typing import Dict, Tuple

import torch

from ..config.spec import ModelSpec
from ..errors import invalid
from ..parts.base import ParamDecl
from ..parts.registry import build_block, build_norm


def model_param_decls(spec: ModelSpec) -> Dict[str, ParamDecl]:
    """Every tensor the model needs: internal name -> declaration."""
    decls: Dict[str, ParamDecl] = {
        "embedding.weight": ParamDecl((spec.vocab_size, spec.hidden_size), fan_in=spec.hidden_size),
    }
    for b in spec.blocks:
        blk = build_block(b)
        for name, d in blk.param_decls().items():
            decls[b.prefix + name] = d
    for name, d in build_norm(spec.final_norm).param_decls().items():
        decls["final_norm." + name] = d
    if not spec.tie_embedding:
        decls["lm_head.weight"] = ParamDecl((spec.vocab_size, spec.hidden_size), fan_in=spec.hidden_size)
    return decls


def bind_tensors(spec: ModelSpec, found: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors -> internal names; one error for everything that does not fit."""
    decls = model_param_decls(spec)
    used = set()
    out: Dict[str, torch.Tensor] = {}
    missing, misshaped = [], []
    for internal, decl in decls.items():
        names = spec.external_names(internal)
        hit = next((n for n in names if n in found), None)
        if hit is None:
            missing.append(names[0] if len(names) == 1 else f"{names[0]} (or {', '.join(names[1:])})")
            continue
        used.add(hit)
        t = found[hit]
        shape = tuple(t.shape)
        if shape != tuple(decl.shape) and shape not in decl.alt_shapes:
            misshaped.append(f"{hit}: expected {tuple(decl.shape)}, found {shape}")
            continue
        out[internal] = t.reshape(decl.shape)
    # a tied head may be stored as a copy of the embedding
    tied_head_differs = False
    if spec.tie_embedding:
        for n in spec.external_names("lm_head.weight"):
            if n in found:
                used.add(n)
                emb = out.get("embedding.weight")
                if emb is not None and (tuple(found[n].shape) != tuple(emb.shape) or
                                        not torch.equal(found[n], emb)):
                    tied_head_differs = True
                    misshaped.append(f"{n}: embeddings are tied but this head differs from the embedding")
    ignorable = [re.compile(p) for p in spec.ignorable_tensors]
    unexpected = sorted(n for n in found if n not in used and not any(p.match(n) for p in ignorable))
    if missing or misshaped or unexpected:
        parts = []
        if missing:
            parts.append(f"missing tensors ({len(missing)}): " + "; ".join(sorted(missing)))
        if unexpected:
            parts.append(f"unexpected tensors ({len(unexpected)}): " + "; ".join(unexpected))
        if misshaped:
            parts.append(f"wrong tensors ({len(misshaped)}): " + "; ".join(misshaped))
        raise invalid(f"checkpoint does not fit {spec.architecture}: " + " | ".join(parts))
    del tied_head_differs
    return out


def place_tensor(t: torch.Tensor, decl: ParamDecl, run_dtype: torch.dtype, device) -> torch.Tensor:
    """Device copy in the type the engine keeps it in.

    vector -> float32; table -> int32; matrix -> float32 in a float32 run, else
    bfloat16 unless the checkpoint stores it in 32 bit, which stays 32 bit.
    """
    if decl.role == "table":
        return t.to(device=device, dtype=torch.int32).contiguous()
    if decl.role == "vector":
        return t.to(device=device, dtype=torch.float32).contiguous()
    if run_dtype == torch.float32 or t.dtype == torch.float32:
        return t.to(device=device, dtype=torch.float32).contiguous()
    return t.to(device=device, dtype=torch.bfloat16).contiguous()


def load_model_tensors(model_dir: str, spec: ModelSpec) -> Tuple[Dict[str, torch.Tensor], Dict[str, ParamDecl]]:
    from .safetensors_io import read_model_tensors
    found = read_model_tensors(model_dir)
    return bind_tensors(spec, found), model_param_decls(spec)
