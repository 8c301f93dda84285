"""One registry from an architecture's name to the adapter that reads its config.

``config.json`` names its model class in ``architectures[0]`` (``model_type``
is the fallback key).  An adapter turns the parsed JSON object into a
:class:`~gesso_b200.config.spec.ModelSpec`.  An unknown name is refused with
the list of known names, as the reference's adapter table does
(src/Inference/arch_adapters.jl:1075-1109).
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Mapping

from ..errors import invalid
from .spec import ModelSpec

Adapter = Callable[[Mapping[str, Any]], ModelSpec]

_ARCHITECTURES: Dict[str, Adapter] = {}


def register_architecture(name: str, adapter: Adapter, *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise invalid(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = adapter


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def _reject_duplicate_keys(pairs):
    seen = {}
    for k, v in pairs:
        if k in seen:
            raise invalid(f"config.json: key {k!r} appears twice")
        seen[k] = v
    return seen


def parse_strict_json(text: str, what: str = "config.json") -> dict:
    """JSON object with duplicate keys refused (src/Inference/llama_import.jl:43-63)."""
    try:
        obj = json.loads(text, object_pairs_hook=_reject_duplicate_keys)
    except json.JSONDecodeError as e:
        raise invalid(f"{what}: not valid JSON ({e})") from None
    if not isinstance(obj, dict):
        raise invalid(f"{what}: top level must be an object")
    return obj


def architecture_name(config: Mapping[str, Any]) -> str:
    archs = config.get("architectures")
    if isinstance(archs, (list, tuple)) and len(archs) >= 1 and isinstance(archs[0], str):
        return archs[0]
    mt = config.get("model_type")
    if isinstance(mt, str):
        for name in _ARCHITECTURES:
            if getattr(_ARCHITECTURES[name], "model_type", None) == mt:
                return name
        raise invalid(
            f"config.json: model_type {mt!r} is not registered; known architectures: "
            f"{known_architectures()}"
        )
    raise invalid("config.json: neither 'architectures' nor 'model_type' names a model class")


def spec_from_config(config: Mapping[str, Any]) -> ModelSpec:
    name = architecture_name(config)
    adapter = _ARCHITECTURES.get(name)
    if adapter is None:
        raise invalid(
            f"architecture {name!r} is not registered; known architectures: {known_architectures()}"
        )
    return adapter(config)


def read_config(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise invalid(f"{model_dir}: no config.json")
    with open(path, "r", encoding="utf-8") as f:
        return parse_strict_json(f.read(), path)


def spec_from_dir(model_dir: str) -> ModelSpec:
    return spec_from_config(read_config(model_dir))
