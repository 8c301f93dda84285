"""Registries from a part's ``kind`` to the class that implements it.

A new mixer, feed-forward, norm, position encoding or block arrangement is one
class plus one ``register_*`` call; the engine, the cache manager and the
weight loader find it through these tables and need no change.
"""
from __future__ import annotations

from typing import Callable, Dict

from ..config.spec import PartSpec
from ..errors import invalid

_TABLES: Dict[str, Dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {},
}


def _register(table: str, kind: str, cls: Callable, replace: bool) -> None:
    if kind in _TABLES[table] and not replace:
        raise invalid(f"{table} kind {kind!r} is already registered")
    _TABLES[table][kind] = cls


def _build(table: str, spec: PartSpec, *args):
    cls = _TABLES[table].get(spec.kind)
    if cls is None:
        raise invalid(f"unknown {table} kind {spec.kind!r}; registered: {sorted(_TABLES[table])}")
    return cls(spec, *args)


def register_mixer(kind: str, cls: Callable, *, replace: bool = False) -> None:
    _register("mixer", kind, cls, replace)


def register_feed_forward(kind: str, cls: Callable, *, replace: bool = False) -> None:
    _register("feed_forward", kind, cls, replace)


def register_norm(kind: str, cls: Callable, *, replace: bool = False) -> None:
    _register("norm", kind, cls, replace)


def register_position(kind: str, cls: Callable, *, replace: bool = False) -> None:
    _register("position", kind, cls, replace)


def register_block(arrangement: str, cls: Callable, *, replace: bool = False) -> None:
    _register("block", arrangement, cls, replace)


def unregister(table: str, kind: str) -> None:
    _TABLES[table].pop(kind, None)


def build_mixer(spec: PartSpec):
    return _build("mixer", spec)


def build_feed_forward(spec: PartSpec):
    return _build("feed_forward", spec)


def build_norm(spec: PartSpec):
    return _build("norm", spec)


def build_position(spec: PartSpec):
    return _build("position", spec)


def build_block(block_spec):
    cls = _TABLES["block"].get(block_spec.arrangement)
    if cls is None:
        raise invalid(f"unknown block arrangement {block_spec.arrangement!r}; "
                      f"registered: {sorted(_TABLES['block'])}")
    return cls(block_spec)


def registered(table: str) -> list[str]:
    return sorted(_TABLES[table])
