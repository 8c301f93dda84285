"""What every part of a layer has to offer.

A part is built from its :class:`~gesso_b200.config.spec.PartSpec` alone (no
device work), declares the tensors it needs, is bound to those tensors once
they are on the device, and then runs on the flat token axis of a step.  No
part knows which model it is in: sizes and constants arrive as parameters.

Interfaces
----------
``Norm``         ``param_decls()``, ``bind(tensors, rt)``,
                 ``add_norm(h, delta, delta_bias, rows=None) -> normed`` — adds
                 ``delta`` (+ bias) into the 32-bit residual ``h`` in place and
                 returns the normed rows in the run dtype.
``Position``     ``bind(rt)``, ``tables(max_positions) -> (cos, sin)`` or
                 whatever its consumer mixer expects.
``Mixer``        ``param_decls()``, ``cache_need()`` (none, one need, or a list of
                 page and state needs), ``bind(tensors, rt)``,
                 ``forward(x, ctx, cache) -> (delta, delta_bias)``.
``FeedForward``  ``param_decls()``, ``bind(tensors, rt)``,
                 ``forward(x, ctx) -> (delta, delta_bias)``.
``Block``        the arrangement: owns the residual order of its parts,
                 ``forward(h, pending, ctx, cache) -> pending``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple


@dataclass(frozen=True)
class ParamDecl:
    """One tensor a part needs.

    role ``matrix``: kept in its stored 16-bit type in bfloat16 runs (a matrix
    stored in 32 bit stays 32 bit and is multiplied in 32 bit); ``vector``:
    small tensors (norm weights, conv taps, biases) always held in float32;
    ``table``: integer tables, held as int32.
    """

    shape: Tuple[int, ...]
    role: str = "matrix"
    alt_shapes: Tuple[Tuple[int, ...], ...] = ()   # accepted spellings with unit axes
    init: str = "normal"                            # random-weights mode: normal | ones | zeros
    fan_in: Optional[int] = None


# ---- what a mixer needs from the cache manager -----------------------------------------
@dataclass(frozen=True)
class PagedNeed:
    """Keys and values of ``n_kv_heads`` heads of ``head_dim`` per token, in pages.

    ``window`` is ``None`` when every earlier key is read, or the number of most
    recent positions (the current one included) that a query reads; pages wholly
    behind the window are given back.
    """

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A per-request state of fixed ``shape``, zero at the start of a request.  ``dtype`` is the name of a
    torch dtype (``float32``, ``bfloat16``, ``int32``, ...)."""

    shape: Tuple[int, ...]
    dtype: str = "float32"


class Part:
    """Base of all parts: declares tensors, is bound once."""

    # False if the part's forward synchronises with the host or launches work whose shape depends
    # on the step's contents; the engine then runs decoding steps eagerly instead of as a CUDA graph.
    graph_safe = True

    def __init__(self, spec):
        self.spec = spec

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {}

    def bind(self, tensors: Dict[str, "torch.Tensor"], rt) -> None:  # noqa: F821
        pass


class Mixer(Part):
    def cache_need(self):
        """What this mixer keeps per request between steps: ``None``, one ``PagedNeed`` or ``StateNeed``
        (``forward`` then gets that one view as ``cache``), or a list of them, pages and states in any
        mix (``forward`` gets a tuple of views in the same order)."""
        return None

    def forward(self, x, ctx, cache):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx):
        raise NotImplementedError


class Norm(Part):
    # True if ``add_norm`` takes ``lazy=True``: with nothing to add it may then return a norm that has not
    # run yet (``ops.LazyNorm``) for a consumer that can apply it in the prologue of its matrix product.
    supports_lazy = False

    def add_norm(self, h, delta, delta_bias, rows=None):
        raise NotImplementedError


class Position(Part):
    pass
