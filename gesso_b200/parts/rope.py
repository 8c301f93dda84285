"""Rotary position encoding.

Pair ``(i, i + d/2)`` of a head is rotated by ``theta_i = pos * base^(-2i/d)``
(src/Operators/cpu.jl:357-371; ``interleaved=false`` is the LFM layout,
src/Inference/architecture_spec.jl:66).  The reference computes angle, cos and
sin in Float64 (cpu.jl:359-369); here the host fills a float32 table
``[max_positions, d/2]`` from float64 angles once per (base, d) and the kernels
read it, so no precision is lost at large positions.

Parameters: ``theta``; ``rotary_dim`` (even, at most the head size: the leading
``rotary_dim`` features of a head are rotated with ``d = rotary_dim``, the rest are
left alone; LFM2 rotates the whole head, and its configuration reader refuses
anything else as the reference does, src/Inference/lfm2.jl:66-70); ``interleaved``
(pairs ``(2i, 2i+1)`` instead of the halves; default false).  A position part hands
the attention part ``tables()`` = (cos, sin) and ``layout()`` = (rotary size,
interleaved).
"""
from __future__ import annotations

import torch

from ..errors import invalid
from .base import Position
from .registry import register_position


def rope_tables(theta: float, dim: int, max_positions: int):
    """(cos, sin) float32 CPU tensors ``[max_positions, dim/2]`` from float64 angles."""
    i = torch.arange(dim // 2, dtype=torch.float64)
    inv_freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / dim)
    ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
    return torch.cos(ang).to(torch.float32), torch.sin(ang).to(torch.float32)


class RotaryPosition(Position):
    def __init__(self, spec):
        super().__init__(spec)
        self.theta = float(spec["theta"])
        self.rotary_dim = int(spec["rotary_dim"])
        self.interleaved = bool(spec.get("interleaved", False))
        if self.rotary_dim % 2 != 0 or self.rotary_dim < 2:
            raise invalid("rope: rotary_dim must be even and at least 2")
        self.cos = self.sin = None

    def check_head_dim(self, head_dim: int) -> None:
        if self.rotary_dim > head_dim:
            raise invalid(f"rope: rotary_dim {self.rotary_dim} exceeds the head size {head_dim}")

    def layout(self):
        """(how many leading features of a head are rotated, whether neighbours are paired)."""
        return self.rotary_dim, self.interleaved

    def bind(self, tensors, rt) -> None:
        key = ("rope", self.theta, self.rotary_dim)
        if key not in rt.shared:
            cos, sin = rope_tables(self.theta, self.rotary_dim, rt.max_positions)
            rt.shared[key] = (cos.to(rt.device).contiguous(), sin.to(rt.device).contiguous())
        self.cos, self.sin = rt.shared[key]

    def tables(self):
        return self.cos, self.sin


class NoPosition(Position):
    """No position encoding: the mixer's queries and keys are used as projected."""

    def check_head_dim(self, head_dim: int) -> None:
        pass

    def tables(self):
        return None, None

    def layout(self):
        return 0, False


register_position("rope", RotaryPosition, replace=True)
register_position("none", NoPosition, replace=True)
