"""Rotary position encoding, half-split pairing.

For pair j of a head (features j and j + rotary_dim/2) at position p: angle = p * theta^(-2j/rotary_dim),
``(y_j, y_{j+half}) = (x_j cos - x_{j+half} sin, x_{j+half} cos + x_j sin)``
(crates/mrun-engine/src/models/common.rs:215-230, 264-280).  The part only produces the table of
(cos, sin) per token and pair, once per step; the attention's fused kernel applies it.
"""
from __future__ import annotations

import math

import torch

from ..config.spec import RotarySpec, ScaledRotarySpec
from ..kernels import ops
from .base import Runtime, register_position


@register_position("rotary")
class Rotary:
    @staticmethod
    def tensor_specs(spec: RotarySpec, prefix: str):
        return []

    def __init__(self, spec: RotarySpec, tensors, runtime: Runtime):
        if spec.rotary_dim % 2 or not 0 < spec.rotary_dim <= spec.head_dim:
            raise ValueError(f"rotary_dim must be even and in (0, head_dim={spec.head_dim}], got {spec.rotary_dim}")
        self.spec = spec
        self.rotary_dim = spec.rotary_dim
        half = spec.rotary_dim // 2
        exponents = torch.arange(half, dtype=torch.float64) * (-2.0 / spec.rotary_dim)
        self.inv_freq = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), exponents).to(runtime.device)

    def rotation(self, ctx) -> torch.Tensor:
        key = ("rotary", self.spec)
        table = ctx.shared.get(key)
        if table is None:
            table = torch.empty((ctx.num_tokens, self.rotary_dim // 2, 2), dtype=torch.float32,
                                device=self.inv_freq.device)
            ops.rotary_table(ctx.positions, self.inv_freq, table)
            ctx.shared[key] = table
        return table


def scaled_frequencies(spec: ScaledRotarySpec):
    """(float64 frequency of every pair, factor on cos and sin) of a :class:`ScaledRotarySpec`."""
    pairs = spec.dims // 2
    freq = torch.pow(torch.tensor(float(spec.base), dtype=torch.float64),
                     torch.arange(pairs, dtype=torch.float64) * (-2.0 / spec.dims))
    if spec.linear_factor is not None:
        freq = freq / float(spec.linear_factor)
    if spec.scaling is None:
        return freq, 1.0
    factor, original, fast, slow = (float(v) for v in spec.scaling)
    turn_pair = lambda turns: spec.dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(spec.base))
    lo = max(math.floor(turn_pair(fast)), 0)
    hi = min(math.ceil(turn_pair(slow)), spec.dims - 1)
    ramp = ((torch.arange(pairs, dtype=torch.float64) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


@register_position("rotary_scaled")
class ScaledRotary:
    """Rotary positions with a choice of pairing and an optional band-wise stretch of the
    frequencies (the formulas are with :class:`ScaledRotarySpec`).  The part makes the step's
    table of (cos, sin) per token and pair; ``pairing`` tells the kernel that applies it which
    two features pair i is."""

    @staticmethod
    def tensor_specs(spec: ScaledRotarySpec, prefix: str):
        return []

    def __init__(self, spec: ScaledRotarySpec, tensors, runtime: Runtime):
        if spec.dims % 2 or spec.dims < 2:
            raise ValueError(f"the number of rotating features must be even and positive, got {spec.dims}")
        if spec.pairing not in ops.PAIRINGS:
            raise ValueError(f"pairing must be one of {sorted(ops.PAIRINGS)}, got {spec.pairing!r}")
        self.spec = spec
        self.rotary_dim = spec.dims
        self.pairing = spec.pairing
        freq, self.magnitude = scaled_frequencies(spec)
        self.inv_freq = freq.to(runtime.device)

    def rotation(self, ctx) -> torch.Tensor:
        key = ("rotary_scaled", self.spec)
        table = ctx.shared.get(key)
        if table is None:
            table = torch.empty((ctx.num_tokens, self.rotary_dim // 2, 2), dtype=torch.float32,
                                device=self.inv_freq.device)
            ops.rotary_table(ctx.positions, self.inv_freq, table, self.magnitude)
            ctx.shared[key] = table
        return table
