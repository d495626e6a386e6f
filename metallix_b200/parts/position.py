"""Rotary position encodings over the first ``rotary_dim`` values of a head.

``rope_half`` pairs value i with value i + rotary_dim / 2
(crates/models/qwen/src/forward.rs:2031-2054: dims = head_dim, traditional =
false, base = rope_theta, scale 1); ``rope_interleaved`` pairs value 2i with
value 2i + 1. Either way pair i at position p turns by the angle p f_i,
f_i = theta^(-2i / rotary_dim): (a, b) -> (a cos - b sin, b cos + a sin); the
values beyond ``rotary_dim`` pass unchanged.

``scaling`` (optional) stretches the long wavelengths for contexts beyond
those a model was trained on. Let n_i = original * f_i / (2 pi) be the number
of full turns pair i makes over ``original`` positions. A pair that turns more
than ``high`` times keeps its frequency; one that turns fewer than ``low``
times gets f_i / factor; in between the two are mixed, f_i (s + (1 - s) /
factor) with s = (n_i - low) / (high - low) rising from 0 to 1.

A second form of ``scaling`` (keys factor, original, fast, slow: the one known
as YaRN) places the ramp on the pair index instead. With
where(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta), the index of the
pair that makes t turns over ``original`` positions, lo = max(floor(where(fast)),
0), hi = min(ceil(where(slow)), rotary_dim - 1) and ramp_i = clamp((i - lo) /
max(hi - lo, 0.001), 0, 1), pair i gets f_i / factor * ramp_i + f_i (1 - ramp_i),
and cos and sin are both multiplied by 0.1 ln(factor) + 1 (``rotary_magnitude``).

Angles are formed in float64 (position times frequency), cos and sin are
rounded once to float32 tables that the kernels index by position.
"""
from __future__ import annotations

import math
from typing import Mapping, Optional

import torch

from .. import ops
from ..config.spec import PartSpec
from .registry import Runtime, WeightStore, register_part


def rotary_frequencies(theta: float, rotary_dim: int, scaling: Optional[Mapping] = None) -> torch.Tensor:
    """float64 ``[rotary_dim / 2]``: f_i = theta^(-2i / rotary_dim), stretched by
    ``scaling`` (factor, low, high, original) as described above."""
    index = torch.arange(rotary_dim // 2, dtype=torch.float64)
    frequency = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * index / rotary_dim)
    if scaling and "fast" in scaling:
        factor, original = float(scaling["factor"]), float(scaling["original"])
        fast, slow = float(scaling["fast"]), float(scaling["slow"])
        if not (factor > 0.0 and original > 0.0 and fast > 0.0 and slow > 0.0 and float(theta) > 1.0):
            raise ValueError(f"rotary scaling needs positive factor, original, fast and slow, got {dict(scaling)}")
        where = lambda turns: rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(theta)))
        lo = max(math.floor(where(fast)), 0)
        hi = min(math.ceil(where(slow)), rotary_dim - 1)
        ramp = torch.clamp((index - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        frequency = frequency / factor * ramp + frequency * (1.0 - ramp)
    elif scaling:
        factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
        original = float(scaling["original"])
        if not (factor > 0.0 and high > low and original > 0.0):
            raise ValueError(f"rotary scaling needs factor > 0, high > low and original > 0, got {dict(scaling)}")
        turns = original * frequency / (2.0 * math.pi)
        share = (turns - low) / (high - low)
        mixed = frequency * (share + (1.0 - share) / factor)
        frequency = torch.where(turns > high, frequency, torch.where(turns < low, frequency / factor, mixed))
    return frequency


def rotary_magnitude(scaling: Optional[Mapping] = None) -> float:
    """What cos and sin are multiplied by: 0.1 ln(factor) + 1 for the form of
    ``scaling`` with fast and slow, else 1."""
    if scaling and "fast" in scaling:
        return 0.1 * math.log(float(scaling["factor"])) + 1.0
    return 1.0


def _scaling_key(scaling: Optional[Mapping]) -> tuple:
    return tuple(sorted((str(k), float(v)) for k, v in scaling.items())) if scaling else ()


class Rotary:
    """Both pairings; ``interleaved`` says which."""

    fused_tables = True  # the attention mixer may hand cos/sin to its fused kernel
    interleaved = False

    def __init__(self, theta: float, rotary_dim: int, head_dim: int, runtime: Runtime,
                 scaling: Optional[Mapping] = None):
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and within head_dim {head_dim}")
        self.theta, self.rotary_dim, self.head_dim = float(theta), rotary_dim, head_dim
        self.scaling = dict(scaling) if scaling else None
        # Layers with the same parameters share one pair of tables (the pairing
        # does not enter: pair i has the same angle in both).
        key = ("rope", self.theta, rotary_dim, _scaling_key(self.scaling), runtime.max_positions, str(runtime.device))
        if key not in runtime.shared:
            frequency = rotary_frequencies(self.theta, rotary_dim, self.scaling).to(runtime.device)
            position = torch.arange(runtime.max_positions, dtype=torch.float64, device=runtime.device)
            angle = position[:, None] * frequency[None, :]
            magnitude = rotary_magnitude(self.scaling)
            runtime.shared[key] = ((torch.cos(angle) * magnitude).to(torch.float32).contiguous(),
                                   (torch.sin(angle) * magnitude).to(torch.float32).contiguous())
        self.cos, self.sin = runtime.shared[key]
        self._shared, self._key = runtime.shared, key

    def inverse_sin(self) -> torch.Tensor:
        """The sine table of the turn back (by minus the position), made at first use and shared like the others."""
        key = self._key + ("inverse",)
        if key not in self._shared:
            self._shared[key] = (-self.sin).contiguous()
        return self._shared[key]

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor):
        """Rotates q [tokens, heads * head_dim] and k [tokens, kv_heads * head_dim];
        returns (q_rotated [tokens, heads, head_dim], k_rotated [tokens, kv_heads, head_dim])."""
        q_out = ops.norm_rotate_heads(q, self.head_dim, positions, cos=self.cos, sin=self.sin,
                                      interleaved=self.interleaved)
        k_out = ops.norm_rotate_heads(k, self.head_dim, positions, cos=self.cos, sin=self.sin,
                                      interleaved=self.interleaved)
        return q_out, k_out


class RotaryHalf(Rotary):
    kind = "rope_half"


class RotaryInterleaved(Rotary):
    kind = "rope_interleaved"
    interleaved = True


def _builder(cls):
    def build(spec: PartSpec, weights: WeightStore, runtime: Runtime):
        return cls(spec["theta"], spec["rotary_dim"], spec["head_dim"], runtime, scaling=spec.get("scaling"))
    return build


register_part("position", "rope_half", _builder(RotaryHalf))
register_part("position", "rope_interleaved", _builder(RotaryInterleaved))
