"""A causal convolution over time on each channel, a few taps long, whose last
inputs are part of a request's state.

    y_t = bias + sum_j w[:, j] * x_(t - taps + 1 + j)        (zeros before the sequence's start)

The weight is ``[channels, taps]``, its last column the current token's. With
``residual`` the part returns x + y (the convolution as a correction of what a
sublayer reads), with ``activation="silu"`` the result passes silu. The
``taps - 1`` inputs that the next step still needs are kept per request in a
state entry of the cache (float32 ``[taps - 1, channels]``), so a position's
output does not depend on where a prompt was cut. Used by a block ahead of its
sublayers and by a recurrent mixer on its own input.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.spec import CacheNeed, PartSpec
from .recurrent import request_rows, request_rows_of
from .registry import CacheView, Runtime, StepContext, WeightStore


class ShortConv:
    kind = "short_conv"
    graph_safe = True
    step_key = "request_rows"
    prepare_step = staticmethod(request_rows)

    def __init__(self, spec: PartSpec, weights: WeightStore, runtime: Runtime):
        self.channels, self.taps = int(spec["channels"]), int(spec["taps"])
        if self.taps < 1:
            raise ValueError(f"a convolution needs at least one tap, got {self.taps}")
        weight = weights.take(spec["weight"])
        if tuple(weight.shape) != (self.channels, self.taps):
            raise ValueError(f"{spec['weight']} is {tuple(weight.shape)}, expected {(self.channels, self.taps)}")
        # tap-major for the kernel: neighbouring channels' weights side by side
        self.weight = weight.to(device=runtime.device, dtype=torch.float32).t().contiguous()
        self.bias: Optional[torch.Tensor] = None
        if spec.get("bias"):
            bias = weights.take(spec["bias"])
            if bias.numel() != self.channels:
                raise ValueError(f"{spec['bias']} has {bias.numel()} values, expected {self.channels}")
            self.bias = bias.to(device=runtime.device, dtype=torch.float32).reshape(-1).contiguous()
        self.residual = bool(spec.get("residual", False))
        self.activation = spec.get("activation")
        if self.activation not in (None, "silu"):
            raise ValueError(f"activation {self.activation!r}; None or 'silu'")

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="state", state_shape=(self.taps - 1, self.channels), state_dtype="float32")

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        """x ``[tokens, channels]`` (rows may be strided) -> ``[tokens, channels]``; moves the state on."""
        if cache.state is None:
            raise ValueError("the convolution needs a state entry of the cache")
        rows = request_rows_of(ctx)
        return ops.short_conv(x, self.weight, self.bias, cache.state, ctx.token_request, rows["row_start"],
                              rows["row_length"], ctx.request_slots, residual=self.residual,
                              activation=self.activation, longest=rows.get("longest", 0))

    def weight_bytes(self) -> int:
        return self.weight.numel() * 4
