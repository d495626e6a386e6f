"""A layer's own input from the token, gated by the residual stream.

With a table row per token, of which the layer owns ``dim`` values from
``offset`` on:

    e = table[token, offset : offset + dim]
    g = gelu_tanh(x Wg^T) * e            x: the residual stream, in the compute type
    y = g Wp^T
    x <- x + norm(y)

``forward`` adds what is still pending to the stream, makes y (float32) and
hands it on with its norm as a ``Pending``, so that the norm of y, the sum and
the next layer's first norm run as one kernel. Layers share one copy of the
table on the device.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .linear import Linear
from .registry import Pending, Runtime, StepContext, WeightStore, build_part


class TokenInput:
    kind = "token_input"

    def __init__(self, spec: PartSpec, weights: WeightStore, runtime: Runtime):
        hidden, self.dim, self.offset = spec["hidden_size"], int(spec["dim"]), int(spec["offset"])
        key = ("token_table", spec["table"], str(runtime.device), str(runtime.dtype))
        if key not in runtime.shared:   # the first layer to be built takes the table for all
            runtime.shared[key] = weights.take(spec["table"]).to(device=runtime.device, dtype=runtime.dtype).contiguous()
        self.table = runtime.shared[key]
        if self.table.dim() != 2 or self.offset + self.dim > self.table.shape[1]:
            raise ValueError(f"{spec['table']} is {tuple(self.table.shape)}; columns {self.offset} .. "
                             f"{self.offset + self.dim} are asked for")
        self.gate = Linear(weights.take(spec["gate_proj"]), runtime)
        self.out = Linear(weights.take(spec["out_proj"]), runtime)
        if (self.gate.out_features, self.gate.in_features) != (self.dim, hidden) \
                or (self.out.out_features, self.out.in_features) != (hidden, self.dim):
            raise ValueError(f"{spec['gate_proj']} is {tuple(self.gate.weight.shape)}, {spec['out_proj']} is "
                             f"{tuple(self.out.weight.shape)}; expected {(self.dim, hidden)} and {(hidden, self.dim)}")
        self.norm = build_part("norm", spec["norm"], weights, runtime)
        self.dtype = runtime.dtype

    def parts(self):
        return [self.norm]

    def forward(self, residual: torch.Tensor, pending, ctx: StepContext) -> Pending:
        """``residual`` (float32, in place) takes ``pending`` (a tensor or None); returns what this input adds, not
        yet normed or added."""
        if ctx.token_ids is None:
            raise ValueError("the step's token ids were not handed to the parts")
        x = ops.add_cast(residual, pending, self.dtype)
        gated = ops.gelu_gate_rows(self.gate.forward(x), self.table, ctx.token_ids, self.offset)
        return Pending(self.out.forward(gated, out_dtype=torch.float32), self.norm)

    def weight_bytes(self) -> int:
        return self.gate.weight_bytes() + self.out.weight_bytes()
