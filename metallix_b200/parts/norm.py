"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, the weight multiplying
directly (crates/models/qwen/src/forward.rs:2442-2449). Sum of squares and
scale are float32 in both precisions. A checkpoint may store the weight around
zero (``one_plus``): the factor is then 1 + w, formed once in float32 when the
part is built. It may also store one number for all coordinates (``scalar``)
or none at all (the row over its root mean square).

Dynamic Tanh: y = tanh(alpha * x) * w + b with a scalar alpha, computed value
by value in float32; it takes no mean or variance of the row, so it has no
epsilon."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.spec import PartSpec
from .registry import Pending, Runtime, WeightStore, register_part


class RMSNorm:
    kind = "rmsnorm"
    adds_summands = True   # add_forward also takes [parts, rows, size]: a sum its producer left in parts

    def __init__(self, weight: torch.Tensor, eps: float, runtime: Runtime, one_plus: bool = False):
        weight = weight.to(device=runtime.device, dtype=torch.float32)
        self.weight = (weight + 1.0 if one_plus else weight).contiguous()
        self.size = self.weight.numel()
        self.eps = float(eps)

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype,
                rows_index: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype, rows_index=rows_index)

    def add_forward(self, residual: torch.Tensor, delta, out_dtype: torch.dtype) -> torch.Tensor:
        """residual += delta (float32, in place), then the norm of the sum.
        ``delta`` may be float32 ``[parts, rows, size]``: its parts are added up
        first. A ``Pending`` delta passes its own norm before the sum, in the
        same pass over the row when that norm is an RMSNorm too."""
        if delta is not None and hasattr(delta, "settle"):   # a block arrangement's own way of joining the stream
            delta.settle(residual)
            delta = None
        if delta is None:
            return ops.rmsnorm(residual, self.weight, self.eps, out_dtype)
        if isinstance(delta, Pending):
            if isinstance(delta.norm, RMSNorm):
                return ops.postnorm_add_rmsnorm(residual, delta.delta, delta.norm.weight, delta.norm.eps,
                                                self.weight, self.eps, out_dtype)
            delta.norm.add_normed(residual, delta.delta)
            return ops.rmsnorm(residual, self.weight, self.eps, out_dtype)
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, out_dtype)

    def add_normed(self, residual: torch.Tensor, delta: torch.Tensor) -> None:
        """residual += norm(delta) (float32, in place): this norm as the one a
        sublayer's output passes on its way into the residual stream."""
        ops.postnorm_add_rmsnorm(residual, delta, self.weight, self.eps)


def _build(spec: PartSpec, weights: WeightStore, runtime: Runtime) -> RMSNorm:
    """``weight`` None: the row over its root mean square and nothing else;
    ``scalar``: the stored weight is one number for all coordinates."""
    if spec.get("weight") is None:
        return RMSNorm(torch.ones(spec["size"]), spec["eps"], runtime)
    weight = weights.take(spec["weight"])
    if spec.get("scalar"):
        if weight.numel() != 1:
            raise ValueError(f"{spec['weight']} has {weight.numel()} values, a scalar norm weight has one")
        weight = weight.to(torch.float32).reshape(1).expand(spec["size"])
    if weight.numel() != spec["size"]:
        raise ValueError(f"{spec['weight']} has {weight.numel()} values, the norm is over {spec['size']}")
    return RMSNorm(weight, spec["eps"], runtime, one_plus=bool(spec.get("one_plus", False)))


register_part("norm", "rmsnorm", _build)


class DynamicTanh:
    kind = "dynamic_tanh"
    adds_summands = False
    elementwise = True   # nothing is reduced over a row: a kernel that makes the row may apply it as it goes

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], alpha: torch.Tensor, runtime: Runtime):
        as_float = lambda t: t.to(device=runtime.device, dtype=torch.float32).contiguous()
        self.weight = as_float(weight).reshape(-1)
        self.bias = as_float(bias).reshape(-1) if bias is not None else None
        self.alpha = as_float(alpha).reshape(1)
        self.size = self.weight.numel()
        if self.bias is not None and self.bias.numel() != self.size:
            raise ValueError(f"the norm's bias has {self.bias.numel()} values, its weight {self.size}")
        self._one = torch.ones(1, dtype=torch.float32, device=runtime.device)

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype,
                rows_index: Optional[torch.Tensor] = None) -> torch.Tensor:
        rows = x.reshape(-1, self.size)
        if rows.dtype != torch.float32:
            rows = rows.float()
        out = ops.stream_mix(rows.view(rows.shape[0], 1, self.size), alpha=self.alpha, norm_weight=self.weight,
                             norm_bias=self.bias, out_dtype=out_dtype, rows_index=rows_index)
        return out if rows_index is not None else out.view(x.shape)

    def add_forward(self, residual: torch.Tensor, delta, out_dtype: torch.dtype) -> torch.Tensor:
        """residual += delta (float32, in place), then the norm of the sum, in one pass."""
        if delta is not None and not isinstance(delta, torch.Tensor):
            from .registry import settle
            settle(residual, delta)      # whatever else a block left pending joins first
            delta = None
        if delta is not None and delta.dim() == 3:
            delta = delta.sum(0)
        return ops.stream_mix(residual.view(residual.shape[0], 1, self.size), result=delta, mix=self._one,
                              out_weights=self._one, alpha=self.alpha, norm_weight=self.weight, norm_bias=self.bias,
                              out_dtype=out_dtype)

    def add_normed(self, residual: torch.Tensor, delta: torch.Tensor) -> None:
        if delta.dim() == 3:
            delta = delta.sum(0)
        ops.add_(residual, self.forward(delta, torch.float32))


def _build_dynamic_tanh(spec: PartSpec, weights: WeightStore, runtime: Runtime) -> DynamicTanh:
    weight = weights.take(spec["weight"])
    if weight.numel() != spec["size"]:
        raise ValueError(f"{spec['weight']} has {weight.numel()} values, the norm is over {spec['size']}")
    bias = weights.take(spec["bias"]) if spec.get("bias") else None
    return DynamicTanh(weight, bias, weights.take(spec["alpha"]), runtime)


register_part("norm", "dynamic_tanh", _build_dynamic_tanh)
