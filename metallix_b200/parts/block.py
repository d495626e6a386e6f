"""Arrangement of one layer's parts.

``prenorm_residual`` is the reference's layer
(crates/models/qwen/src/forward.rs:1856-1885, :1889-1922):
r = x + mixer(norm1(x)); x' = r + feed_forward(norm2(r)). The residual stream
is float32; a block receives the previous block's output not yet added
(``pending``) so that every residual sum runs inside the norm kernel that
follows it.

``sandwich_residual`` puts a second norm behind each sublayer:
r = x + post1(mixer(norm1(x))); x' = r + post2(feed_forward(norm2(r))), the
feed-forward half being optional. What a sublayer leaves is handed on with
the norm it still has to pass (``Pending``), so that this norm, the residual
sum and the next sublayer's norm run as one kernel.

``hyper_connections`` keeps s copies x_1 .. x_s of the residual stream
(``[tokens, s, hidden]``, float32). Sublayer q reads u = sum_s in_q[s] x_s,
runs on norm(u), and its result y, times a per-channel layer scale, goes back
to all streams at once: x_t <- sum_s mix_q[s, t] x_s + out_q[t] y. What a
sublayer leaves is handed on as a ``StreamWrite``; the write, the next read
and (when it is elementwise) the next norm are one kernel.

``conv_prenorm_residual`` is the pre-norm layer with two additions, each
optional: what a sublayer reads passes a short causal convolution over time
first (h <- h + conv(h), whose last inputs are part of a request's state),
and after the feed-forward the layer takes an input from the token itself,
x <- x + norm(input(x, token)).

``parallel_residual`` lets both sublayers read the same input:
x' = x + m (mixer(norm1(x)) + feed_forward(norm2(x))) with a constant m, the
feed-forward being optional. What the layer leaves is a ``PairSum`` (the two
results and m); the next layer's first kernel adds it to the stream and makes
both of that layer's norms from one pass over the row (two RMS norms of the
same row share its mean square).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config.spec import LayerSpec
from dataclasses import dataclass

from .. import ops
from .registry import CacheView, Pending, Runtime, StepContext, WeightStore, build_part, register_part, settle


class PreNormResidualBlock:
    kind = "prenorm_residual"

    def __init__(self, layer: LayerSpec, weights: WeightStore, runtime: Runtime):
        self.name = layer.name
        self.mixer_norm = build_part("norm", layer.mixer_norm, weights, runtime)
        self.mixer = build_part("mixer", layer.mixer, weights, runtime)
        self.feed_forward_norm = build_part("norm", layer.feed_forward_norm, weights, runtime)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, weights, runtime)
        self.dtype = runtime.dtype
        # A mixer may leave its output as summands [parts, tokens, hidden] when
        # the norm that takes it next adds them up in its own pass over the row.
        summands = getattr(self.mixer, "forward_summands", None)
        self.mix = summands if summands is not None and getattr(self.feed_forward_norm, "adds_summands", False) \
            else self.mixer.forward

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, residual: torch.Tensor, pending, ctx: StepContext,
                cache: CacheView) -> torch.Tensor:
        """``residual`` (float32, updated in place) plus ``pending`` (a tensor,
        or a ``Pending`` that carries the norm it passes first) is the layer's
        input; returns the feed-forward output, to be added by whoever runs
        next."""
        mixer_in = self.mixer_norm.add_forward(residual, pending, self.dtype)
        mixed = self.mix(mixer_in, ctx, cache)
        feed_in = self.feed_forward_norm.add_forward(residual, mixed, self.dtype)
        return self.feed_forward.forward(feed_in, ctx)


class SandwichNormBlock:
    kind = "sandwich_residual"

    def __init__(self, layer: LayerSpec, weights: WeightStore, runtime: Runtime):
        self.name = layer.name
        if layer.mixer_post_norm is None:
            raise ValueError(f"{layer.name}: a sandwich block needs the norm behind its mixer")
        self.mixer_norm = build_part("norm", layer.mixer_norm, weights, runtime)
        self.mixer = build_part("mixer", layer.mixer, weights, runtime)
        self.mixer_post_norm = build_part("norm", layer.mixer_post_norm, weights, runtime)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, weights, runtime)
        self.feed_forward_norm = self.feed_forward_post_norm = None
        if self.feed_forward is not None:
            if layer.feed_forward_norm is None or layer.feed_forward_post_norm is None:
                raise ValueError(f"{layer.name}: a feed-forward in a sandwich block needs both of its norms")
            self.feed_forward_norm = build_part("norm", layer.feed_forward_norm, weights, runtime)
            self.feed_forward_post_norm = build_part("norm", layer.feed_forward_post_norm, weights, runtime)
        self.dtype = runtime.dtype
        # Summands [parts, tokens, hidden] are taken where the kernel that adds
        # the mixer's output up is known to be this block's own.
        summands = getattr(self.mixer, "forward_summands", None)
        fused = (self.feed_forward is not None and getattr(self.feed_forward_norm, "adds_summands", False)
                 and getattr(self.mixer_post_norm, "adds_summands", False))
        self.mix = summands if summands is not None and fused else self.mixer.forward

    def parts(self):
        return [self.mixer_norm, self.mixer, self.mixer_post_norm, self.feed_forward_norm, self.feed_forward,
                self.feed_forward_post_norm]

    def forward(self, residual: torch.Tensor, pending, ctx: StepContext, cache: CacheView):
        mixer_in = self.mixer_norm.add_forward(residual, pending, self.dtype)
        mixed = Pending(self.mix(mixer_in, ctx, cache), self.mixer_post_norm)
        if self.feed_forward is None:
            return mixed
        feed_in = self.feed_forward_norm.add_forward(residual, mixed, self.dtype)
        return Pending(self.feed_forward.forward(feed_in, ctx), self.feed_forward_post_norm)


register_part("block", "sandwich_residual",
              lambda layer, weights, runtime: SandwichNormBlock(layer, weights, runtime))
register_part("block", "prenorm_residual",
              lambda layer, weights, runtime: PreNormResidualBlock(layer, weights, runtime))


@dataclass
class StreamWrite:
    """A sublayer's result on its way into several residual streams."""

    result: torch.Tensor                    # [tokens, hidden]
    channel_scale: Optional[torch.Tensor]   # [hidden] or None
    mix: torch.Tensor                       # [s, s], indexed [from, to]
    out_weights: torch.Tensor               # [s]
    second: Optional[torch.Tensor] = None   # a second result: weights[0] * result + weights[1] * second is what joins
    weights: tuple = (1.0, 1.0)

    def fields(self) -> dict:
        return dict(result=self.result, channel_scale=self.channel_scale, mix=self.mix, out_weights=self.out_weights,
                    second=self.second, weights=self.weights)

    def settle(self, streams: torch.Tensor) -> None:
        ops.stream_mix(streams, read=False, **self.fields())


def read_streams(streams: torch.Tensor, pending, in_weights: Optional[torch.Tensor], norm, out_dtype: torch.dtype,
                 rows_index: Optional[torch.Tensor] = None, keep_streams: bool = True) -> torch.Tensor:
    """norm(sum_s in_weights[s] x_s) (the plain sum without ``in_weights``)
    after ``pending`` has joined the streams, in one kernel where the norm is
    elementwise and the pending result a ``StreamWrite``."""
    if pending is not None and not isinstance(pending, StreamWrite):
        settle(streams, pending)
        pending = None
    write = pending.fields() if pending is not None else {}
    if getattr(norm, "elementwise", False) and getattr(norm, "kind", None) == "dynamic_tanh":
        return ops.stream_mix(streams, in_weights=in_weights, alpha=norm.alpha, norm_weight=norm.weight,
                              norm_bias=norm.bias, out_dtype=out_dtype, rows_index=rows_index,
                              keep_streams=keep_streams, **write)
    mixed = ops.stream_mix(streams, in_weights=in_weights, out_dtype=torch.float32, rows_index=rows_index,
                           keep_streams=keep_streams, **write)
    return norm.forward(mixed, out_dtype) if norm is not None else mixed.to(out_dtype)


def open_streams(embedded: torch.Tensor, count: int) -> torch.Tensor:
    """``count`` copies of the embedding output side by side: [tokens, count, hidden]."""
    return embedded.unsqueeze(1).expand(-1, count, -1).contiguous()


def sum_of_streams(streams: torch.Tensor) -> torch.Tensor:
    """[tokens, hidden]: what the streams add up to (float32)."""
    return ops.stream_mix(streams, out_dtype=torch.float32)


class HyperConnectionBlock:
    kind = "hyper_connections"

    def __init__(self, layer: LayerSpec, weights: WeightStore, runtime: Runtime):
        self.name = layer.name
        params = layer.block
        self.streams = int(params["streams"])
        if not 1 <= self.streams <= ops.MAX_STREAMS:
            raise ValueError(f"{layer.name}: {self.streams} residual streams; 1..{ops.MAX_STREAMS} are taken")
        self.mixer_norm = build_part("norm", layer.mixer_norm, weights, runtime)
        self.mixer = build_part("mixer", layer.mixer, weights, runtime)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, weights, runtime)
        self.feed_forward_norm = None
        if self.feed_forward is not None:
            if layer.feed_forward_norm is None:
                raise ValueError(f"{layer.name}: a feed-forward needs its norm")
            self.feed_forward_norm = build_part("norm", layer.feed_forward_norm, weights, runtime)
        self.dtype = runtime.dtype
        # A mixer made of two may hand both results over with their weights: the sum is then made by the kernel
        # that writes the streams, not by one of its own.
        self.mix_pair = getattr(self.mixer, "forward_pair", None)
        s = self.streams

        def small(name, shape):
            tensor = weights.take(name)
            if tuple(tensor.shape) != shape:
                raise ValueError(f"{name} is {tuple(tensor.shape)}, expected {shape}")
            return tensor.to(device=runtime.device, dtype=torch.float32).contiguous()

        def sublayer(prefix):
            names = params[prefix]
            scale = names.get("scale")
            return {"in": small(names["in"], (s,)), "out": small(names["out"], (s,)),
                    "mix": small(names["mix"], (s, s)),
                    "scale": small(scale, (params["hidden_size"],)) if scale else None}

        self.mixer_streams = sublayer("mixer")
        self.feed_forward_streams = sublayer("feed_forward") if self.feed_forward is not None else None

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, streams: torch.Tensor, pending, ctx: StepContext, cache: CacheView):
        """``streams`` (float32 [tokens, s, hidden], updated in place) with
        ``pending`` still to join; returns the last sublayer's ``StreamWrite``."""
        own = self.mixer_streams
        mixer_in = read_streams(streams, pending, own["in"], self.mixer_norm, self.dtype)
        if self.mix_pair is not None:
            first, second, weights = self.mix_pair(mixer_in, ctx, cache)
            left = StreamWrite(first, own["scale"], own["mix"], own["out"], second=second, weights=weights)
        else:
            left = StreamWrite(self.mixer.forward(mixer_in, ctx, cache), own["scale"], own["mix"], own["out"])
        if self.feed_forward is None:
            return left
        own = self.feed_forward_streams
        feed_in = read_streams(streams, left, own["in"], self.feed_forward_norm, self.dtype)
        return StreamWrite(self.feed_forward.forward(feed_in, ctx), own["scale"], own["mix"], own["out"])


register_part("block", "hyper_connections",
              lambda layer, weights, runtime: HyperConnectionBlock(layer, weights, runtime))


class ConvPreNormBlock:
    """x <- x + mixer(c1(norm1(x))); x <- x + ff(c2(norm2(x))); x <- x + norm(token_input(x, token)), with
    c(h) = h + conv(h). The convolutions' states join the mixer's own need as members of one cache entry:
    [mixer, mixer's convolution, feed-forward's convolution] as far as they exist."""

    kind = "conv_prenorm_residual"

    def __init__(self, layer: LayerSpec, weights: WeightStore, runtime: Runtime):
        from .short_conv import ShortConv
        from .token_input import TokenInput
        params = layer.block
        self.name = layer.name
        self.mixer_norm = build_part("norm", layer.mixer_norm, weights, runtime)
        self.mixer = build_part("mixer", layer.mixer, weights, runtime)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, weights, runtime)
        self.feed_forward_norm = None
        if self.feed_forward is not None:
            if layer.feed_forward_norm is None:
                raise ValueError(f"{layer.name}: a feed-forward needs its norm")
            self.feed_forward_norm = build_part("norm", layer.feed_forward_norm, weights, runtime)
        conv = lambda key: ShortConv(params[key], weights, runtime) if params.get(key) is not None else None
        self.mixer_conv = conv("mixer_conv")
        self.feed_forward_conv = conv("feed_forward_conv") if self.feed_forward is not None else None
        self.token_input = TokenInput(params["token_input"], weights, runtime) \
            if params.get("token_input") is not None else None
        self.dtype = runtime.dtype
        self._members = [self.mixer] + [c for c in (self.mixer_conv, self.feed_forward_conv) if c is not None]

    def parts(self):
        return [self.mixer_norm, self.mixer_conv, self.mixer, self.feed_forward_norm, self.feed_forward_conv,
                self.feed_forward, self.token_input]

    def cache_need(self):
        from ..config.spec import CacheNeed
        return CacheNeed(kind="several", members=tuple(part.cache_need() for part in self._members))

    def forward(self, residual: torch.Tensor, pending, ctx: StepContext, cache: CacheView):
        views = list(cache.members)
        if len(views) != len(self._members):
            raise ValueError(f"{self.name}: the cache entry has {len(views)} members, the layer needs {len(self._members)}")
        own, at = views[0], 1
        read = self.mixer_norm.add_forward(residual, pending, self.dtype)
        if self.mixer_conv is not None:
            read = self.mixer_conv.forward(read, ctx, views[at])
            at += 1
        left = self.mixer.forward(read, ctx, own)
        if self.feed_forward is not None:
            read = self.feed_forward_norm.add_forward(residual, left, self.dtype)
            if self.feed_forward_conv is not None:
                read = self.feed_forward_conv.forward(read, ctx, views[at])
            left = self.feed_forward.forward(read, ctx)
        if self.token_input is None:
            return left
        return self.token_input.forward(residual, left, ctx)


register_part("block", "conv_prenorm_residual",
              lambda layer, weights, runtime: ConvPreNormBlock(layer, weights, runtime))


@dataclass
class PairSum:
    """Two sublayers' results on their way into the residual stream: x += scale * (first + second)."""

    first: torch.Tensor
    second: Optional[torch.Tensor]
    scale: float

    def settle(self, residual: torch.Tensor) -> None:
        ops.pair_add_rmsnorm(residual, self.first, self.second, self.scale, None, None, 0.0, torch.float32)


class ParallelResidualBlock:
    """x <- x + m (mixer(norm1(x)) + feed_forward(norm2(x))): both sublayers on the same x."""

    kind = "parallel_residual"

    def __init__(self, layer: LayerSpec, weights: WeightStore, runtime: Runtime):
        from .norm import RMSNorm
        self.name = layer.name
        self.scale = float(layer.block.get("residual_scale", 1.0))
        self.mixer_norm = build_part("norm", layer.mixer_norm, weights, runtime)
        self.mixer = build_part("mixer", layer.mixer, weights, runtime)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, weights, runtime)
        self.feed_forward_norm = None
        if self.feed_forward is not None:
            if layer.feed_forward_norm is None:
                raise ValueError(f"{layer.name}: a feed-forward needs its norm")
            self.feed_forward_norm = build_part("norm", layer.feed_forward_norm, weights, runtime)
        self.dtype = runtime.dtype
        norms = [n for n in (self.mixer_norm, self.feed_forward_norm) if n is not None]
        vector = 8 if self.dtype == torch.bfloat16 else 4
        # one kernel for the sum and both norms: RMS norms with one epsilon over rows the kernel's vectors divide
        self.fused = (all(isinstance(n, RMSNorm) for n in norms) and len({n.eps for n in norms}) == 1
                      and layer.block["hidden_size"] % vector == 0)

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, residual: torch.Tensor, pending, ctx: StepContext, cache: CacheView):
        first = second = None
        scale = 1.0
        if isinstance(pending, PairSum) and self.fused:
            first, second, scale = pending.first, pending.second, pending.scale
        elif pending is not None:
            settle(residual, pending)
        if self.fused:
            second_weight = self.feed_forward_norm.weight if self.feed_forward_norm is not None else None
            normed = ops.pair_add_rmsnorm(residual, first, second, scale, self.mixer_norm.weight, second_weight,
                                          self.mixer_norm.eps, self.dtype)
            mixer_in, feed_in = normed if second_weight is not None else (normed, None)
        else:
            mixer_in = self.mixer_norm.forward(residual, self.dtype)
            feed_in = self.feed_forward_norm.forward(residual, self.dtype) if self.feed_forward is not None else None
        mixed = self.mixer.forward(mixer_in, ctx, cache)
        fed = self.feed_forward.forward(feed_in, ctx) if self.feed_forward is not None else None
        return PairSum(mixed, fed, self.scale)


register_part("block", "parallel_residual",
              lambda layer, weights, runtime: ParallelResidualBlock(layer, weights, runtime))
