"""Grouped-query attention over the paged cache.

q = a Wq^T, k = a Wk^T, v = a Wv^T; optional per-head norms of q and k before
the position encoding; K and V written into the cache; s = (q k^T) * scale with
a causal mask (and an optional window), softmax over keys, query head j reading
key/value head j // (heads / kv_heads); then the output projection
(crates/models/qwen/src/forward.rs:2012-2065, :1967-1989, :2070-2093).

Variants, each a parameter: the norms of q and k may run over a token's whole
projection instead of head by head (``qk_norm_scope="projection"``); a model
without a value projection reuses the key projection's raw output (ahead of
its norm and rotation) as the values (no ``v_proj``); ``chunk`` lets a query
reach back only to the last absolute multiple of that many positions;
``gate_proj`` multiplies the concatenated heads by sigmoid(a Wg^T) ahead of the
output projection (``gate_scope="head"``: Wg has one row per head, and a
head's whole output is multiplied by one number); ``softcap`` c bounds the
scores, s <- c tanh(s / c), ahead of the softmax; ``value_dim`` lets the
values be wider or narrower than the keys (a page then holds rows as wide as
the wider of the two, the others padded with zeros). Values of another width
than the keys run on the general kernel only; a per-head gate is spread over
the head's values for the tensor-core kernels. ``sink`` adds one more key
without a value to every query's softmax, with that score (0.0: the
denominator is 1 + the sum); a tensor's name instead of a number gives every
query head a learned score of its own. ``q_bias`` / ``k_bias`` / ``v_bias``
(tensor names) are added to the projections before their one rounding to the
compute type. ``shared_kv`` marks a layer without key and value projections:
it reads the rows another layer of the same head layout and rotation wrote
into the cache entry it is given, with its own queries, mask, cap and sink.
``value_position`` (a rotary position part over
the values' width) turns the value of position j by j before it is cached and
turns each head's output at position i back by i, so that what a query takes
from a value depends on their distance.

Every size and constant is a parameter. When the head norms are RMSNorms (or
absent) and the position encoding offers cos/sin tables (or is absent), norm,
rotation and cache write run as one kernel; any other norm or position part is
called through its own interface and only the cache write stays here.
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

from .. import ops
from ..config.spec import CacheNeed, PartSpec
from .linear import Linear
from .norm import RMSNorm
from .registry import (CacheView, Prepared, Runtime, StepContext, StepPlan, WeightStore, build_part,
                       register_part)

TILE_TOKENS = 16     # query tokens per tile of the general kernel (csrc/kernels/attention_tile.cu)
WIDE_TOKENS = 128    # ... of the tensor-core prompt kernels (csrc/kernels/attention_prefill*.cu)
PROJECT_TOKENS = 32  # decode steps of up to this many tokens merge their splits and project in one kernel
LONG_CONTEXT = 2048  # a portion of a prompt that sees this many keys or more counts as behind a long context


def attention_tiles(plan: StepPlan) -> Prepared:
    """The lists the attention kernels walk, for one step.

    ``tile_*``: query tiles of up to 16 consecutive tokens of one request,
    those of the requests that bring several tokens first (``multi_tiles`` of
    them), then one per request that brings a single token. ``decode_token`` /
    ``decode_request``: (token, request row) of the requests that bring one
    token, for the split-key kernel (a negative token is a padding row).
    ``wide_*``: tiles of up to 128 tokens over the requests that bring
    several, those with most keys first, for the tensor-core prompt kernels.
    Facts: ``longest_context`` bounds position + 1 of the single tokens,
    ``longest_keys`` the keys a wide tile sees. A portion of a prompt behind
    ``LONG_CONTEXT`` keys or more runs other launches (its keys are shared out
    among blocks) than the same portion at a prompt's start: that is the
    ``graph_key``."""
    counts, starts, live = plan.counts, plan.starts, plan.live
    rows = len(counts)
    if all(count == 1 for count in counts):     # a decode step: no loop over the rows
        index = np.arange(rows, dtype=np.int32)
        alive = index < live
        arrays = {"tile_request": index, "tile_start": index, "tile_length": alive.astype(np.int32),
                  "decode_token": np.where(alive, index, -1).astype(np.int32), "decode_request": index}
        empty = np.empty(0, dtype=np.int32)
        arrays.update(wide_request=empty, wide_start=empty, wide_length=empty)
        longest = plan.context_bound if plan.replayable else max(
            [starts[row] + 1 for row in range(min(live, rows))], default=1)
        return Prepared(arrays, {"multi_tiles": 0, "decode_rows": rows, "longest_context": longest,
                                 "longest_keys": 0}, graph_key=False)
    tile_request, tile_start, tile_length = [], [], []
    singles, wide = [], []
    longest, longest_keys, begin = 0, 0, 0
    for row, (count, start) in enumerate(zip(counts, starts)):
        if count == 1:
            singles.append((row, begin, 1 if row < live else 0))
            longest = max(longest, start + 1)
        else:
            for first in range(0, count, TILE_TOKENS):
                tile_request.append(row)
                tile_start.append(begin + first)
                tile_length.append(min(TILE_TOKENS, count - first))
            longest_keys = max(longest_keys, start + count)
            for first in range(0, count, WIDE_TOKENS):
                size = min(WIDE_TOKENS, count - first)
                wide.append((start + first + size, row, begin + first, size))
        begin += count
    multi_tiles = len(tile_request)
    wide.sort(key=lambda item: -item[0])   # the tiles with most keys start first
    for row, token, length in singles:
        tile_request.append(row)
        tile_start.append(token)
        tile_length.append(length)
    many_keys = longest_keys >= LONG_CONTEXT
    if plan.replayable:   # a graph serves every context of its kind
        longest = plan.context_bound
        longest_keys = plan.context_bound if many_keys else LONG_CONTEXT - 1
    as_array = lambda values: np.asarray(values, dtype=np.int32)
    arrays = {"tile_request": as_array(tile_request), "tile_start": as_array(tile_start),
              "tile_length": as_array(tile_length),
              "decode_token": as_array([token if length else -1 for _, token, length in singles]),
              "decode_request": as_array([row for row, _, _ in singles]),
              "wide_request": as_array([w[1] for w in wide]), "wide_start": as_array([w[2] for w in wide]),
              "wide_length": as_array([w[3] for w in wide])}
    return Prepared(arrays, {"multi_tiles": multi_tiles, "decode_rows": len(singles), "longest_context": longest,
                             "longest_keys": longest_keys}, graph_key=many_keys)


def tiles_of(ctx: StepContext) -> Dict[str, object]:
    """The step's tile lists: what the engine prepared, or (for a caller
    that built a context by hand) made here from the host lists."""
    tiles = ctx.extras.get("attention_tiles")
    if tiles is None:
        if ctx.request_offsets is None:
            raise ValueError("the attention's tile lists were not prepared for this step")
        counts = [ctx.request_offsets[row + 1] - ctx.request_offsets[row] for row in range(ctx.num_requests)]
        ends = [start + count for start, count in zip(ctx.request_positions, counts)]
        prepared = attention_tiles(StepPlan(counts, ctx.request_positions, len(counts), max(ends)))
        tiles = dict(prepared.facts)
        for name, array in prepared.arrays.items():
            tiles[name] = torch.from_numpy(array).to(ctx.device)
        ctx.extras["attention_tiles"] = tiles
    return tiles


def attend_cached(q_heads: torch.Tensor, cache: CacheView, ctx: StepContext, *, scale: float, window: int = 0,
                  chunk: int = 0, softcap: float = 0.0, gate: Optional[torch.Tensor] = None, gate_per_head: bool = False,
                  split_decode: bool = False, flash: bool = False, project=None, sink: Optional[float] = None):
    """Attention of a step's queries ``[tokens, heads, head_dim]`` over what the
    cache entry holds (this step's rows included), each kind of request on the
    kernel made for it: single tokens split along the keys, portions of prompts
    on the tensor cores in tiles of 128, whatever is left (and everything, where
    those kernels do not take the head layout or the type) on the general
    kernel. Returns (``[tokens, heads, head_dim]``, False); with ``project`` (the
    output projection, a ``Linear``) a step of few single tokens may come back
    as (float32 ``[heads, tokens, hidden]`` summands, True), merged and
    projected by one kernel."""
    tokens, heads, head_dim = q_heads.shape
    tiles = tiles_of(ctx)
    multi_tiles = tiles["multi_tiles"]
    split = tiles["decode_rows"] and split_decode
    kv_heads = cache.pool.shape[2]
    # The gate, if any, rides in whichever kernel writes a token's output.
    if (project is not None and split and multi_tiles == 0 and tokens <= PROJECT_TOKENS and project.rows_are_short()
            and ops.decode_project_supported(head_dim, heads, kv_heads, q_heads.dtype, tokens, project.weight)):
        # Only single tokens, at most 64 of them: the splits are merged
        # and projected by one kernel, one summand per head.
        return ops.paged_attention_decode_project(
            q_heads, cache.pool, cache.block_tables, tiles["decode_token"], tiles["decode_request"],
            ctx.positions, scale, tiles["longest_context"], project.weight, window, chunk, gate=gate,
            softcap=softcap, sink=sink), True
    out = torch.empty_like(q_heads)
    if split:
        # Requests that bring one token: split along the keys.
        ops.paged_attention_decode(q_heads, cache.pool, out, cache.block_tables, tiles["decode_token"],
                                   tiles["decode_request"], ctx.positions, scale, tiles["longest_context"], window,
                                   chunk=chunk, gate=gate, softcap=softcap, sink=sink)
    if flash:
        # Requests that bring several tokens: tensor cores, tiles of 128.
        if tiles["wide_request"].numel():
            ops.flash_prefill(q_heads, cache.pool, out, cache.block_tables, tiles["wide_request"],
                              tiles["wide_start"], tiles["wide_length"], ctx.positions, scale, window,
                              longest_context=tiles["longest_keys"], chunk=chunk, gate=gate, softcap=softcap,
                              sink=sink)
        rest = None if split else slice(multi_tiles, None)   # single tokens not yet served
    else:
        rest = slice(0, multi_tiles) if split else slice(0, None)
    if rest is not None and tiles["tile_request"][rest].numel():
        ops.paged_attention_tile(q_heads, cache.pool, out, cache.block_tables, tiles["tile_request"][rest],
                                 tiles["tile_start"][rest], tiles["tile_length"][rest], ctx.positions,
                                 scale, window, chunk, gate=gate, softcap=softcap, gate_per_head=gate_per_head,
                                 sink=sink)
    return out, False


class GQAttention:
    kind = "gqa_attention"
    graph_safe = True  # launches the same kernels whatever the step's integers are
    step_key = "attention_tiles"   # every attention layer of a model walks the same lists
    prepare_step = staticmethod(attention_tiles)

    def __init__(self, spec: PartSpec, weights: WeightStore, runtime: Runtime):
        self.hidden_size = spec["hidden_size"]
        self.num_heads = spec["num_heads"]
        self.num_kv_heads = spec["num_kv_heads"]
        self.head_dim = spec["head_dim"]
        self.scale = float(spec["scale"])
        self.window = spec.get("window") or 0
        self.chunk = spec.get("chunk") or 0
        self.norm_scope = spec.get("qk_norm_scope") or "head"
        if self.norm_scope not in ("head", "projection"):
            raise ValueError(f"qk_norm_scope must be 'head' or 'projection', got {self.norm_scope!r}")
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} query heads cannot share {self.num_kv_heads} key/value heads")
        if self.head_dim % 2 or not 0 < self.head_dim <= 256:
            raise ValueError(f"head_dim {self.head_dim}: the attention kernels take even sizes up to 256")
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.value_dim = spec.get("value_dim") or self.head_dim
        self.softcap = float(spec.get("softcap") or 0.0)
        self.gate_scope = spec.get("gate_scope") or "value"
        if self.gate_scope not in ("value", "head"):
            raise ValueError(f"gate_scope must be 'value' or 'head', got {self.gate_scope!r}")
        if self.softcap < 0.0 or not 0 < self.value_dim <= 576:
            raise ValueError(f"softcap {self.softcap} or value_dim {self.value_dim} out of range")
        self.v_size = self.num_kv_heads * self.value_dim
        self.out_size = self.num_heads * self.value_dim
        self.row_dim = max(self.head_dim, self.value_dim)      # width of a cached row
        # v_proj absent: the key projection's raw output is the values too. gate_proj: an
        # output gate over the concatenated heads, from the mixer's own input.
        # shared_kv: no key or value projection at all; the cache entry another layer writes is read.
        self.own_keys = not spec.get("shared_kv")
        self.own_values = spec.get("v_proj") is not None and self.own_keys
        self.gated = spec.get("gate_proj") is not None
        stacked, biases, biased = [], [], False
        if self.own_keys and not self.own_values and self.value_dim != self.head_dim:
            raise ValueError("values taken from the key projection are as wide as the keys")
        gate_rows = self.num_heads if self.gate_scope == "head" else self.out_size
        for name, rows, present, bias in (("q_proj", self.q_size, True, "q_bias"),
                                          ("k_proj", self.kv_size, self.own_keys, "k_bias"),
                                          ("v_proj", self.v_size, self.own_values, "v_bias"),
                                          ("gate_proj", gate_rows, self.gated, None)):
            if not present:
                continue
            weight = weights.take(spec[name])
            if tuple(weight.shape) != (rows, self.hidden_size):
                raise ValueError(f"{spec[name]} is {tuple(weight.shape)}, expected {(rows, self.hidden_size)}")
            stacked.append(weight)
            if bias is not None and spec.get(bias):
                values = weights.take(spec[bias])
                if values.numel() != rows:
                    raise ValueError(f"{spec[bias]} has {values.numel()} values, expected {rows}")
                biases.append(values.to(device=runtime.device, dtype=torch.float32).reshape(-1))
                biased = True
            else:
                biases.append(torch.zeros(rows, dtype=torch.float32, device=runtime.device))
        # rows: all q heads, then k heads, then v heads (if any), then the gate (if any)
        self.qkv = Linear.stacked(stacked, runtime)
        self.bias = torch.cat(biases).contiguous() if biased else None   # one value per row of the stacked product
        if not self.own_keys:
            self.kv_size = self.v_size = 0     # nothing of them in the stacked product
        self.gate_offset = self.q_size + self.kv_size + (self.v_size if self.own_values else 0)
        self.gate_rows = gate_rows
        self.o = Linear(weights.take(spec["o_proj"]), runtime)
        if (self.o.out_features, self.o.in_features) != (self.hidden_size, self.out_size):
            raise ValueError(f"{spec['o_proj']} is {tuple(self.o.weight.shape)}")
        self.q_norm = build_part("norm", spec.get("q_norm"), weights, runtime)
        self.k_norm = build_part("norm", spec.get("k_norm"), weights, runtime)
        self.position = build_part("position", spec.get("position"), weights, runtime)
        sink = spec.get("sink")
        if isinstance(sink, str):     # a learned score per query head
            values = weights.take(sink)
            if values.numel() != self.num_heads:
                raise ValueError(f"{sink} has {values.numel()} values, expected one per head ({self.num_heads})")
            self.sink = values.to(device=runtime.device, dtype=torch.float32).reshape(-1).contiguous()
        else:
            self.sink = None if sink is None else float(sink)
        self.value_position = build_part("position", spec.get("value_position"), weights, runtime)
        if self.value_position is not None:
            if not getattr(self.value_position, "fused_tables", False) or self.value_position.head_dim != self.value_dim:
                raise ValueError("value_position must be a rotary part with cos/sin tables over value_dim")
            if self.gated:
                raise ValueError("an output gate inside the attention kernels cannot follow the values' turn back")
        for name, norm, width in (("q_norm", self.q_norm, self.q_size), ("k_norm", self.k_norm, self.kv_size)):
            expected = self.head_dim if self.norm_scope == "head" else width
            if norm is not None and getattr(norm, "size", expected) != expected:
                raise ValueError(f"{name} is over {norm.size} values; with qk_norm_scope {self.norm_scope!r} "
                                 f"it must be over {expected}")
        norms_fuse = all(n is None or isinstance(n, RMSNorm) for n in (self.q_norm, self.k_norm))
        eps_agree = (self.q_norm is None or self.k_norm is None or self.q_norm.eps == self.k_norm.eps)
        position_fuses = self.position is None or getattr(self.position, "fused_tables", False)
        self.dtype = runtime.dtype
        # What only the general kernel does: values of another width than the keys.
        self.general_only = self.value_dim != self.head_dim
        self.fused = norms_fuse and eps_agree and position_fuses and self.value_dim == self.head_dim
        self.split_decode = not self.general_only and ops.decode_attention_supported(
            self.head_dim, self.num_heads, self.num_kv_heads, self.dtype)
        self.flash = not self.general_only and ops.flash_prefill_supported(
            self.head_dim, self.num_heads, self.num_kv_heads, self.dtype)

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="kv_pages", kv_heads=self.num_kv_heads, head_dim=self.row_dim,
                         window=self.window or None, chunk=self.chunk or None)

    def parts(self):
        return [self.q_norm, self.k_norm, self.position, self.value_position]

    def _turn_values(self, v: torch.Tensor, ctx: StepContext, back: bool = False) -> torch.Tensor:
        """``[tokens, n * value_dim]`` turned by each token's position (``back``: by minus it)."""
        turn = self.value_position
        return ops.norm_rotate_heads(v, self.value_dim, ctx.positions, cos=turn.cos,
                                     sin=turn.inverse_sin() if back else turn.sin, interleaved=turn.interleaved)

    def _tiles(self, ctx: StepContext) -> Dict[str, object]:
        return tiles_of(ctx)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        return self._attend(x, ctx, cache, summands=False)

    def forward_summands(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        """``forward`` for a caller that adds up summands: where one kernel can
        put the splits of a decode step together and project them head by head,
        the result is float32 ``[heads, tokens, hidden]`` whose sum over the
        heads is ``forward``'s output; otherwise ``forward``'s output itself."""
        return self._attend(x, ctx, cache, summands=True)

    def _attend(self, x: torch.Tensor, ctx: StepContext, cache: CacheView, summands: bool) -> torch.Tensor:
        tokens = x.shape[0]
        if self.bias is not None:
            # the product leaves in float32 and meets the bias there: one rounding to the compute type
            qkv = ops.add_bias(self.qkv.forward(x, out_dtype=torch.float32), self.bias, self.dtype)
        else:
            qkv = self.qkv.forward(x)
        q = qkv[:, :self.q_size]
        k = qkv[:, self.q_size:self.q_size + self.kv_size]
        v = qkv[:, self.q_size + self.kv_size:self.q_size + self.kv_size + self.v_size] if self.own_values else k
        gate = qkv[:, self.gate_offset:self.gate_offset + self.gate_rows] if self.gated else None
        per_head = self.norm_scope == "head"
        if self.value_position is not None and self.own_keys:     # cached turned by their own position
            v = self._turn_values(v, ctx).view(tokens, self.v_size)
        if self.value_dim != self.head_dim:
            return self._attend_unequal(x, q, k, v, gate, ctx, cache)
        q_heads = torch.empty((tokens, self.num_heads, self.head_dim), dtype=self.dtype, device=x.device)
        write = cache.write and cache.slots is not None and self.own_keys
        if not self.own_keys and self.fused:
            # queries only: their norm and rotation; the keys and values are another layer's, in the cache already
            q_heads = ops.norm_rotate_heads(
                q, self.head_dim, ctx.positions, weight=self.q_norm.weight if self.q_norm is not None else None,
                cos=self.position.cos if self.position is not None else None,
                sin=self.position.sin if self.position is not None else None,
                eps=self.q_norm.eps if self.q_norm is not None else 0.0,
                interleaved=bool(getattr(self.position, "interleaved", False)), norm_scope=self.norm_scope)
        elif self.fused:
            eps = self.q_norm.eps if self.q_norm is not None else (self.k_norm.eps if self.k_norm else 0.0)
            ops.qk_norm_rope_cache(
                q, k, v, q_heads, cache.pool if write else None, cache.slots if write else None,
                ctx.positions,
                self.q_norm.weight if self.q_norm is not None else None,
                self.k_norm.weight if self.k_norm is not None else None,
                self.position.cos if self.position is not None else None,
                self.position.sin if self.position is not None else None, eps,
                interleaved=bool(getattr(self.position, "interleaved", False)), norm_scope=self.norm_scope)
        else:
            if not self.own_keys:
                raise ValueError("a layer that reads another layer's keys needs head norms and a position part "
                                 "that the fused kernel takes")
            if not self.own_values:
                v = k   # as projected: before the norm and the rotation below
            if self.q_norm is not None:
                rows = (tokens * self.num_heads, self.head_dim) if per_head else (tokens, self.q_size)
                q = self.q_norm.forward(q.reshape(rows).contiguous(), self.dtype).view(tokens, self.q_size)
            if self.k_norm is not None:
                rows = (tokens * self.num_kv_heads, self.head_dim) if per_head else (tokens, self.kv_size)
                k = self.k_norm.forward(k.reshape(rows).contiguous(), self.dtype).view(tokens, self.kv_size)
            if self.position is not None:
                q_rot, k_rot = self.position.apply(q, k, ctx.positions)
                q_heads = q_rot.contiguous().view(tokens, self.num_heads, self.head_dim)
                k = k_rot.contiguous().view(tokens, self.kv_size)
            else:
                q_heads = q.contiguous().view(tokens, self.num_heads, self.head_dim)
            if write:
                ops.write_cache(k, v, cache.pool, cache.slots, ctx.positions)
        if self.gate_scope == "head" and gate is not None and (self.split_decode or self.flash):
            # the tensor-core kernels take one gate per value: a head's number is spread over its values
            gate = gate.unsqueeze(2).expand(tokens, self.num_heads, self.head_dim).reshape(tokens, self.q_size)
            per_head_gate = False
        else:
            per_head_gate = self.gate_scope == "head"
        out, projected = attend_cached(
            q_heads, cache, ctx, scale=self.scale, window=self.window, chunk=self.chunk, softcap=self.softcap, gate=gate,
            gate_per_head=per_head_gate, split_decode=self.split_decode, flash=self.flash,
            project=self.o if summands and self.value_position is None else None, sink=self.sink)
        if projected:
            return out
        if self.value_position is not None:
            out = self._turn_values(out.view(tokens, self.q_size), ctx, back=True)
        return self.o.forward(out.view(tokens, self.q_size))

    def _attend_unequal(self, x, q, k, v, gate, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        """Values wider or narrower than the keys: a cached row is as wide as
        the wider of the two; queries, keys or values are padded with zeros up
        to it, and the output keeps the first ``value_dim`` values."""
        tokens, width = x.shape[0], self.row_dim
        per_head = self.norm_scope == "head"
        parts = []
        for rows, norm, heads in ((q, self.q_norm, self.num_heads), (k, self.k_norm, self.num_kv_heads)):
            if rows is k and not self.own_keys:
                parts.append(None)     # another layer's keys and values, in the cache already
                continue
            weight = norm.weight if norm is not None else None
            if norm is not None and not isinstance(norm, RMSNorm):
                shape = (tokens * heads, self.head_dim) if per_head else (tokens, heads * self.head_dim)
                rows = norm.forward(rows.reshape(shape).contiguous(), self.dtype).view(tokens, heads * self.head_dim)
                weight = None
            tables = self.position is not None and getattr(self.position, "fused_tables", False)
            if self.position is not None and not tables:
                raise ValueError("values of another width than the keys need a position part with cos/sin tables")
            parts.append(ops.norm_rotate_heads(
                rows, self.head_dim, ctx.positions, weight=weight, cos=self.position.cos if tables else None,
                sin=self.position.sin if tables else None, eps=norm.eps if weight is not None else 0.0,
                interleaved=bool(getattr(self.position, "interleaved", False)), norm_scope=self.norm_scope))
        q_heads, k_heads = parts
        pad = lambda t, have: torch.nn.functional.pad(t, (0, width - have)) if have < width else t
        q_rows = pad(q_heads, self.head_dim).contiguous()
        if cache.write and cache.slots is not None and self.own_keys:
            k_rows = pad(k_heads, self.head_dim).reshape(tokens, self.num_kv_heads * width)
            v_rows = pad(v.reshape(tokens, self.num_kv_heads, self.value_dim), self.value_dim) \
                .reshape(tokens, self.num_kv_heads * width)
            ops.write_cache(k_rows, v_rows, cache.pool, cache.slots, ctx.positions)
        tiles = tiles_of(ctx)
        out = torch.empty((tokens, self.num_heads, self.value_dim), dtype=self.dtype, device=x.device)
        ops.paged_attention_tile(q_rows, cache.pool, out, cache.block_tables, tiles["tile_request"],
                                 tiles["tile_start"], tiles["tile_length"], ctx.positions, self.scale, self.window,
                                 self.chunk, gate=gate, softcap=self.softcap,
                                 gate_per_head=self.gate_scope == "head", sink=self.sink)
        if self.value_position is not None:
            out = self._turn_values(out.view(tokens, self.out_size), ctx, back=True)
        return self.o.forward(out.view(tokens, self.out_size))

    def weight_bytes(self) -> int:
        return self.qkv.weight_bytes() + self.o.weight_bytes()


register_part("mixer", "gqa_attention", lambda spec, weights, runtime: GQAttention(spec, weights, runtime))
