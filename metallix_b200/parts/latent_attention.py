"""Attention whose keys and values come from one small latent per position.

With H heads, per head D unrotated and R rotated query/key values, value
width V, latent width r (and a query latent of width rq):

    cq = RMSNorm(a Wdq^T),  q = cq Wuq^T          per head [D unrotated | R rotated]
    a Wdkv^T = [z (r values) | kr (R values)],  c = RMSNorm(z)
    head h:  k_h = Wuk_h c,  v_h = Wuv_h c
    score = (q_u . k_h + rot(q_r) . rot(kr)) * scale,  causal softmax,  out = concat_h(sum_j p_j v_h,j) Wo^T

Only c and rot(kr) are cached: one row of r + R values per position, shared
by all heads (a pool of one plane and one key/value head). The up-projections
are moved to the query's side, which is the same arithmetic in another order:
q_u . (Wuk_h c) = (Wuk_h^T q_u) . c, and sum_j p_j Wuv_h c_j = Wuv_h (sum_j p_j c_j).
So a head's query against the cache is [Wuk_h^T q_u | rot(q_r)] (r + R values),
its output a mixture of latents (r values) that Wuv_h widens to V afterwards:
attention with H query heads over one shared key/value head, whatever the
context's length. That is ``cache_mode="latent"``: the least memory, on the
general attention kernel.

Without ``q_rank`` the queries come from one projection, q = a Wq^T, with no
latent of their own. ``window`` lets a query see only the last that many
positions (its own included), ``sink`` adds one more key without a value to
every query's softmax, with one score for all heads (a number) or a learned
score per head (a tensor's name); both reach whichever kernel serves the step.

``cache_mode="heads"`` keeps the equations in their first order instead: every
position's latent is widened once, when it arrives, to each head's key
[k_h | rot(kr)] and value v_h, and those rows are cached per head (padded
with zeros to a head size the tensor-core kernels take: 64, 128 or 256). The
cache is H (D + R + V) / (r + R) times as large; prompts and decode steps then
run on the same kernels as grouped-query attention. ``"auto"`` takes the
per-head rows where such a head size exists (keys and values up to 256 wide).
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import CacheNeed, PartSpec
from .attention import attend_cached, attention_tiles, tiles_of
from .linear import Linear
from .registry import CacheView, Runtime, StepContext, WeightStore, build_part, register_part


class LatentAttention:
    kind = "latent_attention"
    graph_safe = True
    step_key = "attention_tiles"
    prepare_step = staticmethod(attention_tiles)

    def __init__(self, spec: PartSpec, weights: WeightStore, runtime: Runtime):
        hidden = spec["hidden_size"]
        self.heads, self.dim, self.rot = spec["num_heads"], spec["head_dim"], spec["rotary_head_dim"]
        self.vdim, self.rank, self.q_rank = spec["value_dim"], spec["kv_rank"], spec.get("q_rank") or 0
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.width = self.rank + self.rot           # what a position's cache row holds
        if not 0 < self.width <= 576:
            raise ValueError(f"latent plus rotated key is {self.width} values wide; the kernel takes up to 576")
        H, D, R, V = self.heads, self.dim, self.rot, self.vdim

        def matrix(name, shape):
            weight = weights.take(spec[name])
            if tuple(weight.shape) != shape:
                raise ValueError(f"{spec[name]} is {tuple(weight.shape)}, expected {shape}")
            return weight

        if self.q_rank:
            self.dq = Linear(matrix("q_down_proj", (self.q_rank, hidden)), runtime)
            self.uq = Linear(matrix("q_up_proj", (H * (D + R), self.q_rank)), runtime)
            self.q_norm = build_part("norm", spec["q_norm"], weights, runtime)
        else:   # queries straight from the mixer's input
            self.dq, self.q_norm = None, None
            self.uq = Linear(matrix("q_proj", (H * (D + R), hidden)), runtime)
        self.dkv = Linear(matrix("kv_down_proj", (self.width, hidden)), runtime)
        self.window = int(spec.get("window") or 0)
        sink = spec.get("sink")
        if isinstance(sink, str):
            values = weights.take(sink)
            if values.numel() != H:
                raise ValueError(f"{sink} has {values.numel()} values, expected one per head ({H})")
            self.sink = values.to(device=runtime.device, dtype=torch.float32).reshape(-1).contiguous()
        else:
            self.sink = None if sink is None else float(sink)
        self.kv_norm = build_part("norm", spec["kv_norm"], weights, runtime)
        on_device = lambda t: t.to(device=runtime.device, dtype=runtime.dtype).contiguous()
        uk = on_device(matrix("k_up_proj", (H * D, self.rank))).view(H, D, self.rank)
        self.uk = uk                                            # [H, D, r]: q_u @ uk[h] -> latent side
        self.uk_t = uk.transpose(1, 2).contiguous() if runtime.dtype == torch.float32 else None   # [H, r, D]
        self.uv = on_device(matrix("v_up_proj", (H * V, self.rank))).view(H, V, self.rank)
        self.o = Linear(matrix("o_proj", (hidden, H * V)), runtime)
        self.position = build_part("position", spec.get("position"), weights, runtime)
        self.dtype = runtime.dtype
        mode = spec.get("cache_mode") or "auto"
        if mode not in ("auto", "latent", "heads"):
            raise ValueError(f"cache_mode must be 'auto', 'latent' or 'heads', got {mode!r}")
        widest = max(D + R, V)
        self.head_size = next((size for size in (64, 128, 256) if size >= widest), 0)
        if mode == "heads" and not self.head_size:
            raise ValueError(f"keys of {D + R} and values of {V} do not fit a head of up to 256 values")
        self.per_head = mode == "heads" or (mode == "auto" and bool(self.head_size))
        if self.per_head:
            hd = self.head_size
            # keys and values from the latent in one product: rows of uk, then rows of uv
            self.kv_up = Linear.stacked([self.uk.reshape(H * D, self.rank), self.uv.reshape(H * V, self.rank)], runtime)
            if V != hd:   # the output projection over padded heads: zero columns where the padding is
                padded = torch.zeros((hidden, H, hd), dtype=self.o.weight.dtype, device=self.o.weight.device)
                padded[:, :, :V] = self.o.weight.view(hidden, H, V)
                self.o = Linear(padded.view(hidden, H * hd), runtime)
            self.uk = self.uk_t = self.uv = None
            self.split_decode = ops.decode_attention_supported(hd, H, H, self.dtype)
            self.flash = ops.flash_prefill_supported(hd, H, H, self.dtype)

    def cache_need(self) -> CacheNeed:
        if self.per_head:
            return CacheNeed(kind="kv_pages", kv_heads=self.heads, head_dim=self.head_size, window=self.window or None)
        return CacheNeed(kind="kv_pages", kv_heads=1, head_dim=self.width, planes=1, window=self.window or None)

    def _queries(self, x: torch.Tensor) -> torch.Tensor:
        """[tokens, H * (D + R)]: through their own normed latent, or straight from the input."""
        if self.dq is None:
            return self.uq.forward(x)
        return self.uq.forward(self.q_norm.forward(self.dq.forward(x), self.dtype))

    def parts(self):
        return [self.q_norm, self.kv_norm, self.position]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        tokens, H, D, R, V, r = x.shape[0], self.heads, self.dim, self.rot, self.vdim, self.rank
        cos = self.position.cos if self.position is not None else None
        sin = self.position.sin if self.position is not None else None
        paired = bool(getattr(self.position, "interleaved", False))
        if self.per_head:
            return self._forward_per_head(x, ctx, cache, cos, sin, paired)
        # the position's cache row: normed latent, rotated shared key part
        if cache.write and cache.slots is not None:
            ops.latent_cache(self.dkv.forward(x), self.kv_norm.weight, self.kv_norm.eps, r, cache.pool, cache.slots,
                             ctx.positions, cos, sin, paired)
        # queries: through their own latent, then onto the cache's side
        q = self._queries(x)                                                            # [tokens, H * (D + R)]
        q_heads = q.view(tokens, H, D + R)
        q_cache = torch.empty((tokens, H, self.width), dtype=self.dtype, device=x.device)
        if self.dtype == torch.float32:
            for h in range(H):
                ops.gemm_simple(q_heads[:, h, :D], self.uk_t[h], out=q_cache[:, h, :r])
        else:
            q_cache[:, :, :r].copy_(torch.bmm(q_heads[:, :, :D].transpose(0, 1), self.uk).transpose(0, 1))
        ops.rotate_into(q, D, D + R, q_cache, r, R, ctx.positions, cos, sin, paired)
        tiles = tiles_of(ctx)
        mixed = torch.empty((tokens, H, r), dtype=self.dtype, device=x.device)
        ops.paged_attention_tile(q_cache, cache.pool, mixed, cache.block_tables, tiles["tile_request"],
                                 tiles["tile_start"], tiles["tile_length"], ctx.positions, self.scale, self.window,
                                 sink=self.sink)
        # latents back to values, head by head
        if self.dtype == torch.float32:
            values = torch.empty((tokens, H * V), dtype=self.dtype, device=x.device)
            for h in range(H):
                ops.gemm_simple(mixed[:, h, :], self.uv[h], out=values[:, h * V:(h + 1) * V])
        else:
            values = torch.bmm(mixed.transpose(0, 1), self.uv.transpose(1, 2)).transpose(0, 1).reshape(tokens, H * V)
        return self.o.forward(values)

    def _forward_per_head(self, x, ctx: StepContext, cache: CacheView, cos, sin, paired: bool) -> torch.Tensor:
        tokens, H, D, R, V, r, hd = x.shape[0], self.heads, self.dim, self.rot, self.vdim, self.rank, self.head_size
        # [normed latent | rotated shared key part] of this step's tokens, then every head's keys and values
        rows = ops.latent_cache(self.dkv.forward(x), self.kv_norm.weight, self.kv_norm.eps, r, None, None,
                                ctx.positions, cos, sin, paired)
        widened = self.kv_up.forward(rows[:, :r])                                       # [tokens, H * D + H * V]
        q = self._queries(x)                                                            # [tokens, H * (D + R)]
        q_heads = torch.empty((tokens, H, hd), dtype=self.dtype, device=x.device)
        write = cache.write and cache.slots is not None
        ops.latent_heads(q, widened, rows, r, q_heads, cache.pool if write else None, cache.slots if write else None,
                         ctx.positions, cos, sin, paired, D, R, V)
        out, _ = attend_cached(q_heads, cache, ctx, scale=self.scale, window=self.window, split_decode=self.split_decode,
                               flash=self.flash, sink=self.sink)
        return self.o.forward(out.view(tokens, H * hd))

    def weight_bytes(self) -> int:
        queries = self.uq.weight_bytes() + (self.dq.weight_bytes() if self.dq is not None else 0)
        if self.per_head:
            return queries + self.dkv.weight_bytes() + self.o.weight_bytes() + self.kv_up.weight_bytes()
        element = self.uk.element_size()
        return (queries + self.dkv.weight_bytes() + self.o.weight_bytes()
                + (self.uk.numel() + self.uv.numel()) * element)


register_part("mixer", "latent_attention", lambda spec, weights, runtime: LatentAttention(spec, weights, runtime))
