"""The matrix-memory recurrence (mLSTM) as a mixer with its state in the
cache's request slots.

Per head, with key width D and value width V, a request carries a matrix
C [D, V], a vector n [D] and a running maximum m (all float32, all zero at
the start of a sequence; m starts at 0, not at minus infinity). A token with
input a brings q = a Wq^T D^-1/2, k = a Wk^T, v = a Wv^T and, with a cap c,

    i = c tanh((a Wi^T + bi) / c)             log of the input gate
    f = logsigmoid(c tanh((a Wf^T + bf) / c)) log of the forget gate
    m' = max(f + m, i)
    C' = exp(f + m - m') C + exp(i - m') k v^T,   n' likewise with k alone
    o  = C'^T q / (max(|n' . q|, exp(-m')) + 1e-6)

Each head's o is divided by its root mean square, the heads side by side are
multiplied by a weight and by sigmoid(a Wg^T), and projected by Wo. The six
projections are one product whose output stays float32, since the gates, the
state and everything that meets them are float32 in both precisions.

A step's tokens of one request are walked in order by one kernel, whether the
step brings one token or a portion of a prompt; what is carried between steps
is the exact state, so a position's output does not depend on how the prompt
was cut.
"""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch

from .. import ops
from ..config.spec import CacheNeed, PartSpec
from .linear import Linear
from .registry import CacheView, Prepared, Runtime, StepContext, StepPlan, WeightStore, register_part


def request_rows(plan: StepPlan) -> Prepared:
    """Where each request row's tokens lie in the packed step: ``row_start``
    and ``row_length`` (0 for a padding row, which owns no state); ``longest``,
    the most tokens any row brings, decides which form of the recurrence's
    kernel runs (and with it which steps may share a captured graph)."""
    counts = np.asarray(plan.counts, dtype=np.int64)
    starts = np.zeros(len(counts), dtype=np.int64)
    np.cumsum(counts[:-1], out=starts[1:])
    lengths = np.where(np.arange(len(counts)) < plan.live, counts, 0)
    longest = int(counts.max()) if len(counts) else 1
    return Prepared({"row_start": starts.astype(np.int32), "row_length": lengths.astype(np.int32)},
                    {"longest": longest}, graph_key=longest >= 8)


def request_rows_of(ctx: StepContext) -> Dict[str, torch.Tensor]:
    """The step's request rows: what the engine prepared, or (for a caller that
    built a context by hand) made here from the host lists."""
    rows = ctx.extras.get("request_rows")
    if rows is None:
        if ctx.request_offsets is None:
            raise ValueError("the request rows were not prepared for this step")
        counts = [ctx.request_offsets[row + 1] - ctx.request_offsets[row] for row in range(ctx.num_requests)]
        prepared = request_rows(StepPlan(counts, ctx.request_positions, len(counts), 0))
        rows = dict(prepared.facts)
        rows.update({name: torch.from_numpy(array).to(ctx.device) for name, array in prepared.arrays.items()})
        ctx.extras["request_rows"] = rows
    return rows


class MatrixMemory:
    kind = "mlstm"
    graph_safe = True
    step_key = "request_rows"
    prepare_step = staticmethod(request_rows)

    def __init__(self, spec: PartSpec, weights: WeightStore, runtime: Runtime):
        hidden = spec["hidden_size"]
        self.heads, self.dim, self.vdim = spec["num_heads"], spec["head_dim"], spec["value_dim"]
        self.cap, self.eps = float(spec["gate_cap"]), float(spec["eps"])
        if self.cap <= 0.0:
            raise ValueError(f"gate_cap must be positive, got {self.cap}")
        k_size, v_size = self.heads * self.dim, self.heads * self.vdim
        stacked, self.offsets, cursor = [], {}, 0
        for name, rows in (("q_proj", k_size), ("k_proj", k_size), ("v_proj", v_size), ("gate_proj", v_size),
                           ("input_gate_proj", self.heads), ("forget_gate_proj", self.heads)):
            weight = weights.take(spec[name])
            if tuple(weight.shape) != (rows, hidden):
                raise ValueError(f"{spec[name]} is {tuple(weight.shape)}, expected {(rows, hidden)}")
            stacked.append(weight)
            self.offsets[name] = cursor
            cursor += rows
        self.inputs = Linear.stacked(stacked, runtime)   # rows: q, k, v, output gate, input gate, forget gate
        as_float = lambda name, size: self._vector(weights.take(spec[name]), size, spec[name], runtime)
        self.input_bias = as_float("input_gate_bias", self.heads)
        self.forget_bias = as_float("forget_gate_bias", self.heads)
        self.norm_weight = as_float("norm", v_size)
        self.o = Linear(weights.take(spec["o_proj"]), runtime)
        if (self.o.out_features, self.o.in_features) != (hidden, v_size):
            raise ValueError(f"{spec['o_proj']} is {tuple(self.o.weight.shape)}")
        self.dtype = runtime.dtype
        self.state_values = self.heads * (self.dim * self.vdim + (-(-self.vdim // 32)) * (self.dim + 1))

    @staticmethod
    def _vector(tensor: torch.Tensor, size: int, name: str, runtime: Runtime) -> torch.Tensor:
        if tensor.numel() != size:
            raise ValueError(f"{name} has {tensor.numel()} values, expected {size}")
        return tensor.to(device=runtime.device, dtype=torch.float32).reshape(-1).contiguous()

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="state", state_shape=(self.state_values,), state_dtype="float32")

    def _rows(self, ctx: StepContext) -> Dict[str, torch.Tensor]:
        return request_rows_of(ctx)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        if cache.state is None:
            raise ValueError("the matrix-memory mixer needs a state entry of the cache")
        rows = self._rows(ctx)
        proj = self.inputs.forward(x, out_dtype=torch.float32)
        at = self.offsets
        memory = ops.mlstm_scan(proj, (at["q_proj"], at["k_proj"], at["v_proj"], at["input_gate_proj"],
                                       at["forget_gate_proj"]), self.input_bias, self.forget_bias, self.cap,
                                cache.state, rows["row_start"], rows["row_length"], ctx.request_slots,
                                self.heads, self.dim, self.vdim, longest=rows.get("longest", 1))
        gate = proj[:, at["gate_proj"]:at["gate_proj"] + self.heads * self.vdim]
        return self.o.forward(ops.head_norm_gate(memory, self.norm_weight, gate, self.heads, self.eps, self.dtype))

    def weight_bytes(self) -> int:
        return self.inputs.weight_bytes() + self.o.weight_bytes()


register_part("mixer", "mlstm", lambda spec, weights, runtime: MatrixMemory(spec, weights, runtime))


class SelectiveScan:
    """The selective state-space mixer (Mamba): a Win^T = [x | z]; x passes a
    short causal convolution with bias and silu; x Wx^T = [dt | B | C] with a
    low-rank step size dt <- softplus(dt Wdt^T + b); A = -exp(A_log); per
    channel c and state n

        S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n,    y_c = sum_n S[c, n] C_n + D_c x_c;

    then y * silu(z) and the output projection. The state S (float32,
    ``[inner, states]``), and the convolution's last inputs, are kept per request
    in the cache's state slots. Step sizes, decays and the recurrence are
    float32 in both precisions (the step size's product leaves in float32);
    the projections, the convolution and what they hand on are in the compute
    type."""

    kind = "selective_scan"
    graph_safe = True
    step_key = "request_rows"
    prepare_step = staticmethod(request_rows)

    def __init__(self, spec: PartSpec, weights: WeightStore, runtime: Runtime):
        from .short_conv import ShortConv
        hidden = spec["hidden_size"]
        self.inner, self.states, self.rank = int(spec["inner_size"]), int(spec["state_size"]), int(spec["step_rank"])
        if not 0 < self.states <= ops.SCAN_STATES:
            raise ValueError(f"{self.states} states per channel; the scan takes up to {ops.SCAN_STATES}")

        def matrix(name, shape):
            weight = weights.take(spec[name])
            if tuple(weight.shape) != shape:
                raise ValueError(f"{spec[name]} is {tuple(weight.shape)}, expected {shape}")
            return weight

        def vector(name, size):
            tensor = weights.take(spec[name])
            if tensor.numel() != size:
                raise ValueError(f"{spec[name]} has {tensor.numel()} values, expected {size}")
            return tensor.to(device=runtime.device, dtype=torch.float32).reshape(-1).contiguous()

        self.inputs = Linear(matrix("in_proj", (2 * self.inner, hidden)), runtime)      # rows: x, then z
        self.conv = ShortConv(PartSpec("short_conv", {
            "channels": self.inner, "taps": int(spec["conv_taps"]), "weight": spec["conv_weight"],
            "bias": spec.get("conv_bias"), "activation": "silu"}), weights, runtime)
        self.selectors = Linear(matrix("x_proj", (self.rank + 2 * self.states, self.inner)), runtime)   # dt, B, C
        self.step = Linear(matrix("step_proj", (self.inner, self.rank)), runtime)
        self.step_bias = vector("step_bias", self.inner)
        a_log = matrix("a_log", (self.inner, self.states))
        self.decay = (-torch.exp(a_log.to(device=runtime.device, dtype=torch.float32))).contiguous()
        self.skip = vector("skip", self.inner)
        self.o = Linear(matrix("o_proj", (hidden, self.inner)), runtime)
        self.dtype = runtime.dtype

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="several", members=(
            CacheNeed(kind="state", state_shape=(self.inner, self.states), state_dtype="float32"),
            self.conv.cache_need()))

    def parts(self):
        return [self.conv]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        if len(cache.members) != 2 or cache.members[0].state is None:
            raise ValueError("the selective scan needs its two state entries of the cache")
        rows = request_rows_of(ctx)
        both = self.inputs.forward(x)
        u = self.conv.forward(both[:, :self.inner], ctx, cache.members[1])
        picked = self.selectors.forward(u)
        low = picked[:, :self.rank]
        step = self.step.forward(low if low.is_contiguous() else low.contiguous(), out_dtype=torch.float32)
        mixed = ops.selective_scan(
            u, step, self.step_bias, self.decay, picked[:, self.rank:self.rank + self.states],
            picked[:, self.rank + self.states:], self.skip, both[:, self.inner:], cache.members[0].state,
            rows["row_start"], rows["row_length"], ctx.request_slots, longest=rows.get("longest", 0))
        return self.o.forward(mixed)

    def weight_bytes(self) -> int:
        return (self.inputs.weight_bytes() + self.selectors.weight_bytes() + self.step.weight_bytes()
                + self.o.weight_bytes() + self.decay.numel() * 4)


register_part("mixer", "selective_scan", lambda spec, weights, runtime: SelectiveScan(spec, weights, runtime))


class ChannelDelta:
    """The gated delta rule with one decay per head and key channel. With H
    heads over G groups of queries and keys (head h reads group h // (H / G)),
    key width D and value width V:

        [q | k | v] = conv(a [Wq; Wk; Wv]^T), then silu      a short causal convolution per channel
        qn = q / sqrt(sum q^2 + 1e-6) * D^-1/2,  kn = k / sqrt(sum k^2 + 1e-6)       per head
        beta = sigmoid(a Wb^T)                               one per head
        g = exp(-exp(A_log_h) * softplus((a Wa1^T) Wa2^T + dt_bias))   [H, D], rows of S
        S <- g S;  u = beta (v - S^T kn);  S <- S + kn u^T;  o = S^T qn                per head

    Each head's o over its root mean square times a weight over V (shared by
    the heads) times sigmoid((a Wg1^T) Wg2^T), then Wo. S (float32, kept
    transposed as ``[H, V, D]``) and the convolution's last inputs are kept per request in
    the cache's state slots. One product gives q, k, v, both low-rank inputs
    and the write strength's pre-activation; the step size's second product
    leaves in float32; unit norms, softplus, decay, sigmoid, the recurrence and
    the head norm are float32 in both precisions; the projections, the
    convolution and its activation hand on the compute type."""

    kind = "channel_delta"
    graph_safe = True
    step_key = "request_rows"
    prepare_step = staticmethod(request_rows)

    def __init__(self, spec: PartSpec, weights: WeightStore, runtime: Runtime):
        from .short_conv import ShortConv
        hidden = spec["hidden_size"]
        self.heads, self.groups = int(spec["num_heads"]), int(spec.get("num_kv_heads") or spec["num_heads"])
        self.dim, self.vdim, self.eps = int(spec["head_dim"]), int(spec["value_dim"]), float(spec["eps"])
        if self.heads % self.groups:
            raise ValueError(f"{self.heads} heads cannot share {self.groups} groups of queries and keys")
        if not 0 < self.dim <= ops.delta_rule_max_dim():
            raise ValueError(f"keys of {self.dim} channels; the recurrence takes up to {ops.delta_rule_max_dim()}")
        H, G, D, V = self.heads, self.groups, self.dim, self.vdim

        def matrix(name, shape):
            weight = weights.take(spec[name])
            if tuple(weight.shape) != shape:
                raise ValueError(f"{spec[name]} is {tuple(weight.shape)}, expected {shape}")
            return weight

        def vector(name, size):
            tensor = weights.take(spec[name])
            if tensor.numel() != size:
                raise ValueError(f"{spec[name]} has {tensor.numel()} values, expected {size}")
            return tensor.to(device=runtime.device, dtype=torch.float32).reshape(-1).contiguous()

        # the two low ranks are sizes that only the checkpoint's tensors give
        step_rank, gate_rank = weights.shape(spec["step_down_proj"])[0], weights.shape(spec["gate_down_proj"])[0]
        self.conv_channels = 2 * G * D + H * V
        stacked, self.offsets, cursor = [], {}, 0
        for name, rows in (("q_proj", G * D), ("k_proj", G * D), ("v_proj", H * V), ("step_down_proj", step_rank),
                           ("gate_down_proj", gate_rank), ("beta_proj", H)):
            stacked.append(matrix(name, (rows, hidden)))
            self.offsets[name] = cursor
            cursor += rows
        self.inputs = Linear.stacked(stacked, runtime)     # rows: q, k, v, step latent, gate latent, write strength
        self.step_rank, self.gate_rank = step_rank, gate_rank
        self.step_up = Linear(matrix("step_up_proj", (H * D, step_rank)), runtime)
        self.gate_up = Linear(matrix("gate_up_proj", (H * V, gate_rank)), runtime)
        self.step_bias = vector("step_bias", H * D)
        self.rate = torch.exp(vector("a_log", H)).contiguous()
        self.norm_weight = vector("norm", V).repeat(H).contiguous()       # one weight over V, the same for every head
        taps = int(spec["conv_taps"])
        conv_weight = torch.cat([matrix(name, (rows, taps)) for name, rows in
                                 (("q_conv", G * D), ("k_conv", G * D), ("v_conv", H * V))], dim=0)
        store = WeightStore({"conv": conv_weight})
        self.conv = ShortConv(PartSpec("short_conv", {"channels": self.conv_channels, "taps": taps, "weight": "conv",
                                                      "bias": None, "activation": "silu"}), store, runtime)
        self.o = Linear(matrix("o_proj", (hidden, H * V)), runtime)
        self.dtype = runtime.dtype

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="several", members=(
            CacheNeed(kind="state", state_shape=(self.heads, self.vdim, self.dim), state_dtype="float32"),
            self.conv.cache_need()))

    def parts(self):
        return [self.conv]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        if len(cache.members) != 2 or cache.members[0].state is None:
            raise ValueError("the delta-rule mixer needs its two state entries of the cache")
        rows = request_rows_of(ctx)
        H, G, D, V, at = self.heads, self.groups, self.dim, self.vdim, self.offsets
        proj = self.inputs.forward(x)       # every later step reads column ranges of it in place
        qkv = self.conv.forward(proj[:, :self.conv_channels], ctx, cache.members[1])
        step = self.step_up.forward(proj[:, at["step_down_proj"]:at["step_down_proj"] + self.step_rank],
                                    out_dtype=torch.float32)
        mixed = ops.delta_rule(qkv, (0, G * D, 2 * G * D), proj[:, at["beta_proj"]:at["beta_proj"] + H], step,
                               self.step_bias, self.rate, cache.members[0].state, rows["row_start"],
                               rows["row_length"], ctx.request_slots, H, G, D, V, longest=rows.get("longest", 0))
        gate = self.gate_up.forward(proj[:, at["gate_down_proj"]:at["gate_down_proj"] + self.gate_rank])
        return self.o.forward(ops.head_norm_gate(mixed, self.norm_weight, gate, H, self.eps, self.dtype))

    def weight_bytes(self) -> int:
        return (self.inputs.weight_bytes() + self.step_up.weight_bytes() + self.gate_up.weight_bytes()
                + self.o.weight_bytes())


register_part("mixer", "channel_delta", lambda spec, weights, runtime: ChannelDelta(spec, weights, runtime))
