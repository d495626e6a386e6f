"""SwiGLU feed-forward: d = ((sigmoid(g) * g) * u) Wd^T with g = m Wg^T and
u = m Wu^T (crates/models/qwen/src/forward.rs:1904-1920). Gate and up weights
are stacked so that one product yields both; SiLU and the product with u are
float32 inside the kernel. ``activation="gelu_tanh"`` puts the tanh form of
gelu in SiLU's place, in every kernel that holds the activation.

``dense_ff`` is the feed-forward without a gate: d = act(m Wu^T) Wd^T, the
activation a parameter (``relu_squared``: max(z, 0)^2).

``routed_experts`` is a mixture of such feed-forwards: a router picks ``top``
of ``experts`` (+ ``identity`` outputs that stand for experts returning their
input) per token by softmax score plus a correction, and the output is the sum
of the chosen experts' outputs weighted by their scores over the chosen
scores' sum. Parameters widen it: ``scores="sigmoid"`` scores every output on
its own; ``groups`` = (count, keep) lets the choice fall only on the best
groups of neighbouring experts; ``scale`` multiplies the weights;
``activation="swiglu"`` makes an expert a gated feed-forward
down(silu(gate(h)) * up(h)); ``shared`` names a gated feed-forward that every
token uses, added behind a sigmoid gate of one number per token."""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .linear import Linear
from .registry import Runtime, StepContext, WeightStore, build_part, register_part

FUSED_ACTIVATION_ROWS = 1536   # from here on "auto" takes the tcgen05 product with the SwiGLU epilogue


class SwiGLU:
    kind = "swiglu"

    def __init__(self, spec: PartSpec, weights: WeightStore, runtime: Runtime):
        hidden, inter = spec["hidden_size"], spec["intermediate_size"]
        gate, up = weights.take(spec["gate_proj"]), weights.take(spec["up_proj"])
        down = weights.take(spec["down_proj"])
        for name, weight, shape in (("gate_proj", gate, (inter, hidden)), ("up_proj", up, (inter, hidden)),
                                    ("down_proj", down, (hidden, inter))):
            if tuple(weight.shape) != shape:
                raise ValueError(f"{spec[name]} is {tuple(weight.shape)}, expected {shape}")
        self.gate_up = Linear.stacked([gate, up], runtime)  # rows: gate, then up
        self.down = Linear(down, runtime)
        self.intermediate_size = inter
        self.activation = spec.get("activation") or "silu"
        if self.activation not in ops.GATE_ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r}; one of {sorted(ops.GATE_ACTIVATIONS)}")

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        few = ops.SKINNY_ROWS if x.shape[1] <= ops.STREAM_K else ops.SKINNY_ROWS // 2   # as ops.gemm_bf16
        if (x.shape[0] <= few and self.gate_up.backend in ("auto", "skinny")
                and ops.gemm_skinny_takes(x, self.gate_up.weight, swiglu=True)):
            # A decode step: gate, up and the activation in one pass over the weights.
            return self.down.forward(ops.gemm_skinny(x, self.gate_up.weight, swiglu=True, activation=self.activation))
        # From about 1,500 rows on the tcgen05 product with the activation in its
        # epilogue beats the library's product followed by an activation pass
        # (28 against 31 us at 2,048 rows of this model; 21 against 19 at 1,024,
        # 10 against 8 at 128): below that the library keeps the product, as in
        # the reference, unless the part is told to use the tcgen05 kernel.
        fused = self.gate_up.backend == "tcgen05" or (self.gate_up.backend == "auto"
                                                      and x.shape[0] >= FUSED_ACTIVATION_ROWS)
        if self.gate_up.dtype == torch.bfloat16 and fused:
            from .. import tensor_core
            if tensor_core.supports(x, self.gate_up.weight, torch.bfloat16):
                # gate, up and the activation in the product's epilogue
                return self.down.forward(tensor_core.gemm_swiglu(x, self.gate_up.weight, activation=self.activation))
        return self.down.forward(ops.silu_mul(self.gate_up.forward(x), activation=self.activation))

    def weight_bytes(self) -> int:
        return self.gate_up.weight_bytes() + self.down.weight_bytes()


register_part("feed_forward", "swiglu", lambda spec, weights, runtime: SwiGLU(spec, weights, runtime))


class DenseFeedForward:
    kind = "dense_ff"
    ACTIVATIONS = {"relu_squared": ops.relu_squared}

    def __init__(self, spec: PartSpec, weights: WeightStore, runtime: Runtime):
        hidden, inter = spec["hidden_size"], spec["intermediate_size"]
        up, down = weights.take(spec["up_proj"]), weights.take(spec["down_proj"])
        for name, weight, shape in (("up_proj", up, (inter, hidden)), ("down_proj", down, (hidden, inter))):
            if tuple(weight.shape) != shape:
                raise ValueError(f"{spec[name]} is {tuple(weight.shape)}, expected {shape}")
        if spec["activation"] not in self.ACTIVATIONS:
            raise ValueError(f"activation {spec['activation']!r}; one of {sorted(self.ACTIVATIONS)}")
        self.activation = self.ACTIVATIONS[spec["activation"]]
        self.up, self.down = Linear(up, runtime), Linear(down, runtime)
        self.intermediate_size = inter

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return self.down.forward(self.activation(self.up.forward(x)))

    def weight_bytes(self) -> int:
        return self.up.weight_bytes() + self.down.weight_bytes()


register_part("feed_forward", "dense_ff", lambda spec, weights, runtime: DenseFeedForward(spec, weights, runtime))


class RoutedExperts:
    """z = m Wr^T (float32); s = softmax(z) over all experts + identity
    outputs; the ``top`` largest s + correction are chosen; weights are the
    chosen s over their sum (+ 1e-20); d = sum_k weight_k expert_k(m), an
    expert being Wdown act(Wup m) or, for the last ``identity`` outputs, m
    itself. Steps of up to ``ROUTED_TOKENS`` tokens, and float32, go row by
    row through the chosen experts' weights; larger steps sort the (token,
    choice) pairs by expert and run two grouped tensor-core products over
    them, each tile of rows against its expert's matrices."""

    kind = "routed_experts"
    ROUTED_TOKENS = 1     # from two tokens on experts are shared often enough for the grouped products to read less
    ACTIVATIONS = ("relu_squared", "swiglu")

    def __init__(self, spec: PartSpec, weights: WeightStore, runtime: Runtime):
        hidden, ff = spec["hidden_size"], spec["intermediate_size"]
        self.experts, self.identity, self.top = int(spec["experts"]), int(spec.get("identity") or 0), int(spec["top"])
        outputs = self.experts + self.identity
        if not 0 < self.top <= outputs or outputs > ops.ROUTER_OUTPUTS:
            raise ValueError(f"top {self.top} of {outputs} router outputs (at most {ops.ROUTER_OUTPUTS}) cannot be chosen")
        if spec["activation"] not in self.ACTIVATIONS:
            raise ValueError(f"activation {spec['activation']!r}; one of {self.ACTIVATIONS}")
        self.gated = spec["activation"] == "swiglu"
        self.scores = spec.get("scores") or "softmax"
        self.groups = tuple(int(v) for v in spec["groups"]) if spec.get("groups") else None
        self.weight_scale = float(spec.get("scale") or 1.0)
        if self.scores not in ("softmax", "sigmoid"):
            raise ValueError(f"scores {self.scores!r}; 'softmax' or 'sigmoid'")
        if self.groups is not None:
            count, keep = self.groups
            if count < 1 or outputs % count or not 1 <= keep <= count or keep * (outputs // count) < self.top:
                raise ValueError(f"{count} groups of which {keep} are kept do not fit {outputs} outputs and top {self.top}")
        ups, downs = [], []
        for index in range(self.experts):
            up, down = weights.take(spec["up_proj"].format(index)), weights.take(spec["down_proj"].format(index))
            if tuple(up.shape) != (ff, hidden) or tuple(down.shape) != (hidden, ff):
                raise ValueError(f"expert {index}: up is {tuple(up.shape)}, down is {tuple(down.shape)}; "
                                 f"expected {(ff, hidden)} and {(hidden, ff)}")
            if self.gated:   # an expert's gate rows, then its up rows
                gate = weights.take(spec["gate_proj"].format(index))
                if tuple(gate.shape) != (ff, hidden):
                    raise ValueError(f"expert {index}: gate is {tuple(gate.shape)}, expected {(ff, hidden)}")
                ups.append(gate.to(runtime.device))
            ups.append(up.to(runtime.device))
            downs.append(down.to(runtime.device))
        # up: rows e * ff + f (gated: e * 2 ff + f for the gate, + ff for up); down: rows e * hidden + c:
        # one expert's matrix after the other
        self.up = Linear(torch.cat(ups, dim=0), runtime) if ups else None
        self.down = Linear(torch.cat(downs, dim=0), runtime) if downs else None
        router = weights.take(spec["router"])
        if tuple(router.shape) != (outputs, hidden):
            raise ValueError(f"{spec['router']} is {tuple(router.shape)}, expected {(outputs, hidden)}")
        self.outputs = outputs
        self.shared = None
        if spec.get("shared") is not None:
            # an expert for every token, out += sigmoid(h . w) shared(h): its gate's row rides under the router's
            self.shared = build_part("feed_forward", spec["shared"], weights, runtime)
            gate = weights.take(spec["shared_gate"])
            if gate.numel() != hidden:
                raise ValueError(f"{spec['shared_gate']} has {gate.numel()} values, expected {hidden}")
            router = torch.cat([router.to(runtime.device), gate.reshape(1, hidden).to(runtime.device)], dim=0)
        self.router = Linear(router, runtime)
        correction = weights.take(spec["correction"]) if spec.get("correction") else torch.zeros(outputs)
        if correction.numel() != outputs:
            raise ValueError(f"{spec['correction']} has {correction.numel()} values, expected {outputs}")
        self.correction = correction.to(device=runtime.device, dtype=torch.float32).reshape(-1).contiguous()
        self.hidden_size, self.intermediate_size = hidden, ff

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """float32 ``[tokens, hidden]``."""
        logits = self.router.forward(x, out_dtype=torch.float32)
        out = self._routed(x, logits[:, :self.outputs])
        if self.shared is not None:
            ops.add_gated_rows(out, self.shared.forward(x, ctx), logits[:, self.outputs:])
        return out

    def _routed(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        chosen, weights, dense, on_identity = ops.route_experts(logits, self.correction, self.experts, self.top,
                                                                scores=self.scores, groups=self.groups,
                                                                scale=self.weight_scale)
        if self.up is None:     # identity experts only
            return ops.experts_add_identity(torch.zeros(x.shape, dtype=torch.float32, device=x.device), x, on_identity)
        if x.shape[0] > self.ROUTED_TOKENS and self.grouped(x):
            from .. import tensor_core
            position, tile_group, rows = ops.expert_rows(chosen, self.experts)
            act = tensor_core.gemm_grouped(ops.expert_gather_rows(x, position, rows), self.up.weight, tile_group,
                                           self.experts, tensor_core.SWIGLU if self.gated else tensor_core.RELU_SQUARED)
            out = tensor_core.gemm_grouped(act, self.down.weight, tile_group, self.experts, tensor_core.STORE_F32)
            return ops.expert_combine_rows(out, position, weights, on_identity, x)
        return ops.experts_routed(x, self.up.weight, self.down.weight, chosen, weights, self.experts,
                                  self.intermediate_size, gated=self.gated)

    def grouped(self, x: torch.Tensor) -> bool:
        """Whether the grouped tensor-core products take this step."""
        from .. import tensor_core
        return (self.intermediate_size % 8 == 0 and self.down.weight.data_ptr() % 16 == 0
                and tensor_core.supports(x, self.up.weight, torch.bfloat16))

    def weight_bytes(self) -> int:
        """What a decode step of one token reads: the router and ``top`` experts."""
        per_expert = (self.up.weight_bytes() + self.down.weight_bytes()) // self.experts if self.up is not None else 0
        shared = self.shared.weight_bytes() if self.shared is not None else 0
        return self.router.weight_bytes() + min(self.top, self.experts) * per_expert + shared


register_part("feed_forward", "routed_experts", lambda spec, weights, runtime: RoutedExperts(spec, weights, runtime))
