"""Typed configuration of the Sadosun decoder, read from ``config.json``.

A Sadosun model is a stack of pre-norm layers over one float32 residual
stream that starts as ``embed[token] * embedding.scale``. Its norms are RMS
norms whose weight is a single number. In every layer

* what a sublayer reads passes a short causal convolution over time first,
  h <- h + conv(h) (``canon.taps`` taps per channel, no bias; the last
  ``taps - 1`` inputs belong to a request's state);
* the mixer is one of

  - ``attention``: grouped-query attention; q and k are rotated (neighbouring
    pairs (2i, 2i + 1) over the first ``rot.dims`` values of a head, angle
    p * base^(-2i / dims)) and then divided by their root mean square per head;
    the value of position j is turned by j over its whole width in the same
    pairing (pair m by j * base^(-2m / vdim)), cached so, and every head's
    output at position i is turned back by i; a sliding window of
    ``mask.size`` positions (the query's own included); a softmax whose
    denominator is one larger than the sum (a sink with score 0 and no value);
    the score scale is the configuration's;
  - ``mamba1``: the selective state-space mixer: one projection gives x and z,
    x passes a causal convolution of ``conv`` taps with bias and silu, a
    second projection gives a low-rank step size (``dt_rank``), B and C, the
    step size is softplus(dt Wdt^T + b), A = -exp(A_log), the state
    ``[inner, state]`` is float32 and is carried from token to token, the
    result is y * silu(z), projected;

* the feed-forward (unless ``mlp`` is null) is a mixture of ``experts``
  feed-forwards down(relu(up(h))^2) of which a token uses ``top``: scores are
  the softmax of the router's float32 logits over ``experts + identity``
  outputs, the choice goes by score plus a stored correction, the weights are
  the chosen scores over their sum, and the last ``identity`` outputs stand
  for experts that return h itself;
* at the end the layer takes an input from the token: with e = the layer's
  ``token_side.dim`` columns of ``side.embed[token]``,
  x <- x + rmsnorm(proj(gelu_tanh(gate(x)) * e)) * side.norm.

``config.json``::

    {"architecture": "Sadosun", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "canon": {"taps": K}, "token_side": {"dim": S},
     "layers": [{"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": c, "mask": {"size": w},
                           "rot": {"base": b, "dims": R}},
                 "mlp": {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "identity": I, "top": k}}},
                {"type": "mamba1", "mixer": {"inner": N, "state": n, "dt_rank": r, "conv": K2}, "mlp": null}]}

``canon``, ``token_side``, ``embedding``, a layer's ``mask``, ``rot`` and
``kv_heads`` may be absent: the model is then built without that mechanism
(one key/value head per query head).

Tensors (linear weights ``[out, in]``): ``embed`` [V, W], ``side.embed``
[V, layers * S], ``final.norm`` [], ``head`` [V, W]; per layer i ``l<i>.norm1``,
``norm2`` [], ``l<i>.canon1``, ``canon2`` [W, K], ``l<i>.side.gate`` [S, W],
``.side.proj`` [W, S], ``.side.norm`` [W]; under ``l<i>.mix`` an attention has
``q`` [H D, W], ``k`` [G D, W], ``v`` [G Dv, W], ``o`` [W, H Dv]; a mamba1 has
``in`` [2N, W], ``conv`` [N, K2], ``conv.b`` [N], ``x`` [r + 2n, N], ``dt``
[N, r], ``dt.b`` [N], ``A_log`` [N, n], ``D`` [N], ``o`` [W, N]; under
``l<i>.mlp``: ``e<j>.up`` [F, W], ``e<j>.down`` [W, F], ``router`` [E + I, W],
``correction`` [E + I].
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .mekazen import MAX_POSITIONS, _count, _number, _object
from .qwen3 import ConfigError
from .spec import LayerRun, LayerSpec, ModelSpec, PartSpec


def _positive(raw: Mapping[str, Any], key: str, where: str) -> float:
    value = _number(raw, key, where)
    if value <= 0.0:
        raise ConfigError("Json", f"{where}.{key} must be positive, got {value}")
    return value


@dataclass(frozen=True)
class WindowedAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int            # 0: every earlier position is seen
    rotary_dims: int       # 0: no rotation, of q and k or of the values
    rotary_base: float

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "WindowedAttention":
        raw = _object(raw, where)
        heads, dim = _count(raw, "heads", where), _count(raw, "dim", where)
        kv_heads = _count(raw, "kv_heads", where) if raw.get("kv_heads") is not None else heads
        if heads % kv_heads:
            raise ConfigError("InvalidGroupedQueryLayout", f"{where}: {heads} query heads over {kv_heads} key/value heads")
        vdim = _count(raw, "vdim", where) if raw.get("vdim") is not None else dim
        window = 0
        if raw.get("mask") is not None:
            window = _count(_object(raw["mask"], f"{where}.mask"), "size", f"{where}.mask")
        dims, base = 0, 0.0
        if raw.get("rot") is not None:
            rot = _object(raw["rot"], f"{where}.rot")
            dims, base = _count(rot, "dims", f"{where}.rot"), _positive(rot, "base", f"{where}.rot")
            if dims % 2 or dims > dim:
                raise ConfigError("InvalidRotaryWidth", f"{where}.rot.dims {dims} must be even and at most {dim}")
            if vdim % 2:
                raise ConfigError("InvalidRotaryWidth", f"{where}.vdim {vdim} must be even for its values to be turned")
        return cls(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=_positive(raw, "scale", where),
                   window=window, rotary_dims=dims, rotary_base=base)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads}
        if self.window:
            out["mask"] = {"size": self.window}
        if self.rotary_dims:
            out["rot"] = {"base": self.rotary_base, "dims": self.rotary_dims}
        out.update(scale=self.scale, vdim=self.vdim)
        return out

    def shapes(self, base: str, w: int) -> Dict[str, tuple]:
        return {f"{base}.q": (self.heads * self.dim, w), f"{base}.k": (self.kv_heads * self.dim, w),
                f"{base}.v": (self.kv_heads * self.vdim, w), f"{base}.o": (w, self.heads * self.vdim)}

    def part(self, base: str, w: int, eps: float) -> PartSpec:
        position = value_position = None
        if self.rotary_dims:
            position = PartSpec("rope_interleaved", {"theta": self.rotary_base, "rotary_dim": self.rotary_dims,
                                                     "head_dim": self.dim, "scaling": None})
            value_position = PartSpec("rope_interleaved", {"theta": self.rotary_base, "rotary_dim": self.vdim,
                                                           "head_dim": self.vdim, "scaling": None})
        # A rotation keeps a head's sum of squares, so the division by the root mean square
        # may come first: the fused kernel's order.
        unit = PartSpec("rmsnorm", {"size": self.dim, "eps": eps, "weight": None})
        return PartSpec("gqa_attention", {
            "hidden_size": w, "num_heads": self.heads, "num_kv_heads": self.kv_heads, "head_dim": self.dim,
            "value_dim": self.vdim, "scale": self.scale, "softcap": None, "window": self.window or None,
            "chunk": None, "q_proj": f"{base}.q", "k_proj": f"{base}.k", "v_proj": f"{base}.v", "gate_proj": None,
            "o_proj": f"{base}.o", "qk_norm_scope": "head", "q_norm": unit, "k_norm": unit, "position": position,
            "value_position": value_position, "sink": 0.0})


@dataclass(frozen=True)
class SelectiveMixer:
    inner: int
    state: int
    dt_rank: int
    conv: int

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "SelectiveMixer":
        raw = _object(raw, where)
        return cls(inner=_count(raw, "inner", where), state=_count(raw, "state", where),
                   dt_rank=_count(raw, "dt_rank", where), conv=_count(raw, "conv", where))

    def to_dict(self) -> Dict[str, Any]:
        return {"conv": self.conv, "dt_rank": self.dt_rank, "inner": self.inner, "state": self.state}

    def shapes(self, base: str, w: int) -> Dict[str, tuple]:
        n = self.inner
        return {f"{base}.in": (2 * n, w), f"{base}.conv": (n, self.conv), f"{base}.conv.b": (n,),
                f"{base}.x": (self.dt_rank + 2 * self.state, n), f"{base}.dt": (n, self.dt_rank),
                f"{base}.dt.b": (n,), f"{base}.A_log": (n, self.state), f"{base}.D": (n,), f"{base}.o": (w, n)}

    def part(self, base: str, w: int, eps: float) -> PartSpec:
        return PartSpec("selective_scan", {
            "hidden_size": w, "inner_size": self.inner, "state_size": self.state, "step_rank": self.dt_rank,
            "conv_taps": self.conv, "in_proj": f"{base}.in", "conv_weight": f"{base}.conv",
            "conv_bias": f"{base}.conv.b", "x_proj": f"{base}.x", "step_proj": f"{base}.dt",
            "step_bias": f"{base}.dt.b", "a_log": f"{base}.A_log", "skip": f"{base}.D", "o_proj": f"{base}.o"})


_MIXERS = {"attention": WindowedAttention, "mamba1": SelectiveMixer}


@dataclass(frozen=True)
class ExpertMixture:
    ff: int
    experts: int
    identity: int
    top: int

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "ExpertMixture":
        raw = _object(raw, where)
        if raw.get("kind") != "moe":
            raise ConfigError("UnsupportedFeedForward", f"{where}.kind {raw.get('kind')!r}; 'moe' only")
        router = _object(raw.get("router"), f"{where}.router")
        identity = router.get("identity") or 0
        if isinstance(identity, bool) or not isinstance(identity, int) or identity < 0:
            raise ConfigError("Json", f"{where}.router.identity must be a count, got {identity!r}")
        experts, top = _count(router, "experts", f"{where}.router"), _count(router, "top", f"{where}.router")
        if top > experts + identity:
            raise ConfigError("Json", f"{where}.router: top {top} of {experts + identity} outputs")
        return cls(ff=_count(_object(raw.get("expert"), f"{where}.expert"), "ff", f"{where}.expert"),
                   experts=experts, identity=identity, top=top)

    def to_dict(self) -> Dict[str, Any]:
        return {"expert": {"ff": self.ff}, "kind": "moe",
                "router": {"experts": self.experts, "identity": self.identity, "top": self.top}}

    def shapes(self, base: str, w: int) -> Dict[str, tuple]:
        shapes: Dict[str, tuple] = {}
        for index in range(self.experts):
            shapes[f"{base}.e{index}.up"] = (self.ff, w)
            shapes[f"{base}.e{index}.down"] = (w, self.ff)
        outputs = self.experts + self.identity
        shapes.update({f"{base}.router": (outputs, w), f"{base}.correction": (outputs,)})
        return shapes

    def part(self, base: str, w: int) -> PartSpec:
        return PartSpec("routed_experts", {
            "hidden_size": w, "intermediate_size": self.ff, "experts": self.experts, "identity": self.identity,
            "top": self.top, "activation": "relu_squared", "up_proj": base + ".e{}.up", "down_proj": base + ".e{}.down",
            "router": f"{base}.router", "correction": f"{base}.correction"})


@dataclass(frozen=True)
class SadosunLayer:
    kind: str                          # "attention" or "mamba1"
    mixer: object
    mlp: Optional[ExpertMixture]       # None: no feed-forward

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "SadosunLayer":
        raw = _object(raw, where)
        kind = raw.get("type")
        if kind not in _MIXERS:
            raise ConfigError("UnsupportedLayerType", f"{where}.type {kind!r}; this design has {sorted(_MIXERS)}")
        mlp = ExpertMixture.from_dict(raw["mlp"], f"{where}.mlp") if raw.get("mlp") is not None else None
        return cls(kind=kind, mixer=_MIXERS[kind].from_dict(raw.get("mixer"), f"{where}.mixer"), mlp=mlp)

    def to_dict(self) -> Dict[str, Any]:
        return {"mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp is not None else None,
                "type": self.kind}


@dataclass(frozen=True)
class SadosunConfig:
    """Sizes and constants of one Sadosun checkpoint."""

    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[SadosunLayer, ...]
    embedding_scale: float = 1.0
    canon_taps: int = 0          # 0: sublayers read their norm's output as it is
    side_dim: int = 0            # 0: no per-layer input from the token
    eos_token_ids: tuple = ()

    ARCHITECTURE = "Sadosun"
    MODEL_TYPE = "sadosun"

    @classmethod
    def parse(cls, text: str) -> "SadosunConfig":
        try:
            raw = json.loads(text)
        except json.JSONDecodeError as error:
            raise ConfigError("Json", str(error)) from None
        return cls.from_dict(_object(raw, "config.json"))

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "SadosunConfig":
        if raw.get("architecture") != cls.ARCHITECTURE:
            raise ConfigError("UnsupportedModelType", f"architecture {raw.get('architecture')!r}")
        vocab, width = _count(raw, "vocab", "config"), _count(raw, "width", "config")
        eps = _number(_object(raw.get("norm"), "norm"), "eps", "norm")
        if eps <= 0.0:
            raise ConfigError("InvalidRmsNormEpsilon", str(eps))
        scale = 1.0
        if raw.get("embedding") is not None:
            scale = _number(_object(raw["embedding"], "embedding"), "scale", "embedding")
        taps = _count(_object(raw["canon"], "canon"), "taps", "canon") if raw.get("canon") is not None else 0
        side = _count(_object(raw["token_side"], "token_side"), "dim", "token_side") \
            if raw.get("token_side") is not None else 0
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("MissingDimension", "layers must be a list of at least one layer")
        return cls(vocab=vocab, width=width, norm_eps=eps, embedding_scale=scale, canon_taps=taps, side_dim=side,
                   layers=tuple(SadosunLayer.from_dict(layer, f"layers[{i}]") for i, layer in enumerate(layers)))

    # ------------------------------------------------------------ derived facts
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def parameter_count(self) -> int:
        return sum(math.prod(shape) for shape in self.tensor_shapes().values())

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.ARCHITECTURE}
        if self.canon_taps:
            out["canon"] = {"taps": self.canon_taps}
        out["embedding"] = {"scale": self.embedding_scale}
        out["layers"] = [layer.to_dict() for layer in self.layers]
        out["norm"] = {"eps": self.norm_eps}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        out.update(vocab=self.vocab, width=self.width)
        return out

    # ------------------------------------------------------------- model spec
    def to_model_spec(self) -> ModelSpec:
        w, eps = self.width, self.norm_eps
        norm = lambda name: PartSpec("rmsnorm", {"size": w, "eps": eps, "weight": name, "scalar": True})
        conv = lambda name: PartSpec("short_conv", {"channels": w, "taps": self.canon_taps, "weight": name,
                                                    "bias": None, "residual": True}) if self.canon_taps else None
        layers = []
        for index, layer in enumerate(self.layers):
            base = f"l{index}"
            block: Dict[str, Any] = {"hidden_size": w, "mixer_conv": conv(f"{base}.canon1"),
                                     "feed_forward_conv": conv(f"{base}.canon2") if layer.mlp is not None else None,
                                     "token_input": None}
            if self.side_dim:
                block["token_input"] = PartSpec("token_input", {
                    "hidden_size": w, "dim": self.side_dim, "offset": index * self.side_dim, "table": "side.embed",
                    "gate_proj": f"{base}.side.gate", "out_proj": f"{base}.side.proj",
                    "norm": PartSpec("rmsnorm", {"size": w, "eps": eps, "weight": f"{base}.side.norm"})})
            layers.append(LayerSpec(
                name=base, block=PartSpec("conv_prenorm_residual", block), mixer=layer.mixer.part(f"{base}.mix", w, eps),
                feed_forward=layer.mlp.part(f"{base}.mlp", w) if layer.mlp is not None else None,
                mixer_norm=norm(f"{base}.norm1"),
                feed_forward_norm=norm(f"{base}.norm2") if layer.mlp is not None else None))
        spec = ModelSpec(
            architecture=self.ARCHITECTURE, hidden_size=w, vocab_size=self.vocab, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": w, "weight": "embed",
                                                   "scale": self.embedding_scale}),
            layers=tuple(layers), order=tuple(LayerRun(layer=index) for index in range(len(layers))),
            final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": w, "weight": "head",
                                          "softcap": None}))
        spec.validate()
        return spec

    # ------------------------------------------------ tensors of a checkpoint
    def tensor_shapes(self) -> Dict[str, tuple]:
        w = self.width
        shapes: Dict[str, tuple] = {"embed": (self.vocab, w)}
        if self.side_dim:
            shapes["side.embed"] = (self.vocab, len(self.layers) * self.side_dim)
        for index, layer in enumerate(self.layers):
            base = f"l{index}"
            shapes[f"{base}.norm1"] = ()
            if layer.mlp is not None:
                shapes[f"{base}.norm2"] = ()
            shapes.update(layer.mixer.shapes(f"{base}.mix", w))
            if layer.mlp is not None:
                shapes.update(layer.mlp.shapes(f"{base}.mlp", w))
            if self.canon_taps:
                shapes[f"{base}.canon1"] = (w, self.canon_taps)
                if layer.mlp is not None:
                    shapes[f"{base}.canon2"] = (w, self.canon_taps)
            if self.side_dim:
                shapes.update({f"{base}.side.gate": (self.side_dim, w), f"{base}.side.proj": (w, self.side_dim),
                               f"{base}.side.norm": (w,)})
        shapes["final.norm"] = ()
        shapes["head"] = (self.vocab, w)
        return shapes

    def ignored_tensors(self) -> tuple:
        """The second sublayer's norm and convolution of a layer without a
        feed-forward, should a checkpoint hold them all the same."""
        names = []
        for index, layer in enumerate(self.layers):
            if layer.mlp is None:
                names += [f"l{index}.norm2", f"l{index}.canon2"]
        return tuple(names)

    def norm_tensor(self, name: str):
        """How a tensor of random weights is drawn: False for a matrix
        (N(0, 0.02)); "one" for a factor near 1; "zero" for an offset near 0."""
        last = name.rsplit(".", 1)[-1]
        if last == "b":
            return "zero"
        if last in ("norm1", "norm2", "norm", "D"):
            return "one"
        return False
