"""Typed configuration of the Dimorax decoder, read from ``config.json``.

A Dimorax model is a stack of layers over one float32 residual stream that
starts as ``embed[token]``. Both sublayers of a layer read the same input:

    x <- x + m * (mixer(norm1(x)) + ff(norm2(x)))          m = ``residual_mult``

with RMS norms whose stored weight lies around zero (the factor is 1 + w); a
layer may have no feed-forward. The mixer is one of

* ``channel_delta``: the gated delta rule. q and k (``kv_heads`` groups of
  ``dim``) and v (``heads`` of ``vdim``) each pass a short causal convolution
  over time (``conv`` taps per channel, no bias) and silu; q and k become unit
  vectors per head, q times dim^-1/2; the write strength is sigmoid(Wb a), one
  per head; one decay per head and key channel,
  g = exp(-exp(A_log) softplus(Wa2 (Wa1 a) + dt_bias)); per head
  S <- g S (rows), u = beta (v - S^T k), S <- S + k u^T, o = S^T q; each head's
  o over its root mean square, times a weight over vdim, times
  sigmoid(Wg2 (Wg1 a)), then Wo. S and the convolution's last inputs are state
  of a request;
* ``attention``: grouped-query attention whose q, k and v projections have
  biases; halves of the first ``rot.dims`` values of a head are rotated
  (``rot.scaling``, optional: factor, original, fast, slow); the score scale
  is the configuration's, scores pass softcap * tanh(score / softcap)
  (optional), the mask is causal (``mask.size``, optional: a sliding window),
  and the softmax's denominator also holds exp(sink) of a learned number per
  head. With ``kv_from`` = j the layer has no key and value projections and
  reads what layer j cached, with its own queries;
* ``latent_attention``: q straight from the input, per head [``dim``
  unrotated | ``rot_dim`` rotated]; a down-projection gives ``kv_rank`` values
  that are RMS-normed (the latent) and ``rot_dim`` values that are rotated
  (one key part for all heads); per head the unrotated key and the value are
  up-projections of the latent; a sliding window of ``mask.size`` positions
  (optional), a learned sink per head.

The feed-forward is ``dense``, Wdown (gelu_tanh(Wgate h) * (Wup h)), or ``moe``:
``router.experts`` experts Wdown (silu(Wgate h) * (Wup h)) of which a token
uses ``router.top``; scores are sigmoids of the router's float32 logits; the
choice goes by score plus a stored correction, within the ``groups.keep`` best
of ``groups.count`` equal groups of neighbouring experts (a group's score: the
sum of its two largest corrected scores); the weights are the chosen scores
over their sum, times ``router.scale``; a shared expert (``shared.ff``, the
same form) is added for every token, times sigmoid(Wsg h).

``config.json``::

    {"architecture": "Dimorax", "vocab": V, "width": W, "norm": {"eps": e}, "residual_mult": m,
     "layers": [{"type": "channel_delta", "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "conv": K},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": c, "softcap": s,
                           "rot": {"base": b, "dims": R, "scaling": {"factor": f, "original": n, "fast": x, "slow": y}}},
                 "mlp": {"kind": "moe", "expert": {"ff": F}, "shared": {"ff": Fs},
                         "router": {"experts": E, "top": k, "scale": a, "groups": {"count": n, "keep": j}}}},
                {"type": "latent_attention",
                 "mixer": {"heads": H, "dim": D, "rot_dim": R, "vdim": Dv, "kv_rank": r, "scale": c,
                           "mask": {"size": w}, "rot": {"base": b, "dims": R}}, "mlp": null}]}

Tensors (linear weights ``[out, in]``): ``embed`` [V, W], ``final.norm`` [W],
``head`` [V, W]; per layer i ``l<i>.norm1`` and (with a feed-forward)
``norm2`` [W]; under ``l<i>.mix`` a channel_delta has ``q``, ``k`` [G D, W],
``v`` [H Dv, W], ``q.conv``, ``k.conv``, ``v.conv`` [channels, K], ``b`` [H, W],
``A_log`` [H], ``a1`` [ra, W], ``a2`` [H D, ra], ``dt_bias`` [H D], ``g1`` [rg, W],
``g2`` [H Dv, rg], ``norm`` [Dv], ``o`` [W, H Dv] (the two low ranks ra and rg
are the tensors' own; ``ranks`` in the mixer's configuration names them where
a model is made, not read); an attention has ``q`` [H D, W], ``q.b``, ``sink``
[H], ``o`` [W, H Dv] and, without ``kv_from``, ``k`` [G D, W], ``k.b``, ``v``
[G Dv, W], ``v.b``; a latent_attention has ``q`` [H (D + R), W], ``dkv``
[r + R, W], ``dkv.norm`` [r], ``uk`` [H D, r], ``uv`` [H Dv, r], ``sink`` [H],
``o`` [W, H Dv]. Under ``l<i>.mlp`` a dense feed-forward has ``gate``, ``up``
[F, W], ``down`` [W, F]; a moe has ``e<j>.gate``, ``e<j>.up`` [F, W],
``e<j>.down`` [W, F], ``router`` [E, W], ``correction`` [E] and, with a shared
expert, ``shared.gate``, ``shared.up`` [Fs, W], ``shared.down`` [W, Fs],
``shared.sg`` [1, W].
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .mekazen import MAX_POSITIONS, _count, _number, _object
from .qwen3 import ConfigError
from .sadosun import _positive
from .spec import LayerRun, LayerSpec, ModelSpec, PartSpec


def _window(raw: Mapping[str, Any], where: str) -> int:
    if raw.get("mask") is None:
        return 0
    return _count(_object(raw["mask"], f"{where}.mask"), "size", f"{where}.mask")


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int
    scaling: Optional[Tuple[Tuple[str, float], ...]] = None     # (factor, original, fast, slow) by name

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str, width: int) -> "Rotation":
        raw = _object(raw, where)
        dims, base = _count(raw, "dims", where), _positive(raw, "base", where)
        if dims % 2 or dims > width:
            raise ConfigError("InvalidRotaryWidth", f"{where}.dims {dims} must be even and at most {width}")
        scaling = None
        if raw.get("scaling") is not None:
            given = _object(raw["scaling"], f"{where}.scaling")
            if base <= 1.0:
                raise ConfigError("Json", f"{where}.base must exceed 1 for its wavelengths to be stretched")
            scaling = tuple((key, _positive(given, key, f"{where}.scaling"))
                            for key in ("factor", "original", "fast", "slow"))
        return cls(base=base, dims=dims, scaling=scaling)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = dict(self.scaling)
        return out

    def part(self, head_dim: int) -> PartSpec:
        return PartSpec("rope_half", {"theta": self.base, "rotary_dim": self.dims, "head_dim": head_dim,
                                      "scaling": dict(self.scaling) if self.scaling is not None else None})


@dataclass(frozen=True)
class ChannelDeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: Optional[int] = None      # None: whatever the checkpoint's tensors have
    gate_rank: Optional[int] = None

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "ChannelDeltaMixer":
        raw = _object(raw, where)
        heads, dim = _count(raw, "heads", where), _count(raw, "dim", where)
        kv_heads = _count(raw, "kv_heads", where) if raw.get("kv_heads") is not None else heads
        if heads % kv_heads:
            raise ConfigError("InvalidGroupedQueryLayout", f"{where}: {heads} heads over {kv_heads} query/key heads")
        decay_rank = gate_rank = None
        if raw.get("ranks") is not None:
            ranks = _object(raw["ranks"], f"{where}.ranks")
            decay_rank, gate_rank = _count(ranks, "decay", f"{where}.ranks"), _count(ranks, "gate", f"{where}.ranks")
        return cls(heads=heads, kv_heads=kv_heads, dim=dim,
                   vdim=_count(raw, "vdim", where) if raw.get("vdim") is not None else dim,
                   conv=_count(raw, "conv", where), decay_rank=decay_rank, gate_rank=gate_rank)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads}
        if self.decay_rank is not None and self.gate_rank is not None:
            out["ranks"] = {"decay": self.decay_rank, "gate": self.gate_rank}
        out["vdim"] = self.vdim
        return out

    def shapes(self, base: str, w: int) -> Dict[str, tuple]:
        qk, v = self.kv_heads * self.dim, self.heads * self.vdim
        return {f"{base}.q": (qk, w), f"{base}.q.conv": (qk, self.conv), f"{base}.k": (qk, w),
                f"{base}.k.conv": (qk, self.conv), f"{base}.v": (v, w), f"{base}.v.conv": (v, self.conv),
                f"{base}.b": (self.heads, w), f"{base}.A_log": (self.heads,), f"{base}.norm": (self.vdim,),
                f"{base}.a1": (self.decay_rank, w), f"{base}.a2": (self.heads * self.dim, self.decay_rank),
                f"{base}.dt_bias": (self.heads * self.dim,), f"{base}.g1": (self.gate_rank, w),
                f"{base}.g2": (v, self.gate_rank), f"{base}.o": (w, v)}

    def part(self, base: str, w: int, eps: float) -> PartSpec:
        return PartSpec("channel_delta", {
            "hidden_size": w, "num_heads": self.heads, "num_kv_heads": self.kv_heads, "head_dim": self.dim,
            "value_dim": self.vdim, "conv_taps": self.conv, "eps": eps, "q_proj": f"{base}.q", "k_proj": f"{base}.k",
            "v_proj": f"{base}.v", "q_conv": f"{base}.q.conv", "k_conv": f"{base}.k.conv", "v_conv": f"{base}.v.conv",
            "beta_proj": f"{base}.b", "a_log": f"{base}.A_log", "step_down_proj": f"{base}.a1",
            "step_up_proj": f"{base}.a2", "step_bias": f"{base}.dt_bias", "gate_down_proj": f"{base}.g1",
            "gate_up_proj": f"{base}.g2", "norm": f"{base}.norm", "o_proj": f"{base}.o"})


@dataclass(frozen=True)
class BiasedAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float                  # 0: scores are not capped
    window: int                     # 0: every earlier position is seen
    rot: Optional[Rotation]
    kv_from: Optional[int]          # the layer whose cached keys and values this one reads

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "BiasedAttention":
        raw = _object(raw, where)
        heads, dim = _count(raw, "heads", where), _count(raw, "dim", where)
        kv_heads = _count(raw, "kv_heads", where) if raw.get("kv_heads") is not None else heads
        if heads % kv_heads:
            raise ConfigError("InvalidGroupedQueryLayout", f"{where}: {heads} query heads over {kv_heads} key/value heads")
        softcap = _positive(raw, "softcap", where) if raw.get("softcap") is not None else 0.0
        kv_from = raw.get("kv_from")
        if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int) or kv_from < 0):
            raise ConfigError("Json", f"{where}.kv_from must be a layer's index, got {kv_from!r}")
        return cls(heads=heads, kv_heads=kv_heads, dim=dim,
                   vdim=_count(raw, "vdim", where) if raw.get("vdim") is not None else dim,
                   scale=_positive(raw, "scale", where), softcap=softcap, window=_window(raw, where),
                   rot=Rotation.from_dict(raw["rot"], f"{where}.rot", dim) if raw.get("rot") is not None else None,
                   kv_from=kv_from)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"dim": self.dim, "heads": self.heads}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        out["kv_heads"] = self.kv_heads
        if self.window:
            out["mask"] = {"size": self.window}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        out["scale"] = self.scale
        if self.softcap:
            out["softcap"] = self.softcap
        out["vdim"] = self.vdim
        return out

    def shapes(self, base: str, w: int) -> Dict[str, tuple]:
        q = self.heads * self.dim
        shapes = {f"{base}.q": (q, w), f"{base}.q.b": (q,)}
        if self.kv_from is None:
            k, v = self.kv_heads * self.dim, self.kv_heads * self.vdim
            shapes.update({f"{base}.k": (k, w), f"{base}.k.b": (k,), f"{base}.v": (v, w), f"{base}.v.b": (v,)})
        shapes.update({f"{base}.sink": (self.heads,), f"{base}.o": (w, self.heads * self.vdim)})
        return shapes

    def part(self, base: str, w: int, eps: float) -> PartSpec:
        own = self.kv_from is None
        return PartSpec("gqa_attention", {
            "hidden_size": w, "num_heads": self.heads, "num_kv_heads": self.kv_heads, "head_dim": self.dim,
            "value_dim": self.vdim, "scale": self.scale, "softcap": self.softcap or None, "window": self.window or None,
            "chunk": None, "q_proj": f"{base}.q", "k_proj": f"{base}.k" if own else None,
            "v_proj": f"{base}.v" if own else None, "gate_proj": None, "o_proj": f"{base}.o",
            "q_bias": f"{base}.q.b", "k_bias": f"{base}.k.b" if own else None, "v_bias": f"{base}.v.b" if own else None,
            "shared_kv": not own, "qk_norm_scope": "head", "q_norm": None, "k_norm": None,
            "position": self.rot.part(self.dim) if self.rot is not None else None, "value_position": None,
            "sink": f"{base}.sink"})


@dataclass(frozen=True)
class WindowedLatentAttention:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: int
    rot: Optional[Rotation]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "WindowedLatentAttention":
        raw = _object(raw, where)
        rot_dim = _count(raw, "rot_dim", where)
        rot = Rotation.from_dict(raw["rot"], f"{where}.rot", rot_dim) if raw.get("rot") is not None else None
        if rot is not None and rot.dims != rot_dim:
            raise ConfigError("InvalidRotaryWidth", f"{where}: rot.dims {rot.dims} must be rot_dim {rot_dim}")
        dim = _count(raw, "dim", where)
        return cls(heads=_count(raw, "heads", where), dim=dim, rot_dim=rot_dim,
                   vdim=_count(raw, "vdim", where) if raw.get("vdim") is not None else dim,
                   kv_rank=_count(raw, "kv_rank", where), scale=_positive(raw, "scale", where),
                   window=_window(raw, where), rot=rot)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank}
        if self.window:
            out["mask"] = {"size": self.window}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        out.update(rot_dim=self.rot_dim, scale=self.scale, vdim=self.vdim)
        return out

    def shapes(self, base: str, w: int) -> Dict[str, tuple]:
        H, r = self.heads, self.kv_rank
        return {f"{base}.q": (H * (self.dim + self.rot_dim), w), f"{base}.dkv": (r + self.rot_dim, w),
                f"{base}.dkv.norm": (r,), f"{base}.uk": (H * self.dim, r), f"{base}.uv": (H * self.vdim, r),
                f"{base}.sink": (H,), f"{base}.o": (w, H * self.vdim)}

    def part(self, base: str, w: int, eps: float) -> PartSpec:
        return PartSpec("latent_attention", {
            "hidden_size": w, "num_heads": self.heads, "head_dim": self.dim, "rotary_head_dim": self.rot_dim,
            "value_dim": self.vdim, "kv_rank": self.kv_rank, "q_rank": None, "scale": self.scale, "eps": eps,
            "q_proj": f"{base}.q", "kv_down_proj": f"{base}.dkv", "k_up_proj": f"{base}.uk", "v_up_proj": f"{base}.uv",
            "o_proj": f"{base}.o", "q_norm": None,
            "kv_norm": PartSpec("rmsnorm", {"size": self.kv_rank, "eps": eps, "weight": f"{base}.dkv.norm"}),
            "position": self.rot.part(self.rot_dim) if self.rot is not None else None,
            "window": self.window or None, "sink": f"{base}.sink", "cache_mode": "auto"})


_MIXERS = {"channel_delta": ChannelDeltaMixer, "attention": BiasedAttention, "latent_attention": WindowedLatentAttention}


@dataclass(frozen=True)
class GatedDense:
    ff: int

    def to_dict(self) -> Dict[str, Any]:
        return {"ff": self.ff, "kind": "dense"}

    def shapes(self, base: str, w: int) -> Dict[str, tuple]:
        return {f"{base}.gate": (self.ff, w), f"{base}.up": (self.ff, w), f"{base}.down": (w, self.ff)}

    def part(self, base: str, w: int, activation: str = "gelu_tanh") -> PartSpec:
        return PartSpec("swiglu", {"hidden_size": w, "intermediate_size": self.ff, "gate_proj": f"{base}.gate",
                                   "up_proj": f"{base}.up", "down_proj": f"{base}.down", "activation": activation})


@dataclass(frozen=True)
class GroupedExperts:
    ff: int
    experts: int
    top: int
    scale: float
    group_count: int        # 1: the choice is among all experts
    group_keep: int
    shared_ff: int          # 0: no expert that every token uses

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "GroupedExperts":
        router = _object(raw.get("router"), f"{where}.router")
        experts, top = _count(router, "experts", f"{where}.router"), _count(router, "top", f"{where}.router")
        count, keep = 1, 1
        if router.get("groups") is not None:
            groups = _object(router["groups"], f"{where}.router.groups")
            count, keep = _count(groups, "count", f"{where}.router.groups"), _count(groups, "keep", f"{where}.router.groups")
        if experts % count or keep > count or keep * (experts // count) < top or top > experts:
            raise ConfigError("Json", f"{where}.router: top {top} of {experts} experts in {count} groups of which {keep} are kept")
        shared = 0
        if raw.get("shared") is not None:
            shared = _count(_object(raw["shared"], f"{where}.shared"), "ff", f"{where}.shared")
        return cls(ff=_count(_object(raw.get("expert"), f"{where}.expert"), "ff", f"{where}.expert"), experts=experts,
                   top=top, scale=_number(router, "scale", f"{where}.router") if router.get("scale") is not None else 1.0,
                   group_count=count, group_keep=keep, shared_ff=shared)

    def to_dict(self) -> Dict[str, Any]:
        router: Dict[str, Any] = {"experts": self.experts}
        if self.group_count > 1:
            router["groups"] = {"count": self.group_count, "keep": self.group_keep}
        router.update(scale=self.scale, top=self.top)
        out: Dict[str, Any] = {"expert": {"ff": self.ff}, "kind": "moe", "router": router}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out

    def shapes(self, base: str, w: int) -> Dict[str, tuple]:
        shapes: Dict[str, tuple] = {}
        for index in range(self.experts):
            shapes.update({f"{base}.e{index}.gate": (self.ff, w), f"{base}.e{index}.up": (self.ff, w),
                           f"{base}.e{index}.down": (w, self.ff)})
        shapes.update({f"{base}.router": (self.experts, w), f"{base}.correction": (self.experts,)})
        if self.shared_ff:
            shapes.update(GatedDense(self.shared_ff).shapes(f"{base}.shared", w))
            shapes[f"{base}.shared.sg"] = (1, w)
        return shapes

    def part(self, base: str, w: int) -> PartSpec:
        return PartSpec("routed_experts", {
            "hidden_size": w, "intermediate_size": self.ff, "experts": self.experts, "identity": 0, "top": self.top,
            "activation": "swiglu", "scores": "sigmoid", "scale": self.scale,
            "groups": (self.group_count, self.group_keep) if self.group_count > 1 else None,
            "gate_proj": base + ".e{}.gate", "up_proj": base + ".e{}.up", "down_proj": base + ".e{}.down",
            "router": f"{base}.router", "correction": f"{base}.correction",
            "shared": GatedDense(self.shared_ff).part(f"{base}.shared", w, "silu") if self.shared_ff else None,
            "shared_gate": f"{base}.shared.sg" if self.shared_ff else None})


def _feed_forward(raw: Mapping[str, Any], where: str):
    raw = _object(raw, where)
    kind = raw.get("kind")
    if kind == "dense":
        return GatedDense(ff=_count(raw, "ff", where))
    if kind == "moe":
        return GroupedExperts.from_dict(raw, where)
    raise ConfigError("UnsupportedFeedForward", f"{where}.kind {kind!r}; 'dense' or 'moe'")


@dataclass(frozen=True)
class DimoraxLayer:
    kind: str
    mixer: object
    mlp: Optional[object]       # None: no feed-forward

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "DimoraxLayer":
        raw = _object(raw, where)
        kind = raw.get("type")
        if kind not in _MIXERS:
            raise ConfigError("UnsupportedLayerType", f"{where}.type {kind!r}; this design has {sorted(_MIXERS)}")
        mlp = _feed_forward(raw["mlp"], f"{where}.mlp") if raw.get("mlp") is not None else None
        return cls(kind=kind, mixer=_MIXERS[kind].from_dict(raw.get("mixer"), f"{where}.mixer"), mlp=mlp)

    def to_dict(self) -> Dict[str, Any]:
        return {"mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp is not None else None,
                "type": self.kind}


@dataclass(frozen=True)
class DimoraxConfig:
    """Sizes and constants of one Dimorax checkpoint."""

    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[DimoraxLayer, ...]
    residual_mult: float = 1.0
    eos_token_ids: tuple = ()

    ARCHITECTURE = "Dimorax"
    MODEL_TYPE = "dimorax"

    @classmethod
    def parse(cls, text: str) -> "DimoraxConfig":
        try:
            raw = json.loads(text)
        except json.JSONDecodeError as error:
            raise ConfigError("Json", str(error)) from None
        return cls.from_dict(_object(raw, "config.json"))

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "DimoraxConfig":
        if raw.get("architecture") != cls.ARCHITECTURE:
            raise ConfigError("UnsupportedModelType", f"architecture {raw.get('architecture')!r}")
        vocab, width = _count(raw, "vocab", "config"), _count(raw, "width", "config")
        if width % 8:
            raise ConfigError("MissingDimension", f"width {width} must be a multiple of 8")
        eps = _number(_object(raw.get("norm"), "norm"), "eps", "norm")
        if eps <= 0.0:
            raise ConfigError("InvalidRmsNormEpsilon", str(eps))
        mult = _number(raw, "residual_mult", "config") if raw.get("residual_mult") is not None else 1.0
        given = raw.get("layers")
        if not isinstance(given, list) or not given:
            raise ConfigError("MissingDimension", "layers must be a list of at least one layer")
        layers = tuple(DimoraxLayer.from_dict(layer, f"layers[{i}]") for i, layer in enumerate(given))
        for index, layer in enumerate(layers):
            source = getattr(layer.mixer, "kv_from", None)
            if source is None:
                continue
            where = f"layers[{index}].mixer.kv_from"
            if source >= index or layers[source].kind != "attention" or layers[source].mixer.kv_from is not None:
                raise ConfigError("Json", f"{where} = {source} must name an earlier attention layer with projections of its own")
            theirs, ours = layers[source].mixer, layer.mixer
            if (theirs.kv_heads, theirs.dim, theirs.vdim, theirs.rot) != (ours.kv_heads, ours.dim, ours.vdim, ours.rot):
                raise ConfigError("Json", f"{where}: layer {source}'s key/value heads and rotation differ from this layer's")
            if theirs.window and (not ours.window or ours.window > theirs.window):
                raise ConfigError("Json", f"{where}: layer {source} keeps {theirs.window} positions, this layer needs more")
        return cls(vocab=vocab, width=width, norm_eps=eps, layers=layers, residual_mult=mult)

    # ------------------------------------------------------------ derived facts
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def parameter_count(self) -> int:
        return sum(math.prod(shape) for shape in self.tensor_shapes().values() if None not in shape)

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.ARCHITECTURE, "layers": [layer.to_dict() for layer in self.layers],
                "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab,
                "width": self.width}

    # ------------------------------------------------------------- model spec
    def to_model_spec(self) -> ModelSpec:
        w, eps = self.width, self.norm_eps
        norm = lambda name: PartSpec("rmsnorm", {"size": w, "eps": eps, "weight": name, "one_plus": True})
        layers, order = [], []
        for index, layer in enumerate(self.layers):
            base = f"l{index}"
            layers.append(LayerSpec(
                name=base, block=PartSpec("parallel_residual", {"hidden_size": w, "residual_scale": self.residual_mult}),
                mixer=layer.mixer.part(f"{base}.mix", w, eps),
                feed_forward=layer.mlp.part(f"{base}.mlp", w) if layer.mlp is not None else None,
                mixer_norm=norm(f"{base}.norm1"),
                feed_forward_norm=norm(f"{base}.norm2") if layer.mlp is not None else None))
            source = getattr(layer.mixer, "kv_from", None)
            # a layer without key and value projections reads the cache entry of the layer it names
            order.append(LayerRun(layer=index) if source is None else LayerRun(layer=index, cache=source, write_cache=False))
        spec = ModelSpec(
            architecture=self.ARCHITECTURE, hidden_size=w, vocab_size=self.vocab, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": w, "weight": "embed"}),
            layers=tuple(layers), order=tuple(order), final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": w, "weight": "head", "softcap": None}))
        spec.validate()
        return spec

    # ------------------------------------------------ tensors of a checkpoint
    def tensor_shapes(self) -> Dict[str, tuple]:
        """Shapes by name; None stands for a size that only the checkpoint's tensor gives."""
        w = self.width
        shapes: Dict[str, tuple] = {"embed": (self.vocab, w)}
        for index, layer in enumerate(self.layers):
            base = f"l{index}"
            shapes[f"{base}.norm1"] = (w,)
            if layer.mlp is not None:
                shapes[f"{base}.norm2"] = (w,)
            shapes.update(layer.mixer.shapes(f"{base}.mix", w))
            if layer.mlp is not None:
                shapes.update(layer.mlp.shapes(f"{base}.mlp", w))
        shapes["final.norm"] = (w,)
        shapes["head"] = (self.vocab, w)
        return shapes

    def ignored_tensors(self) -> tuple:
        """The second norm of a layer without a feed-forward, should a checkpoint hold it all the same."""
        return tuple(f"l{index}.norm2" for index, layer in enumerate(self.layers) if layer.mlp is None)

    def norm_tensor(self, name: str):
        """How a tensor of random weights is drawn: False for a matrix
        (N(0, 0.02)); "one" for a factor near 1; "zero" for an offset near 0."""
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2", "b", "sink", "correction", "dt_bias", "A_log") and not name.endswith(".mix.b"):
            return "zero"
        if name == "final.norm":
            return "zero"
        if last == "norm":       # the plain weights of the heads' and the latent's norms
            return "one"
        return False
