"""A plain, slow implementation of the Sadosun decoder in numpy.

Whole sequences, no cache, float64, one function per mechanism; a recurrence
hands its state back so that a test can run it in pieces. It shares no code
with ``metallix_b200`` (files are read with the reader of the other plain
implementation in this folder). Notation: x is ``[T, W]`` (tokens by width),
positions count from 0, weights are ``[out, in]`` and applied as x @ w.T.
"""
from __future__ import annotations

import math

import numpy as np

from plain_qwen3 import read_model  # noqa: F401  (a reader of config.json + safetensors, nothing else)


# ------------------------------------------------------------ small pieces
def silu(z):
    return z / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    """x over sqrt(mean(x^2) + eps) along the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm(x, gain, eps):
    """RMS norm; ``gain`` is one number for all coordinates or one per coordinate."""
    return unit_rms(x, eps) * gain


# ------------------------------------------------ convolution over time
def causal_conv(x, taps_weight, bias=None, before=None):
    """x ``[T, C]``, taps_weight ``[C, K]`` whose last column meets the current
    token: y_t = bias + sum_j w[:, j] x_(t - K + 1 + j). ``before`` ``[K - 1, C]``
    stands for the inputs ahead of x (zeros at a sequence's start). Returns y
    and the last K - 1 inputs, for the next piece."""
    count, channels = x.shape
    k = taps_weight.shape[1]
    if before is None:
        before = np.zeros((k - 1, channels))
    padded = np.concatenate([before, x], axis=0)
    y = np.zeros_like(x)
    for j in range(k):
        y += taps_weight[:, j][None, :] * padded[j:j + count]
    if bias is not None:
        y = y + bias[None, :]
    return y, padded[count:]


def corrected_input(h, taps_weight):
    """What a sublayer reads: h + conv(h)."""
    return h + causal_conv(h, taps_weight)[0]


# ---------------------------------------------------------------- rotation
def turn_pairs(x, positions, base, dims, sign=1.0):
    """x ``[T, heads, D]``: the neighbouring pair (2i, 2i + 1) of the first
    ``dims`` values turns by sign * position * base^(-2i/dims);
    (u, v) -> (u cos - v sin, v cos + u sin)."""
    out = np.array(x, dtype=np.float64, copy=True)
    for i in range(dims // 2):
        angle = sign * np.asarray(positions, dtype=np.float64) * base ** (-2.0 * i / dims)
        c, s = np.cos(angle)[:, None], np.sin(angle)[:, None]
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - v * s
        out[:, :, 2 * i + 1] = v * c + u * s
    return out


# --------------------------------------------------------------- attention
def sink_softmax(scores, visible, sink=0.0):
    """Weights exp(s_j) / (exp(sink) + sum_visible exp(s_j)) along the last
    axis: one more key of score ``sink`` that has no value (None: plain softmax)."""
    masked = np.where(visible, scores, -np.inf)
    peak = masked.max(axis=-1, keepdims=True)
    if sink is not None:
        peak = np.maximum(peak, sink)
    e = np.where(visible, np.exp(masked - peak), 0.0)
    total = e.sum(axis=-1, keepdims=True)
    if sink is not None:
        total = total + np.exp(sink - peak)
    return e / total


def window_mask(count, window):
    """[T, T]: query i sees key j when 0 <= i - j < window (0: every earlier key)."""
    i, j = np.arange(count)[:, None], np.arange(count)[None, :]
    seen = j <= i
    if window:
        seen &= (i - j) < window
    return seen


def windowed_attention(h, wq, wk, wv, wo, *, heads, kv_heads, dim, vdim, scale, window, rot, eps, weights_out=None,
                       sink=0.0):
    """Grouped-query attention with rotated then unit-normed q and k, values
    turned by their own position and the output turned back by the query's,
    a window, and a sink of score 0 (``sink=None``: a plain softmax, which the
    design does not have; for tests that show what the sink changes).
    ``rot`` = (base, dims) or None."""
    count = h.shape[0]
    positions = np.arange(count)
    q = (h @ wq.T).reshape(count, heads, dim)
    k = (h @ wk.T).reshape(count, kv_heads, dim)
    v = (h @ wv.T).reshape(count, kv_heads, vdim)
    if rot is not None:
        base, dims = rot
        q, k = turn_pairs(q, positions, base, dims), turn_pairs(k, positions, base, dims)
        v = turn_pairs(v, positions, base, vdim)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    group = heads // kv_heads
    seen = window_mask(count, window)
    out = np.zeros((count, heads, vdim))
    for head in range(heads):
        scores = (q[:, head] @ k[:, head // group].T) * scale
        p = sink_softmax(scores, seen, sink)
        if weights_out is not None:
            weights_out.append(p)
        out[:, head] = p @ v[:, head // group]
    if rot is not None:
        out = turn_pairs(out, positions, rot[0], vdim, sign=-1.0)
    return out.reshape(count, heads * vdim) @ wo.T


# ---------------------------------------------------- selective state space
def selective_recurrence(x, dt, a, b, c, d, state=None):
    """x, dt ``[T, N]``, a ``[N, n]`` (negative), b, c ``[T, n]``, d ``[N]``:
    S <- exp(dt A) S + dt x B; y = S C + D x. Returns y and the last state."""
    count, channels = x.shape
    s = np.zeros(a.shape) if state is None else np.array(state, dtype=np.float64, copy=True)
    y = np.zeros((count, channels))
    for t in range(count):
        s = np.exp(dt[t][:, None] * a) * s + (dt[t] * x[t])[:, None] * b[t][None, :]
        y[t] = s @ c[t] + d * x[t]
    return y, s


def selective_mixer(h, tensors, base, *, inner, states, rank):
    both = h @ tensors[f"{base}.in"].T
    x, z = both[:, :inner], both[:, inner:]
    x = silu(causal_conv(x, tensors[f"{base}.conv"], tensors[f"{base}.conv.b"].reshape(-1))[0])
    picked = x @ tensors[f"{base}.x"].T
    low, b, c = picked[:, :rank], picked[:, rank:rank + states], picked[:, rank + states:]
    dt = softplus(low @ tensors[f"{base}.dt"].T + tensors[f"{base}.dt.b"].reshape(-1)[None, :])
    y, _ = selective_recurrence(x, dt, -np.exp(tensors[f"{base}.A_log"]), b, c, tensors[f"{base}.D"].reshape(-1))
    return (y * silu(z)) @ tensors[f"{base}.o"].T


# ------------------------------------------------------------ routed experts
def choose_experts(logits, correction, top):
    """Scores = softmax(logits); the ``top`` largest score + correction are
    chosen (the lower index on a tie); weights = chosen scores over their sum.
    Returns chosen ``[T, top]`` and weights ``[T, top]``."""
    z = logits - logits.max(axis=-1, keepdims=True)
    scores = np.exp(z) / np.exp(z).sum(axis=-1, keepdims=True)
    order = np.argsort(-(scores + correction[None, :]), axis=-1, kind="stable")[:, :top]
    picked = np.take_along_axis(scores, order, axis=-1)
    return order, picked / (picked.sum(axis=-1, keepdims=True) + 1e-20)


def expert_mixture(h, tensors, base, *, experts, identity, top, chosen_out=None):
    logits = h @ tensors[f"{base}.router"].T
    chosen, weights = choose_experts(logits, tensors[f"{base}.correction"].reshape(-1), top)
    if chosen_out is not None:
        chosen_out.append(chosen)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weights[t]):
            if e >= experts:      # an expert that returns its input
                out[t] += w * h[t]
            else:
                up, down = tensors[f"{base}.e{e}.up"], tensors[f"{base}.e{e}.down"]
                out[t] += w * (np.square(np.maximum(up @ h[t], 0.0)) @ down.T)
    return out


# ------------------------------------------------------ input from the token
def token_input(x, ids, tensors, base, layer, dim, eps):
    e = tensors["side.embed"][np.asarray(ids)][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ tensors[f"{base}.side.gate"].T) * e
    y = g @ tensors[f"{base}.side.proj"].T
    return unit_rms(y, eps) * tensors[f"{base}.side.norm"].reshape(-1)[None, :]


# ------------------------------------------------------------------ the model
def forward_logits(config, tensors, ids, taps=None, seen=None, sink=0.0, forget_at=0):
    """Logits ``[T, vocab]`` of a whole sequence. ``taps`` (a list) takes the
    residual stream after every layer; ``seen`` (a dict) takes, per layer, the
    attention weights or the chosen experts. ``forget_at`` = t shows what a
    lost state does: convolutions and recurrences start anew at position t
    (attention still sees every key)."""
    def carried(function, h):
        if not forget_at:
            return function(h)
        return np.concatenate([function(h[:forget_at]), function(h[forget_at:])], axis=0)

    eps = config["norm"]["eps"]
    scale = (config.get("embedding") or {}).get("scale", 1.0)
    canon = (config.get("canon") or {}).get("taps", 0)
    side = (config.get("token_side") or {}).get("dim", 0)
    x = tensors["embed"][np.asarray(ids)] * scale
    for index, layer in enumerate(config["layers"]):
        base, mixer = f"l{index}", layer["mixer"]
        h = norm(x, float(tensors[f"{base}.norm1"]), eps)
        if canon:
            h = carried(lambda part: corrected_input(part, tensors[f"{base}.canon1"]), h)
        if layer["type"] == "attention":
            heads = mixer["heads"]
            rot = (mixer["rot"]["base"], mixer["rot"]["dims"]) if mixer.get("rot") else None
            weights = [] if seen is not None else None
            x = x + windowed_attention(
                h, tensors[f"{base}.mix.q"], tensors[f"{base}.mix.k"], tensors[f"{base}.mix.v"], tensors[f"{base}.mix.o"],
                heads=heads, kv_heads=mixer.get("kv_heads") or heads, dim=mixer["dim"], vdim=mixer.get("vdim") or mixer["dim"],
                scale=mixer["scale"], window=(mixer.get("mask") or {}).get("size", 0), rot=rot, eps=eps, weights_out=weights,
                sink=sink)
            if seen is not None:
                seen[(index, "attention")] = weights
        elif layer["type"] == "mamba1":
            x = x + carried(lambda part: selective_mixer(part, tensors, f"{base}.mix", inner=mixer["inner"],
                                                         states=mixer["state"], rank=mixer["dt_rank"]), h)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            h = norm(x, float(tensors[f"{base}.norm2"]), eps)
            if canon:
                h = carried(lambda part: corrected_input(part, tensors[f"{base}.canon2"]), h)
            router = layer["mlp"]["router"]
            chosen = [] if seen is not None else None
            x = x + expert_mixture(h, tensors, f"{base}.mlp", experts=router["experts"], identity=router.get("identity") or 0,
                                   top=router["top"], chosen_out=chosen)
            if seen is not None:
                seen[(index, "experts")] = chosen[0]
        if side:
            x = x + token_input(x, ids, tensors, base, index, side, eps)
        if taps is not None:
            taps.append(x.copy())
    return norm(x, float(tensors["final.norm"]), eps) @ tensors["head"].T
