"""A plain, slow implementation of the Dimorax decoder in numpy.

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
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def over_rms(x, eps):
    """x over sqrt(mean(x^2) + eps) along the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def centred_norm(x, w, eps):
    """The layers' norm: its stored weight lies around zero, the factor is 1 + w."""
    return over_rms(x, eps) * (1.0 + w)


# ------------------------------------------------------------------ rotation
def yarn_frequencies(base, dims, scaling=None):
    """(f [dims / 2], magnitude): f_i = base^(-2i/dims); with ``scaling`` the
    slow pairs are divided by ``factor``, the fast ones kept, a linear ramp
    between, and cos and sin are multiplied by 0.1 ln(factor) + 1."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    where = lambda turns: dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(scaling["fast"])), 0)
    hi = min(math.ceil(where(scaling["slow"])), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def turn_halves(x, positions, base, dims, scaling=None):
    """x ``[T, heads, D]``: value i of the first ``dims`` is paired with value
    i + dims / 2; the pair (u, v) at position p becomes
    (u cos a - v sin a, v cos a + u sin a), a = p f_i."""
    f, magnitude = yarn_frequencies(base, dims, scaling)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(angle) * magnitude)[:, None, :], (np.sin(angle) * magnitude)[:, None, :]
    half = dims // 2
    out = np.array(x, dtype=np.float64, copy=True)
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ------------------------------------------------------------------ softmax
def sink_softmax(scores, visible, sink=None):
    """Weights exp(s_j) / (exp(sink) + sum over visible exp(s_j)) along the last axis."""
    masked = np.where(visible, scores, -np.inf)
    peak = masked.max(axis=-1, keepdims=True)
    if sink is not None:
        peak = np.maximum(peak, sink)
    e = np.where(visible, np.exp(masked - peak), 0.0)
    total = e.sum(axis=-1, keepdims=True)
    if sink is not None:
        total = total + np.exp(sink - peak)
    return e / total


def seen_keys(count, window=0):
    """[T, T]: query i sees key j when j <= i and (with a window) i - j < window."""
    i, j = np.arange(count)[:, None], np.arange(count)[None, :]
    seen = j <= i
    if window:
        seen &= (i - j) < window
    return seen


# ---------------------------------------------------------------- attention
def keys_and_values(h, tensors, base, mixer):
    """Rotated keys ``[T, G, D]`` and values ``[T, G, Dv]`` of an attention layer that has projections."""
    count, G, D, Dv = h.shape[0], mixer.get("kv_heads") or mixer["heads"], mixer["dim"], mixer.get("vdim") or mixer["dim"]
    k = (h @ tensors[f"{base}.k"].T + tensors[f"{base}.k.b"]).reshape(count, G, D)
    v = (h @ tensors[f"{base}.v"].T + tensors[f"{base}.v.b"]).reshape(count, G, Dv)
    rot = mixer.get("rot")
    if rot:
        k = turn_halves(k, np.arange(count), rot["base"], rot["dims"], rot.get("scaling"))
    return k, v


def biased_attention(h, tensors, base, mixer, keys=None, values=None, weights_out=None, use_sink=True):
    """Grouped-query attention with biased projections, rotation of halves,
    capped scores, a causal mask and a learned sink per head. ``keys`` /
    ``values``: another layer's, for a layer without projections of its own."""
    count, H, D = h.shape[0], mixer["heads"], mixer["dim"]
    G, Dv = mixer.get("kv_heads") or H, mixer.get("vdim") or D
    q = (h @ tensors[f"{base}.q"].T + tensors[f"{base}.q.b"]).reshape(count, H, D)
    rot = mixer.get("rot")
    if rot:
        q = turn_halves(q, np.arange(count), rot["base"], rot["dims"], rot.get("scaling"))
    if keys is None:
        keys, values = keys_and_values(h, tensors, base, mixer)
    cap = mixer.get("softcap")
    seen = seen_keys(count, (mixer.get("mask") or {}).get("size", 0))
    out = np.zeros((count, H, Dv))
    for head in range(H):
        group = head // (H // G)
        scores = (q[:, head] @ keys[:, group].T) * mixer["scale"]
        if cap:
            scores = cap * np.tanh(scores / cap)
        p = sink_softmax(scores, seen, float(tensors[f"{base}.sink"][head]) if use_sink else None)
        if weights_out is not None:
            weights_out.append(p)
        out[:, head] = p @ values[:, group]
    return out.reshape(count, H * Dv) @ tensors[f"{base}.o"].T


def latent_attention(h, tensors, base, mixer, eps, weights_out=None, use_sink=True):
    """Keys and values from one normed latent per position plus one rotated
    key part that all heads share; a sliding window; a learned sink per head."""
    count, H, D, R, r = h.shape[0], mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["kv_rank"]
    Dv = mixer.get("vdim") or D
    positions = np.arange(count)
    rot = mixer["rot"]
    q = (h @ tensors[f"{base}.q"].T).reshape(count, H, D + R)
    q_plain, q_turned = q[..., :D], turn_halves(q[..., D:], positions, rot["base"], R, rot.get("scaling"))
    down = h @ tensors[f"{base}.dkv"].T
    c = over_rms(down[:, :r], eps) * tensors[f"{base}.dkv.norm"]
    k_turned = turn_halves(down[:, None, r:], positions, rot["base"], R, rot.get("scaling"))[:, 0]
    k_plain = (c @ tensors[f"{base}.uk"].T).reshape(count, H, D)
    v = (c @ tensors[f"{base}.uv"].T).reshape(count, H, Dv)
    seen = seen_keys(count, (mixer.get("mask") or {}).get("size", 0))
    out = np.zeros((count, H, Dv))
    for head in range(H):
        scores = (q_plain[:, head] @ k_plain[:, head].T + q_turned[:, head] @ k_turned.T) * mixer["scale"]
        p = sink_softmax(scores, seen, float(tensors[f"{base}.sink"][head]) if use_sink else None)
        if weights_out is not None:
            weights_out.append(p)
        out[:, head] = p @ v[:, head]
    return out.reshape(count, H * Dv) @ tensors[f"{base}.o"].T


# ------------------------------------------------------- the delta recurrence
def causal_conv(x, taps_weight, before=None):
    """x ``[T, C]``, taps_weight ``[C, K]`` whose last column meets the current
    token: y_t = sum_j w[:, j] x_(t - K + 1 + j), zeros before the sequence
    (or ``before`` ``[K - 1, C]``). Returns y and the last K - 1 inputs."""
    count, channels = x.shape
    k = taps_weight.shape[1]
    if before is None:
        before = np.zeros((k - 1, channels))
    padded = np.concatenate([before, x], axis=0)
    y = np.zeros_like(x)
    for j in range(k):
        y += taps_weight[:, j][None, :] * padded[j:j + count]
    return y, padded[count:]


def delta_rule(q, k, v, beta, decay, state=None):
    """One head. q, k, decay ``[T, D]``, v ``[T, Dv]``, beta ``[T]``. Per token:
    S <- decay[:, None] * S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.
    Returns o ``[T, Dv]`` and the last S ``[D, Dv]``."""
    count, dim = q.shape
    s = np.zeros((dim, v.shape[1])) if state is None else np.array(state, dtype=np.float64, copy=True)
    out = np.zeros((count, v.shape[1]))
    for t in range(count):
        s = decay[t][:, None] * s
        u = beta[t] * (v[t] - s.T @ k[t])
        s = s + np.outer(k[t], u)
        out[t] = s.T @ q[t]
    return out, s


def channel_delta(h, tensors, base, mixer, eps, carry=None):
    """The gated delta rule with one decay per head and key channel.
    ``carry`` = (conv inputs of q, k, v, states [H, D, Dv]) from an earlier
    piece; returns the output and the new carry."""
    count, H, D = h.shape[0], mixer["heads"], mixer["dim"]
    G, Dv = mixer.get("kv_heads") or H, mixer.get("vdim") or D
    before = carry if carry is not None else (None, None, None, [None] * H)
    q, q_in = causal_conv(h @ tensors[f"{base}.q"].T, tensors[f"{base}.q.conv"], before[0])
    k, k_in = causal_conv(h @ tensors[f"{base}.k"].T, tensors[f"{base}.k.conv"], before[1])
    v, v_in = causal_conv(h @ tensors[f"{base}.v"].T, tensors[f"{base}.v.conv"], before[2])
    q, k, v = silu(q).reshape(count, G, D), silu(k).reshape(count, G, D), silu(v).reshape(count, H, Dv)
    unit = lambda x: x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + 1e-6)
    q, k = unit(q) * D ** -0.5, unit(k)
    beta = sigmoid(h @ tensors[f"{base}.b"].T)                                            # [T, H]
    step = softplus((h @ tensors[f"{base}.a1"].T) @ tensors[f"{base}.a2"].T + tensors[f"{base}.dt_bias"])
    decay = np.exp(-np.exp(tensors[f"{base}.A_log"])[None, :, None] * step.reshape(count, H, D))
    gate = sigmoid((h @ tensors[f"{base}.g1"].T) @ tensors[f"{base}.g2"].T).reshape(count, H, Dv)
    out, states = np.zeros((count, H, Dv)), []
    for head in range(H):
        group = head // (H // G)
        o, s = delta_rule(q[:, group], k[:, group], v[:, head], beta[:, head], decay[:, head], before[3][head])
        out[:, head] = over_rms(o, eps) * tensors[f"{base}.norm"] * gate[:, head]
        states.append(s)
    return out.reshape(count, H * Dv) @ tensors[f"{base}.o"].T, (q_in, k_in, v_in, states)


# ------------------------------------------------------------- feed-forward
def gated_ff(h, gate, up, down, act):
    return (act(h @ gate.T) * (h @ up.T)) @ down.T


def choose_experts(logits, correction, top, groups=None, scale=1.0):
    """s = sigmoid(logits); the choice goes by s + correction among the experts
    of the ``keep`` best groups (a group's score: the sum of its two largest
    s + correction), the ``top`` largest; the lower index wins a tie. Weights:
    the chosen s over their sum (+ 1e-20), times ``scale``."""
    s = sigmoid(logits)
    choice = s + correction[None, :]
    count, experts = s.shape
    if groups:
        size = experts // groups["count"]
        grouped = choice.reshape(count, groups["count"], size)
        best_two = np.sort(grouped, axis=-1)[..., -2:].sum(axis=-1)
        kept = np.argsort(-best_two, axis=-1, kind="stable")[:, :groups["keep"]]
        allowed = np.zeros((count, groups["count"]), dtype=bool)
        np.put_along_axis(allowed, kept, True, axis=-1)
        choice = np.where(np.repeat(allowed, size, axis=-1), choice, -np.inf)
    chosen = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    picked = np.take_along_axis(s, chosen, axis=-1)
    return chosen, picked / (picked.sum(axis=-1, keepdims=True) + 1e-20) * scale


def expert_mixture(h, tensors, base, mlp, chosen_out=None):
    router = mlp["router"]
    chosen, weights = choose_experts(h @ tensors[f"{base}.router"].T, tensors[f"{base}.correction"], router["top"],
                                     router.get("groups"), router.get("scale", 1.0))
    if chosen_out is not None:
        chosen_out.append(chosen)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weights[t]):
            out[t] += w * gated_ff(h[t:t + 1], tensors[f"{base}.e{e}.gate"], tensors[f"{base}.e{e}.up"],
                                   tensors[f"{base}.e{e}.down"], silu)[0]
    if mlp.get("shared"):
        share = sigmoid(h @ tensors[f"{base}.shared.sg"].T)                               # [T, 1]
        out += share * gated_ff(h, tensors[f"{base}.shared.gate"], tensors[f"{base}.shared.up"],
                                tensors[f"{base}.shared.down"], silu)
    return out


def feed_forward(h, tensors, base, mlp, chosen_out=None):
    if mlp["kind"] == "dense":
        return gated_ff(h, tensors[f"{base}.gate"], tensors[f"{base}.up"], tensors[f"{base}.down"], gelu_tanh)
    if mlp["kind"] == "moe":
        return expert_mixture(h, tensors, base, mlp, chosen_out)
    raise ValueError(mlp["kind"])


# ------------------------------------------------------------------ the model
def forward_logits(config, tensors, ids, taps=None, seen=None, use_sink=True):
    """Logits ``[T, vocab]`` of a whole sequence. ``taps`` (a list) takes the
    residual stream after every layer; ``seen`` (a dict) takes, per layer, the
    attention weights or the chosen experts."""
    tensors = {name: np.asarray(t, dtype=np.float64) for name, t in tensors.items()}
    eps, m = config["norm"]["eps"], config.get("residual_mult", 1.0)
    x = tensors["embed"][np.asarray(ids)]
    shared = {}
    for index, layer in enumerate(config["layers"]):
        base, mixer, kind = f"l{index}", layer["mixer"], layer["type"]
        h = centred_norm(x, tensors[f"{base}.norm1"], eps)
        weights = [] if seen is not None else None
        if kind == "channel_delta":
            mixed = channel_delta(h, tensors, f"{base}.mix", mixer, eps)[0]
        elif kind == "attention":
            if mixer.get("kv_from") is not None:
                keys, values = shared[mixer["kv_from"]]
            else:
                keys, values = shared[index] = keys_and_values(h, tensors, f"{base}.mix", mixer)
            mixed = biased_attention(h, tensors, f"{base}.mix", mixer, keys, values, weights, use_sink)
        elif kind == "latent_attention":
            mixed = latent_attention(h, tensors, f"{base}.mix", mixer, eps, weights, use_sink)
        else:
            raise ValueError(kind)
        if seen is not None and weights:
            seen[(index, "attention")] = weights
        if layer.get("mlp") is not None:
            chosen = [] if seen is not None else None
            mixed = mixed + feed_forward(centred_norm(x, tensors[f"{base}.norm2"], eps), tensors, f"{base}.mlp",
                                         layer["mlp"], chosen)
            if seen is not None and chosen:
                seen[(index, "experts")] = chosen[0]
        x = x + m * mixed
        if taps is not None:
            taps.append(x.copy())
    return centred_norm(x, tensors["final.norm"], eps) @ tensors["head"].T
