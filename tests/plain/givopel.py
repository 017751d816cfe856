"""Plain, slow restatement of the Givopel decoder, one function per mechanism.

The oracle of the Givopel tests.  It shares no code with the product package: whole sequences,
no cache, token-by-token loops for every recurrence, numpy float64 throughout.

The design in short.  Every layer is x <- x + mixer(h) + feed_forward(h) with ONE weighted layer
norm h = LN(x) that both read.  A mixer is either a gated linear attention ("gla": a matrix state
per head with a learned decay per key channel) or two mixers side by side ("parallel": softmax
attention with rotated, YaRN-scaled positions and an output gate on the left, a gated delta rule
with short convolutions on the right, each RMS-normed over the width and averaged).  A stretch of
layers may run several times in a row with the same weights; each pass begins by mixing the stream
with the embedding output through one matrix.  The logits are scaled and soft-capped.
"""
from __future__ import annotations

import math

import numpy as np

F64 = np.float64


# ----------------------------------------------------------------------------- small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    x = np.asarray(x, F64)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * weight


def layer_norm(x, weight, eps):
    """(x - mean) / sqrt(var + eps) * w, var = mean of squared deviations, no bias."""
    x = np.asarray(x, F64)
    mean = x.mean(axis=-1, keepdims=True)
    dev = x - mean
    return dev / np.sqrt((dev * dev).mean(axis=-1, keepdims=True) + eps) * weight


# ----------------------------------------------------------------------------- positions
def yarn_frequencies(dims: int, base: float, scaling: dict | None):
    """(frequencies [dims / 2], multiplier of cos and sin)."""
    i = np.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, positions, dims: int, base: float, scaling: dict | None):
    """x [T, heads, dim]: the pair (2i, 2i + 1) of the first ``dims`` dims of every head turns by
    position * f_i; the rest passes."""
    f, mult = yarn_frequencies(dims, base, scaling)
    angle = np.asarray(positions, F64)[:, None] * f[None, :]
    cos, sin = np.cos(angle)[:, None, :] * mult, np.sin(angle)[:, None, :] * mult
    out = np.array(x, F64)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# ----------------------------------------------------------------------------- mixers
def softmax_attention(p: dict, w, prefix: str, h):
    """The left half: grouped-query causal softmax attention with an output gate."""
    T = h.shape[0]
    H, G, dim, vdim = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    q = (h @ w[prefix + "q"].T).reshape(T, H, dim)
    k = (h @ w[prefix + "k"].T).reshape(T, G, dim)
    v = (h @ w[prefix + "v"].T).reshape(T, G, vdim)
    rot = p.get("rot")
    if rot:
        pos = np.arange(T)
        q = rotate_interleaved(q, pos, rot["dims"], rot["base"], rot.get("scaling"))
        k = rotate_interleaved(k, pos, rot["dims"], rot["base"], rot.get("scaling"))
    out = np.zeros((T, H, vdim), F64)
    for head in range(H):
        g = head // (H // G)
        for t in range(T):
            s = (k[:t + 1, g] @ q[t, head]) * p["scale"]
            s = np.exp(s - s.max())
            out[t, head] = (s / s.sum()) @ v[:t + 1, g]
    gate = sigmoid(h @ w[prefix + "g"].T)
    return (out.reshape(T, H * vdim) * gate) @ w[prefix + "o"].T


def short_convolution(x, taps_weight):
    """x [T, C], taps_weight [C, taps]: y_t = sum_j w[:, j] x_(t - (taps - 1) + j), zeros before 0."""
    T, C = x.shape
    taps = taps_weight.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), F64), x])
    y = np.zeros((T, C), F64)
    for j in range(taps):
        y += padded[j:j + T] * taps_weight[:, j]
    return y


def state_scan(q, k, v, decay, beta=None):
    """One head, token by token: S <- decay_t * S (rows); u = v_t, or with ``beta`` the delta rule
    u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t.  q, k, decay [T, dim], v [T, vdim], beta [T]."""
    T, dim = q.shape
    S = np.zeros((dim, v.shape[1]), F64)
    out = np.zeros((T, v.shape[1]), F64)
    for t in range(T):
        S = decay[t][:, None] * S
        u = v[t] if beta is None else beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def gated_delta_rule(p: dict, w, prefix: str, h, eps: float):
    """The right half: a matrix state per head, decayed per key channel, corrected by the delta rule."""
    T = h.shape[0]
    H, G, dim, vdim = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    q = silu(short_convolution(h @ w[prefix + "q"].T, w[prefix + "q.conv"])).reshape(T, G, dim)
    k = silu(short_convolution(h @ w[prefix + "k"].T, w[prefix + "k.conv"])).reshape(T, G, dim)
    v = silu(short_convolution(h @ w[prefix + "v"].T, w[prefix + "v.conv"])).reshape(T, H, vdim)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dim ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[prefix + "b"].T)
    step = softplus((h @ w[prefix + "a1"].T) @ w[prefix + "a2"].T + w[prefix + "dt_bias"]).reshape(T, H, dim)
    decay = np.exp(-np.exp(w[prefix + "A_log"])[None, :, None] * step)
    out = np.zeros((T, H, vdim), F64)
    for head in range(H):
        g = head // (H // G)
        out[:, head] = state_scan(q[:, g], k[:, g], v[:, head], decay[:, head], beta[:, head])
    out = out / np.sqrt((out * out).mean(-1, keepdims=True) + eps) * w[prefix + "norm"]
    gate = sigmoid((h @ w[prefix + "g1"].T) @ w[prefix + "g2"].T)
    return (out.reshape(T, H * vdim) * gate) @ w[prefix + "o"].T


def gated_linear_attention(p: dict, w, prefix: str, h, eps: float):
    """The 'gla' mixer: S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T = h.shape[0]
    H, dim, vdim = p["heads"], p["dim"], p["vdim"]
    q = (h @ w[prefix + "q"].T).reshape(T, H, dim) * dim ** -0.5
    k = (h @ w[prefix + "k"].T).reshape(T, H, dim)
    v = (h @ w[prefix + "v"].T).reshape(T, H, vdim)
    z = (h @ w[prefix + "a1"].T) @ w[prefix + "a2"].T + w[prefix + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / p["tau"])).reshape(T, H, dim)
    out = np.zeros((T, H, vdim), F64)
    for head in range(H):
        out[:, head] = state_scan(q[:, head], k[:, head], v[:, head], alpha[:, head])
    out = rms_norm(out, w[prefix + "norm"], eps)
    return (out.reshape(T, H * vdim) * silu(h @ w[prefix + "g"].T)) @ w[prefix + "o"].T


def side_by_side(p: dict, w, prefix: str, h, eps: float):
    """The 'parallel' mixer: half the sum of the two halves, each RMS-normed over the width."""
    left = softmax_attention(p["left"], w, prefix + "left.", h)
    right = gated_delta_rule(p["right"], w, prefix + "right.", h, eps)
    return 0.5 * (rms_norm(left, w[prefix + "left.out"], eps) + rms_norm(right, w[prefix + "right.out"], eps))


def feed_forward(w, prefix: str, h):
    return (silu(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


# ----------------------------------------------------------------------------- the model
def layer_order(config: dict):
    """[(layer index, first of a pass)] in the order the layers run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for _ in range(times):
        order += [(i, i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def run_layer(config: dict, w, index: int, x):
    layer = config["layers"][index]
    eps = config["norm"]["eps"]
    prefix = f"l{index}."
    h = layer_norm(x, w[prefix + "norm1"], eps)
    if layer["type"] == "gla":
        mixed = gated_linear_attention(layer["mixer"], w, prefix + "mix.", h, eps)
    elif layer["type"] == "parallel":
        mixed = side_by_side(layer["mixer"], w, prefix + "mix.", h, eps)
    else:
        raise ValueError(f"layer type {layer['type']!r}")
    if layer.get("mlp"):
        mixed = mixed + feed_forward(w, prefix + "mlp.", h)
    return x + mixed


def forward(config: dict, weights: dict, tokens, keep_layers: bool = False):
    """Logits [T, vocab] of one sequence (and the stream after every layer run, if asked)."""
    w = {k: np.asarray(v, F64) for k, v in weights.items()}
    x0 = w["embed"][np.asarray(tokens, np.int64)]
    x, streams = x0, []
    for index, first in layer_order(config):
        if first:
            x = np.concatenate([x, x0], axis=-1) @ w["loop.in"].T
        x = run_layer(config, w, index, x)
        streams.append(x)
    logits = layer_norm(x, w["final.norm"], config["norm"]["eps"]) @ w["head"].T * config.get("logit_scale", 1.0)
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * np.tanh(logits / cap)
    return (logits, np.stack(streams)) if keep_layers else logits
