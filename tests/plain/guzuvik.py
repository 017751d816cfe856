"""Plain, slow restatement of the Guzuvik decoder, one function per mechanism.

The oracle of the Guzuvik tests.  It shares no code with the product package: whole sequences, no cache,
token-by-token loops for every recurrence, numpy float64 throughout.

The design in short.  The input is a token embedding plus a hashed embedding of the (previous, current)
token pair.  Every layer is x <- x + LN_1b(mixer(LN_1(x))), then, if it has a feed-forward,
x <- x + LN_2b(ff(LN_2(x))), with layer norms that carry a weight and a bias.  A mixer is a Mamba-2
state-space recurrence (one scalar decay per head and token, B and C shared by the heads of a group) or
softmax attention without rotation: unit-RMS q and k, a tanh cap on the scores, a penalty that grows
linearly with the distance, a window that also keeps the sequence's first tokens, values blended with the
values of the first such layer, and one sigmoid gate per head.  A feed-forward is dense (squared relu) or a
mixture of small gated experts.  The logits are the final norm times the embedding table.
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


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis, no weight."""
    x = np.asarray(x, F64)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def layer_norm(x, weight, bias, eps):
    """(x - mean) / sqrt(var + eps) * w + b, var = mean of squared deviations."""
    x = np.asarray(x, F64)
    dev = x - x.mean(axis=-1, keepdims=True)
    return dev / np.sqrt((dev * dev).mean(axis=-1, keepdims=True) + eps) * weight + bias


# ----------------------------------------------------------------------------- embedding
def bigram_rows(tokens, buckets: int, mul_prev: int, mul_cur: int):
    """Row of the pair table for every token: a hash of (previous, current); the table's last row (number
    ``buckets``) for a sequence's first token."""
    rows = []
    for i, t in enumerate(tokens):
        rows.append(buckets if i == 0 else (int(tokens[i - 1]) * mul_prev + int(t) * mul_cur) % buckets)
    return rows


def embed(tokens, table, pair_table, buckets, mul_prev, mul_cur):
    return np.asarray(table, F64)[list(tokens)] + np.asarray(pair_table, F64)[bigram_rows(tokens, buckets, mul_prev, mul_cur)]


# ----------------------------------------------------------------------------- Mamba-2
def causal_conv(x, weight, bias):
    """x [T, C], weight [C, taps]: y_t = bias + sum_j weight[:, taps - 1 - j] x_(t - j), zeros before the start."""
    x, weight = np.asarray(x, F64), np.asarray(weight, F64)
    n, taps = x.shape[0], weight.shape[1]
    y = np.tile(np.asarray(bias, F64), (n, 1))
    for t in range(n):
        for j in range(taps):
            if t - j >= 0:
                y[t] += weight[:, taps - 1 - j] * x[t - j]
    return y


def ssd_scan(x, b, c, dt, a_log, d_skip, heads, vdim, state, groups):
    """x [T, heads * vdim], b and c [T, groups * state], dt [T, heads] (already positive).  Per head:
    S_t = exp(-exp(a_log) dt_t) S_(t-1) + dt_t b_t x_t^T, y_t = S_t^T c_t + d_skip x_t."""
    n = x.shape[0]
    y = np.zeros((n, heads * vdim), F64)
    per_group = heads // groups
    for h in range(heads):
        g = h // per_group
        s = np.zeros((state, vdim), F64)
        for t in range(n):
            xt = x[t, h * vdim:(h + 1) * vdim]
            bt, ct = b[t, g * state:(g + 1) * state], c[t, g * state:(g + 1) * state]
            s = math.exp(-math.exp(a_log[h]) * dt[t, h]) * s + dt[t, h] * np.outer(bt, xt)
            y[t, h * vdim:(h + 1) * vdim] = s.T @ ct + d_skip[h] * xt
    return y


def gated_group_norm(y, z, weight, parts: int, eps):
    """(y * silu(z)), each of ``parts`` equal stretches of the row divided by its own root mean square, times weight."""
    v = np.asarray(y, F64) * silu(np.asarray(z, F64))
    n, width = v.shape
    v = unit_rms(v.reshape(n, parts, width // parts), eps).reshape(n, width)
    return v * weight


def mamba2(h, w, m, eps):
    """``w``: the mixer's tensors by their short names; ``m``: its sizes."""
    heads, vdim, state, groups = m["heads"], m["vdim"], m["state"], m["groups"]
    inner, gn = heads * vdim, groups * state
    p = np.asarray(h, F64) @ w["in"].T
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * gn], p[:, 2 * inner + 2 * gn:]
    xbc = silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    x, b, c = xbc[:, :inner], xbc[:, inner:inner + gn], xbc[:, inner + gn:]
    dt = softplus(dt + w["dt_bias"])
    y = ssd_scan(x, b, c, dt, w["A_log"], w["D"], heads, vdim, state, groups)
    return gated_group_norm(y, z, w["norm"], m["norm_groups"], eps) @ w["o"].T


# ----------------------------------------------------------------------------- attention
def visible(i: int, j: int, size: int, keep_first: int) -> bool:
    return j <= i and (i - j < size or j < keep_first)


def head_slope(h: int, heads: int) -> float:
    return 2.0 ** (-8.0 * (h + 1) / heads)


def attention_values(h, w, m, v_first):
    """The values of this layer for every token, [T, kv_heads * vdim]: W_v h + b, blended with ``v_first``
    (the values of the first layer that blends) if one is given."""
    v = np.asarray(h, F64) @ w["v"].T + w["v.b"]
    if v_first is not None:
        lam = float(w["vmix"])
        v = (1.0 - lam) * v + lam * v_first
    return v


def attend(q, k, v, m):
    """q [T, heads, dim] and k [T, kv_heads, dim] as they enter the scores, v [T, kv_heads, vdim]: every head's
    softmax-weighted values [T, heads, vdim].  score = cap tanh(q . k scale / cap) - slope_h (i - j) over the keys
    j that position i sees."""
    heads, kv = q.shape[1], k.shape[1]
    size, keep = m["mask"]["size"], m["mask"]["keep_first"]
    scale, cap = m["scale"], m["softcap"]
    n = q.shape[0]
    out = np.zeros((n, heads, v.shape[2]), F64)
    for head in range(heads):
        g = head // (heads // kv)
        slope = head_slope(head, heads)
        for i in range(n):
            js = [j for j in range(i + 1) if visible(i, j, size, keep)]
            s = np.array([q[i, head] @ k[j, g] for j in js]) * scale
            s = cap * np.tanh(s / cap)
            s = s - slope * (i - np.array(js, F64))
            p = np.exp(s - s.max())
            p /= p.sum()
            out[i, head] = p @ v[js, g]
    return out


def attention(h, w, m, eps, v):
    """``v`` from ``attention_values``."""
    heads, kv, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    h = np.asarray(h, F64)
    n = h.shape[0]
    q = unit_rms((h @ w["q"].T + w["q.b"]).reshape(n, heads, dim), eps)
    k = unit_rms((h @ w["k"].T + w["k.b"]).reshape(n, kv, dim), eps)
    gate = sigmoid(h @ w["g"].T)  # [T, heads], one gate a head
    out = attend(q, k, v.reshape(n, kv, vdim), m) * gate[:, :, None]
    return out.reshape(n, heads * vdim) @ w["o"].T


# ----------------------------------------------------------------------------- feed-forward
def dense_ff(h, w):
    u = np.maximum(np.asarray(h, F64) @ w["up"].T, 0.0)
    return (u * u) @ w["down"].T


def expert(h, gate, up, down, limit):
    g = np.minimum(h @ gate.T, limit)
    u = np.clip(h @ up.T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route_margins(h, router, bias, top: int):
    """For every token, how far the last chosen logit lies above the best one that is not chosen (inf if all are)."""
    z = -np.sort(-(np.asarray(h, F64) @ router.T + bias), axis=-1)
    return z[:, top - 1] - z[:, top] if top < z.shape[1] else np.full(z.shape[0], np.inf)


def route(h, router, bias, top: int):
    """([T, top] expert numbers, [T, top] weights): the largest logits, softmax over those alone."""
    z = np.asarray(h, F64) @ router.T + bias
    chosen = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, chosen, axis=-1)
    e = np.exp(zc - zc.max(axis=-1, keepdims=True))
    return chosen, e / e.sum(axis=-1, keepdims=True)


def moe_ff(h, w, mlp):
    h = np.asarray(h, F64)
    chosen, weights = route(h, w["router"], w["router.b"], mlp["router"]["top"])
    out = np.zeros((h.shape[0], w["e0.down"].shape[0]), F64)
    for t in range(h.shape[0]):
        for e, p in zip(chosen[t], weights[t]):
            out[t] += p * expert(h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], mlp["expert"]["limit"])
    return out


# ----------------------------------------------------------------------------- the model
def _sub(tensors, prefix):
    return {k[len(prefix):]: np.asarray(v, F64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, layers_out=None, margins_out=None):
    """Logits [T, vocab] of one whole sequence.  ``layers_out``: a list that receives the stream after every layer;
    ``margins_out``: a list that receives every routed layer's ``route_margins``."""
    eps = config["norm"]["eps"]
    bg = config["embedding"]["bigram"]
    x = embed(tokens, tensors["embed"], tensors["bigram"], bg["buckets"], bg["mul_prev"], bg["mul_cur"])
    v_first = None
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."

        def ln(name, value):
            return layer_norm(value, tensors[p + name], tensors[p + name + ".b"], eps)

        h = ln("norm1", x)
        w = _sub(tensors, p + "mix.")
        if layer["type"] == "mamba2":
            y = mamba2(h, w, layer["mixer"], eps)
        elif layer["type"] == "attention":
            m = layer["mixer"]
            v = attention_values(h, w, m, v_first if m.get("v_mix") else None)
            if m.get("v_mix") and v_first is None:
                v_first = v
            y = attention(h, w, m, eps, v)
        else:
            raise ValueError(layer["type"])
        x = x + ln("norm1b", y)
        if layer.get("mlp"):
            h = ln("norm2", x)
            w = _sub(tensors, p + "mlp.")
            y = dense_ff(h, w) if layer["mlp"]["kind"] == "dense" else moe_ff(h, w, layer["mlp"])
            if margins_out is not None and layer["mlp"]["kind"] == "moe":
                margins_out.append(route_margins(h, w["router"], w["router.b"], layer["mlp"]["router"]["top"]))
            x = x + ln("norm2b", y)
        if layers_out is not None:
            layers_out.append(x.copy())
    x = layer_norm(x, tensors["final.norm"], tensors["final.norm.b"], eps)
    return x @ np.asarray(tensors["embed"], F64).T
