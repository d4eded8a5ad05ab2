"""A plain, slow implementation of the Bamasun design: numpy, float64, whole sequences, no cache.

One function per mechanism, written from the design's equations; nothing here is shared with the
engine.  ``forward`` takes the configuration as the dictionary that config.json holds and the weights
as a dictionary of arrays by checkpoint name.

Notation.  x is the residual stream [T, width].  A layer does x <- x + LN1(mixer(x)) and then, if it has a
feed-forward, x <- x + LN2(ff(x)): the sublayers read x itself and the norm sits on their output.
"""
from __future__ import annotations

import math

import numpy as np


def layer_norm(x, weight, bias, eps):
    """(x - mean) / sqrt(var + eps) * weight + bias, var the mean of the squared deviations."""
    x = np.asarray(x, dtype=np.float64)
    mean = x.mean(axis=-1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
    return (x - mean) / np.sqrt(var + eps) * weight + bias


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight, the weight used as it is."""
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * weight


def embed(tokens, table, scale):
    return np.asarray(table, dtype=np.float64)[np.asarray(tokens)] * scale


def query_temperature(position, coef, every):
    """The factor on the query at ``position``: 1 + coef * ln(floor((position + 1) / every) + 1)."""
    return 1.0 + coef * math.log(math.floor((position + 1) / every) + 1.0)


def distance_slopes(num_heads):
    """slope of head h (0-based) = 2^(-8 (h + 1) / H)."""
    return np.array([2.0 ** (-8.0 * (h + 1) / num_heads) for h in range(num_heads)], dtype=np.float64)


def softmax_rows(s):
    s = s - s.max(axis=-1, keepdims=True)
    e = np.exp(s)
    return e / e.sum(axis=-1, keepdims=True)


def attention_keys_values(h, w, prefix, mixer, eps):
    """Keys after the norm over the whole projection, and values, as a cache would hold them:
    k [T, G, dim], v [T, G, vdim]."""
    G, dim, vdim = mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    k = h @ w[prefix + "k"].T + w[prefix + "k.b"]
    v = h @ w[prefix + "v"].T + w[prefix + "v.b"]
    k = rms_norm(k, w[prefix + "k.norm"], eps)
    return k.reshape(-1, G, dim), v.reshape(-1, G, vdim)


def attention_mixer(h, w, prefix, mixer, eps, keys_values=None):
    """Causal softmax attention with grouped heads, a norm over the whole q (and k) projection, a query
    temperature by position and a bias of -slope_h * (i - j) on the scores; no rotation.
    ``keys_values`` are another layer's (k, v) when this layer has none of its own."""
    T = h.shape[0]
    H, G, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    q = h @ w[prefix + "q"].T + w[prefix + "q.b"]
    q = rms_norm(q, w[prefix + "q.norm"], eps)
    temp = mixer.get("q_temp")
    if temp:
        factors = np.array([query_temperature(p, temp["coef"], temp["every"]) for p in range(T)])
        q = q * factors[:, None]
    q = q.reshape(T, H, dim)
    if keys_values is None:
        keys_values = attention_keys_values(h, w, prefix, mixer, eps)
    k, v = keys_values
    slopes = distance_slopes(H)
    out = np.zeros((T, H, vdim))
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * mixer["scale"] - slopes[head] * (i - j)
        s = np.where(j <= i, s, -np.inf)
        out[:, head] = softmax_rows(s) @ v[:, g]
    return out.reshape(T, H * vdim) @ w[prefix + "o"].T, keys_values


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gla_mixer(h, w, prefix, mixer, eps, state=None):
    """Gated linear attention, token by token: per head S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t, with
    alpha = sigmoid(z)^(1/tau) per key channel, z = W_a2 (W_a1 h) + b; each head's o is RMS-normed over vdim
    with one weight for all heads; the heads side by side are gated by silu(W_g h) and projected."""
    T = h.shape[0]
    H, dim, vdim, tau = mixer["heads"], mixer["dim"], mixer["vdim"], mixer["tau"]
    q = (h @ w[prefix + "q"].T).reshape(T, H, dim) * dim ** -0.5
    k = (h @ w[prefix + "k"].T).reshape(T, H, dim)
    v = (h @ w[prefix + "v"].T).reshape(T, H, vdim)
    gate = silu(h @ w[prefix + "g"].T)
    z = (h @ w[prefix + "a1"].T) @ w[prefix + "a2"].T + w[prefix + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / tau)).reshape(T, H, dim)
    S = np.zeros((H, dim, vdim)) if state is None else state.copy()
    o = np.zeros((T, H, vdim))
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hd,hdv->hv", q[t], S)
    o = rms_norm(o, w[prefix + "norm"], eps)
    return (o.reshape(T, H * vdim) * gate) @ w[prefix + "o"].T, S


def dense_feed_forward(h, w, prefix):
    """W_down relu(W_up h)^2."""
    up = np.maximum(h @ w[prefix + "up"].T, 0.0)
    return (up * up) @ w[prefix + "down"].T


def softcap(logits, cap):
    return cap * np.tanh(logits / cap)


def forward(config, weights, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence run whole; with ``return_layers`` also the stream after every layer."""
    w = {name: np.asarray(value, dtype=np.float64) for name, value in weights.items()}
    eps = config["norm"]["eps"]
    x = embed(tokens, w["embed"], config["embedding"]["scale"])
    kept = {}
    after = []
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        mixer = layer["mixer"]
        if layer["type"] == "attention":
            source = mixer.get("kv_from")
            update, kv = attention_mixer(x, w, p + "mix.", mixer, eps, kept[source] if source is not None else None)
            kept[index] = kv
        elif layer["type"] == "gla":
            update, _ = gla_mixer(x, w, p + "mix.", mixer, eps)
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        x = x + layer_norm(update, w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"feed-forward kind {layer['mlp']['kind']!r}")
            x = x + layer_norm(dense_feed_forward(x, w, p + "mlp."), w[p + "norm2"], w[p + "norm2.b"], eps)
        after.append(x.copy())
    logits = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = softcap(logits, cap)
    return (logits, np.stack(after)) if return_layers else logits
