"""A plain, slow implementation of the Fotanex design: numpy, float64, whole sequences, no cache, one function per
mechanism.  It shares no code with the library; the tests compare the engine against it.

A model is (config, tensors): ``config`` is the dictionary that config.json holds and ``tensors`` maps tensor names
to float64 arrays.  Linear weights are [out, in] and applied as W x.

    layer:      x <- x + mixer(dyt1(x)) + experts(dyt2(x))                    both norms read the same x
    dyt:        tanh(alpha v) * w + b                                          (no statistics)
    loop:       layers start..stop-1 run ``times`` times; before pass t:  x <- W_in [x ; x0] + step[t]
    mixers:     rglru | mamba2 | parallel (chunked attention with sink and head gate, beside a selective scan)
"""
from __future__ import annotations

import numpy as np


def sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


def silu(v):
    return v * sigmoid(v)


def softplus(v):
    return np.logaddexp(0.0, v)


def gelu_tanh(v):
    return 0.5 * v * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (v + 0.044715 * v ** 3)))


def dynamic_tanh(v, weight, bias, alpha):
    return np.tanh(float(alpha) * v) * weight + bias


def rms_divide(v, eps):
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps)


def causal_conv(v, taps, bias):
    """v [T, C]; taps [C, K], the last column weighs the current token; zeros before the first token."""
    count, width = taps.shape[0], taps.shape[1]
    padded = np.concatenate([np.zeros((width - 1, count)), v], axis=0)
    out = np.zeros_like(v)
    for t in range(v.shape[0]):
        out[t] = bias + np.sum(padded[t:t + width].T * taps, axis=1)
    return out


def chunked_sink_attention(h, q_w, k_w, v_w, sink, gate_w, o_w, *, heads, kv_heads, dim, vdim, scale, chunk):
    """Softmax attention whose query at i sees j <= i of its own chunk (i // chunk == j // chunk), without positions
    in the scores; the denominator also holds exp(sink_h); head h's output times sigmoid(gate_w h)_h."""
    count = h.shape[0]
    q = (h @ q_w.T).reshape(count, heads, dim)
    k = (h @ k_w.T).reshape(count, kv_heads, dim)
    v = (h @ v_w.T).reshape(count, kv_heads, vdim)
    out = attend_in_chunks(q, k, v, sink, h @ gate_w.T, scale, chunk)
    return out.reshape(count, heads * vdim) @ o_w.T


def attend_in_chunks(q, k, v, sink, gate_logits, scale, chunk, positions=None):
    """q [R, heads, dim] at ``positions`` (default: row r is position r) over k [T, G, dim], v [T, G, vdim];
    ``sink`` [heads] or None; ``gate_logits`` [R, heads] or None; ``chunk`` None: every earlier key."""
    rows, heads = q.shape[0], q.shape[1]
    per = heads // k.shape[1]
    out = np.zeros((rows, heads, v.shape[2]))
    for r in range(rows):
        i = r if positions is None else int(positions[r])
        first = (i // chunk) * chunk if chunk else 0
        for head in range(heads):
            g = head // per
            scores = (k[first:i + 1, g] @ q[r, head]) * scale
            top = scores.max() if sink is None else max(scores.max(), sink[head])
            weights = np.exp(scores - top)
            denom = weights.sum() + (np.exp(sink[head] - top) if sink is not None else 0.0)
            out[r, head] = (weights / denom) @ v[first:i + 1, g]
            if gate_logits is not None:
                out[r, head] *= sigmoid(gate_logits[r, head])
    return out


def selective_scan(h, in_w, conv_w, conv_b, x_w, dt_w, dt_b, a_log, d, o_w, *, inner, state, dt_rank):
    """Mamba: a state [inner, state] per sequence with a decay and an input that depend on the token."""
    both = h @ in_w.T
    x, z = both[:, :inner], both[:, inner:]
    x = silu(causal_conv(x, conv_w, conv_b))
    low = x @ x_w.T
    dt = softplus(low[:, :dt_rank] @ dt_w.T + dt_b)                # [T, inner]
    b, c = low[:, dt_rank:dt_rank + state], low[:, dt_rank + state:]
    return (selective_recurrence(x, dt, b, c, a_log, d) * silu(z)) @ o_w.T


def selective_recurrence(x, dt, b, c, a_log, d):
    """x, dt [T, inner]; b, c [T, state]; a_log [inner, state]; d [inner] -> y [T, inner], from a zero state."""
    a = -np.exp(a_log)
    s = np.zeros(a_log.shape)
    y = np.zeros_like(x)
    for t in range(x.shape[0]):
        s = np.exp(dt[t][:, None] * a) * s + (dt[t] * x[t])[:, None] * b[t][None, :]
        y[t] = s @ c[t] + d * x[t]
    return y


def parallel_mixer(h, left, right, left_norm, right_norm, eps):
    """Half the sum of two mixers' outputs, each first divided by its root mean square over the model width and
    multiplied by its weight."""
    return 0.5 * (rms_divide(left, eps) * left_norm + rms_divide(right, eps) * right_norm)


def rglru(h, y_w, y_b, x_w, x_b, conv_w, conv_b, ra, ra_b, ri, ri_b, lam, o_w, *, blocks):
    """The recurrent block with a real-gated linear recurrent unit."""
    y = gelu_tanh(h @ y_w.T + y_b)
    u = causal_conv(h @ x_w.T + x_b, conv_w, conv_b)
    count, width = u.shape
    part = width // blocks
    r = np.zeros_like(u)
    i = np.zeros_like(u)
    for b in range(blocks):
        cols = slice(b * part, (b + 1) * part)
        r[:, cols] = sigmoid(u[:, cols] @ ra[b].T + ra_b[b])
        i[:, cols] = sigmoid(u[:, cols] @ ri[b].T + ri_b[b])
    return (gated_recurrence(u, r, i, lam) * y) @ o_w.T


def gated_recurrence(u, r, i, lam, constant=8.0):
    """u, r, i [T, width] (the gates after their sigmoids), lam [width] -> the states [T, width], from zero."""
    a = np.exp(-constant * r * softplus(lam))
    s = np.zeros(u.shape[1])
    out = np.zeros_like(u)
    for t in range(u.shape[0]):
        s = a[t] * s + np.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = s
    return out


def mamba2(h, in_w, conv_w, conv_b, dt_bias, a_log, d, norm_w, o_w, *, heads, vdim, state, groups, norm_groups, eps):
    """State-space duality form: a state [state, vdim] per head with one decay per head and token."""
    inner = heads * vdim
    proj = h @ in_w.T
    z = proj[:, :inner]
    xbc = silu(causal_conv(proj[:, inner:2 * inner + 2 * groups * state], conv_w, conv_b))
    dt = softplus(proj[:, 2 * inner + 2 * groups * state:] + dt_bias)      # [T, heads]
    x = xbc[:, :inner].reshape(-1, heads, vdim)
    b = xbc[:, inner:inner + groups * state].reshape(-1, groups, state)
    c = xbc[:, inner + groups * state:].reshape(-1, groups, state)
    y = state_space_recurrence(x, b, c, dt, a_log, d).reshape(-1, inner) * silu(z)
    return group_rms(y, norm_w, norm_groups, eps) @ o_w.T


def state_space_recurrence(x, b, c, dt, a_log, d):
    """x [T, heads, vdim]; b, c [T, groups, state]; dt [T, heads]; a_log, d [heads] -> y [T, heads, vdim], from zero."""
    heads, vdim = x.shape[1], x.shape[2]
    per = heads // b.shape[1]
    s = np.zeros((heads, b.shape[2], vdim))
    y = np.zeros_like(x)
    for t in range(x.shape[0]):
        for head in range(heads):
            g = head // per
            s[head] = np.exp(-np.exp(a_log[head]) * dt[t, head]) * s[head] + dt[t, head] * np.outer(b[t, g], x[t, head])
            y[t, head] = s[head].T @ c[t, g] + d[head] * x[t, head]
    return y


def group_rms(y, weight, parts, eps):
    """Rows in ``parts`` equal parts, each divided by its own root mean square, times the weight."""
    return rms_divide(y.reshape(y.shape[0], parts, -1), eps).reshape(y.shape) * weight


def routed_experts(h, router_w, experts, top, forced=None):
    """``experts``: list of (gate, up, down).  Softmax over all experts, the ``top`` largest, their scores divided by
    their sum (+ 1e-20).  ``forced`` [T, top] names the experts to use instead of the largest.  Returns the output,
    the experts used and, per token, the gap between the last score taken and the first one left out."""
    logits = h @ router_w.T
    scores = np.exp(logits - logits.max(axis=-1, keepdims=True))
    scores /= scores.sum(axis=-1, keepdims=True)
    out = np.zeros_like(h)
    picked = np.zeros((h.shape[0], top), dtype=np.int64)
    ranked = -np.sort(-scores, axis=-1)
    margins = ranked[:, top - 1] - ranked[:, top] if top < scores.shape[1] else np.full(h.shape[0], np.inf)
    for t in range(h.shape[0]):
        order = np.argsort(-scores[t], kind="stable")[:top] if forced is None else np.asarray(forced[t], dtype=np.int64)
        picked[t] = order
        weights = scores[t, order] / (scores[t, order].sum() + 1e-20)
        for e, w in zip(order, weights):
            gate, up, down = experts[e]
            out[t] += w * (down @ (silu(gate @ h[t]) * (up @ h[t])))
    return out, picked, margins


# ---------------------------------------------------------------------------------------------------- the model

def _norm(tensors, name, v):
    return dynamic_tanh(v, tensors[name], tensors[name + ".b"], tensors[name + ".alpha"])


def mixer_of(config, tensors, index, h):
    layer = config["layers"][index]
    m = layer["mixer"]
    p = f"l{index}.mix."
    eps = config["norm"]["eps"]
    kind = layer["type"]
    if kind == "rglru":
        return rglru(h, tensors[p + "y"], tensors[p + "y.b"], tensors[p + "x"], tensors[p + "x.b"], tensors[p + "conv"],
                     tensors[p + "conv.b"], tensors[p + "ra"], tensors[p + "ra.b"], tensors[p + "ri"], tensors[p + "ri.b"],
                     tensors[p + "lam"], tensors[p + "o"], blocks=m["blocks"])
    if kind == "mamba2":
        return mamba2(h, tensors[p + "in"], tensors[p + "conv"], tensors[p + "conv.b"], tensors[p + "dt_bias"],
                      tensors[p + "A_log"], tensors[p + "D"], tensors[p + "norm"], tensors[p + "o"], heads=m["heads"],
                      vdim=m["vdim"], state=m["state"], groups=m["groups"], norm_groups=m["norm_groups"], eps=eps)
    if kind == "parallel":
        a, s = m["left"], m["right"]
        left = chunked_sink_attention(h, tensors[p + "left.q"], tensors[p + "left.k"], tensors[p + "left.v"],
                                      tensors[p + "left.sink"], tensors[p + "left.g"], tensors[p + "left.o"],
                                      heads=a["heads"], kv_heads=a["kv_heads"], dim=a["dim"], vdim=a["vdim"],
                                      scale=a["scale"], chunk=a["mask"]["size"])
        right = selective_scan(h, tensors[p + "right.in"], tensors[p + "right.conv"], tensors[p + "right.conv.b"],
                               tensors[p + "right.x"], tensors[p + "right.dt"], tensors[p + "right.dt.b"],
                               tensors[p + "right.A_log"], tensors[p + "right.D"], tensors[p + "right.o"],
                               inner=s["inner"], state=s["state"], dt_rank=s["dt_rank"])
        return parallel_mixer(h, left, right, tensors[p + "left.out"], tensors[p + "right.out"], eps)
    raise ValueError(f"layer type {kind!r}")


def feed_forward_of(config, tensors, index, h, picks=None, forced=None):
    """``picks`` (a list) receives (experts used, margins) of this run; ``forced`` (a list) gives up its first entry."""
    mlp = config["layers"][index]["mlp"]
    if mlp is None:
        return np.zeros_like(h)
    p = f"l{index}.mlp."
    count = mlp["router"]["experts"]
    experts = [(tensors[f"{p}e{e}.gate"], tensors[f"{p}e{e}.up"], tensors[f"{p}e{e}.down"]) for e in range(count)]
    out, picked, margins = routed_experts(h, tensors[p + "router"], experts, mlp["router"]["top"],
                                          forced.pop(0) if forced is not None else None)
    if picks is not None:
        picks.append((picked, margins))
    return out


def run_order(config):
    """Layer indices in the order they run, and for each run the number of the pass it opens (None: it opens none)."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(count)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(start)]
    for t in range(times):
        order += [(i, t if i == start else None) for i in range(start, stop)]
    order += [(i, None) for i in range(stop, count)]
    return order


def forward(config, tensors, tokens, layers_out=None, picks=None, forced=None):
    """Logits [T, vocab] of one sequence.  ``layers_out`` (a list) receives the stream after every layer run,
    ``picks`` the experts of every run that has some; ``forced`` lists, in that order, the experts to use instead."""
    forced = list(forced) if forced is not None else None
    x0 = tensors["embed"][np.asarray(tokens)]
    x = x0.copy()
    for index, opens in run_order(config):
        if opens is not None:
            x = np.concatenate([x, x0], axis=1) @ tensors["loop.in"].T + tensors["loop.step"][opens]
        update = mixer_of(config, tensors, index, _norm(tensors, f"l{index}.norm1", x))
        if config["layers"][index]["mlp"] is not None:
            update = update + feed_forward_of(config, tensors, index, _norm(tensors, f"l{index}.norm2", x), picks, forced)
        x = x + update
        if layers_out is not None:
            layers_out.append(x.copy())
    return _norm(tensors, "final.norm", x) @ tensors["head"].T


def greedy(config, tensors, prompt, new_tokens):
    tokens = list(prompt)
    for _ in range(new_tokens):
        tokens.append(int(np.argmax(forward(config, tensors, tokens)[-1])))
    return tokens[len(prompt):]
