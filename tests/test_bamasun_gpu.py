"""The Bamasun design in the engine against the plain implementation of ``plain_bamasun``: each mechanism's kernel
alone, then whole models through the step function, the cache, recorded decode steps and the entry point."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import fieldrun_b200 as fr
import plain_bamasun as pb
from bamasun_configs import ALL, model_folder, plain_weights, request_tokens

pytestmark = pytest.mark.gpu

DEV = "cuda"
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
KERNEL_TOL = {"float32": 5e-6, "bfloat16": 1.2e-2}
# see model_close.  The norms on the sublayers' outputs divide by the spread of an update, so bfloat16 rounding of a
# small update comes back at full size: single rows of these tiny models are 0.12 off, the same rows however the
# tokens are cut into steps.  Faults of the cache, the state or a mask show in float32, where the limit is 3e-5.
MODEL_TOL = {"float32": 3e-5, "bfloat16": 3e-1}
BF16_MOST_ROWS = 5e-2        # nine rows in ten are within this


def ops():
    from fieldrun_b200.csrc import ops as o
    return o


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(DEV).contiguous()


def f64(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def rounded(a, dtype):
    """The values as the device holds them in ``dtype``."""
    return f64(torch.as_tensor(np.asarray(a, dtype=np.float32)).to(TORCH[dtype]))


def close(got, ref, tol, what=""):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), what
    err = np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30)
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol:.1e}"


# ------------------------------------------------------------------------------------------- mechanisms alone

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [40, 257, 3000])
def test_layer_norm_on_the_stream_and_on_an_update(dtype, width):
    rng = np.random.default_rng(width)
    rows = 37
    update = rng.normal(size=(rows, width)) * 3.0 + 1.5
    stream = rng.normal(size=(rows, width))
    w, b = 1.0 + 0.3 * rng.normal(size=width), 0.5 * rng.normal(size=width)
    eps = 1e-3
    # on the stream, with a choice of rows
    pick = np.array([5, 0, 36, 5], dtype=np.int32)
    out = torch.empty((len(pick), width), dtype=TORCH[dtype], device=DEV)
    ops().layernorm(dev(update, torch.float32), dev(w, torch.float32), dev(b, torch.float32), eps, rows=dev(pick), act=out)
    close(f64(out), pb.layer_norm(update[pick].astype(np.float32), w.astype(np.float32), b.astype(np.float32), eps),
          KERNEL_TOL[dtype], "norm of chosen rows")
    # on an update: the stream grows by the normed update and its typed copy follows
    x = dev(stream, torch.float32)
    act = torch.empty((rows, width), dtype=TORCH[dtype], device=DEV)
    ops().layernorm(dev(update, torch.float32), dev(w, torch.float32), dev(b, torch.float32), eps, stream=x, act=act)
    want = stream.astype(np.float32) + pb.layer_norm(update.astype(np.float32), w.astype(np.float32), b.astype(np.float32), eps)
    close(f64(x), want, 5e-6, "stream after the update")
    close(f64(act), want, KERNEL_TOL[dtype], "typed copy of the stream")
    # without a bias
    ops().layernorm(dev(update, torch.float32), dev(w, torch.float32), None, eps, act=act)
    close(f64(act), pb.layer_norm(update.astype(np.float32), w.astype(np.float32), 0.0, eps), KERNEL_TOL[dtype], "no bias")


def test_a_constant_row_norms_to_its_bias():
    width = 64
    x = dev(np.full((2, width), 7.25), torch.float32)
    out = torch.empty((2, width), dtype=torch.float32, device=DEV)
    b = np.linspace(-1, 1, width)
    ops().layernorm(x, dev(np.ones(width), torch.float32), dev(b, torch.float32), 1e-6, act=out)
    close(f64(out), np.broadcast_to(b, (2, width)), 1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_scale_and_typed_copy(dtype):
    rng = np.random.default_rng(1)
    table = dev(rng.normal(size=(50, 36)), TORCH[dtype])
    tokens = np.array([3, 49, 0, 3], dtype=np.int32)
    x = torch.empty((4, 36), dtype=torch.float32, device=DEV)
    act = torch.empty((4, 36), dtype=TORCH[dtype], device=DEV)
    ops().embed_rows(dev(tokens), table, x, 2.5, act)
    close(f64(x), pb.embed(tokens, f64(table), 2.5), 1e-7)
    close(f64(act), pb.embed(tokens, f64(table), 2.5), KERNEL_TOL[dtype])


def test_activations_and_logit_cap():
    z = np.linspace(-6, 6, 1001).reshape(7, 143)
    out = torch.empty((7, 143), dtype=torch.float32, device=DEV)
    ops().unary_unit(dev(z, torch.float32), out, "relu_squared")
    close(f64(out), np.maximum(z, 0) ** 2, 1e-6)
    ops().unary_unit(dev(z, torch.float32), out, "gelu_tanh")
    close(f64(out), 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3))), 1e-6)
    ops().unary_unit(dev(z, torch.float32), out, "silu")
    close(f64(out), pb.silu(z), 1e-6)
    logits = dev(z * 20, torch.float32)
    ops().softcap(logits, 30.0)
    close(f64(logits), pb.softcap(z * 20, 30.0), 1e-6)


@pytest.mark.parametrize("rows,inner,features", [(300, 128, 256), (64, 64, 128), (1000, 192, 384), (257, 256, 1024)])
@pytest.mark.parametrize("activation", ["relu_squared", "gelu_tanh", "silu"])
def test_first_product_of_a_dense_unit_with_its_activation_on_tcgen05(rows, inner, features, activation):
    """The whole step as one expert's rows in tiles: act(x W^T) rounded once to bfloat16."""
    rng = np.random.default_rng(rows + features)
    x = dev(rng.normal(size=(rows, inner)), torch.bfloat16)
    w = dev(rng.normal(size=(features, inner)) * inner ** -0.5, torch.bfloat16)
    z = f64(x) @ f64(w).T
    want = {"relu_squared": np.maximum(z, 0) ** 2, "silu": pb.silu(z),
            "gelu_tanh": 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3)))}[activation]
    for tile_rows in (32, 64, 128, 256):
        count = (rows + tile_rows - 1) // tile_rows
        out = torch.full((rows, features), 7.0, dtype=torch.bfloat16, device=DEV)
        ops().expert_gemm_tc(w.view(1, features, inner), x, dev(np.zeros(count, dtype=np.int32)),
                             dev((np.arange(count) * tile_rows).astype(np.int32)), dev(np.array([count], dtype=np.int32)),
                             dev(np.array([0, rows], dtype=np.int32)), count, tile_rows, out, paired=False, activation=activation)
        ops().tc_status_check(DEV)
        close(f64(out), want, 1.2e-2, f"tiles of {tile_rows}")


def scrambled_pages(rng, slots, lengths, kv_heads, dim, vdim, dtype, spare=3):
    """Keys [slot][T, G, dim], values [slot][T, G, vdim] laid into pages in a scrambled order."""
    per = [(n + 63) // 64 for n in lengths]
    pages = sum(per) + spare
    order = rng.permutation(pages)
    table = np.full((slots, max(per) + 1), -1, dtype=np.int32)
    kc = np.zeros((pages, kv_heads, 64, dim))
    vc = np.zeros((pages, kv_heads, vdim, 64))
    keys, values = [], []
    at = 0
    for s, n in enumerate(lengths):
        k = rounded(rng.normal(size=(n, kv_heads, dim)), dtype)
        v = rounded(rng.normal(size=(n, kv_heads, vdim)), dtype)
        keys.append(k)
        values.append(v)
        for i in range(per[s]):
            page = order[at]
            at += 1
            table[s, i] = page
            chunk = slice(64 * i, min(64 * i + 64, n))
            kc[page, :, :chunk.stop - chunk.start] = k[chunk].transpose(1, 0, 2)
            vc[page, :, :, :chunk.stop - chunk.start] = v[chunk].transpose(1, 2, 0)
    return keys, values, kc, vc, table


def plain_scores_attention(q, keys, values, position, heads, scale, slopes):
    """One query [heads, dim] at ``position`` over keys [T, G, dim] and values [T, G, vdim], keys 0..position."""
    G = keys.shape[1]
    out = np.zeros((heads, values.shape[2]))
    j = np.arange(position + 1)
    for h in range(heads):
        g = h // (heads // G)
        s = keys[:position + 1, g] @ q[h] * scale - slopes[h] * (position - j)
        out[h] = pb.softmax_rows(s[None])[0] @ values[:position + 1, g]
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(6, 2, 32, 16), (3, 3, 24, 40), (8, 1, 64, 64), (2, 1, 100, 7)])
def test_attention_with_distance_slopes_and_value_size(dtype, heads, kv_heads, dim, vdim):
    rng = np.random.default_rng(heads * 100 + dim)
    lengths = [200, 64, 65, 1]
    keys, values, kc, vc, table = scrambled_pages(rng, 4, lengths, kv_heads, dim, vdim, dtype)
    slopes = pb.distance_slopes(heads)
    # queries: every position of the short sequences, some of the long one (page borders among them)
    rows = [(0, p) for p in (0, 1, 62, 63, 64, 65, 127, 128, 199)] + [(1, p) for p in (0, 63)] + [(2, 64)] + [(3, 0)]
    q = rounded(rng.normal(size=(len(rows), heads, dim)), dtype)
    out = torch.empty((len(rows), heads * vdim), dtype=TORCH[dtype], device=DEV)
    ops().attention_generic(dev(q, TORCH[dtype]), dev(kc, TORCH[dtype]), dev(vc, TORCH[dtype]), dev(table),
                            dev(np.array([p for _, p in rows], dtype=np.int32)), dev(np.array([s for s, _ in rows], dtype=np.int32)),
                            out, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, scale=0.17, window=None, v_dim=vdim,
                            slopes=dev(slopes, torch.float32))
    want = np.stack([plain_scores_attention(q[r], keys[s], values[s], p, heads, 0.17, slopes).reshape(-1)
                     for r, (s, p) in enumerate(rows)])
    close(f64(out), want, KERNEL_TOL[dtype], "attention")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_weighs_a_far_key_by_its_distance(dtype):
    """One key hundreds of positions back is made to stand out; what it gets is exp(score - slope * distance)
    against the near keys, head by head: a slope that is left out, taken with the wrong sign or of the wrong head
    changes the result by whole units."""
    rng = np.random.default_rng(11)
    heads, kv_heads, dim, vdim, n = 4, 2, 32, 8, 700
    keys, values, kc, vc, table = scrambled_pages(rng, 1, [n], kv_heads, dim, vdim, dtype)
    q = rounded(rng.normal(size=(1, heads, dim)) * 0.1, dtype)
    far = 13
    for g in range(kv_heads):
        keys[0][far, g] = rounded(q[0, g * 2] * 40.0, dtype)          # a large score for the first head of each group
        values[0][far, g] = 50.0
    page, place = table[0, far // 64], far % 64
    kc[page, :, place] = keys[0][far]
    vc[page, :, :, place] = values[0][far]
    slopes = pb.distance_slopes(heads)
    out = torch.empty((1, heads * vdim), dtype=TORCH[dtype], device=DEV)
    ops().attention_generic(dev(q, TORCH[dtype]), dev(kc, TORCH[dtype]), dev(vc, TORCH[dtype]), dev(table),
                            dev(np.array([n - 1], dtype=np.int32)), dev(np.array([0], dtype=np.int32)), out, num_heads=heads,
                            num_kv_heads=kv_heads, head_dim=dim, scale=1.0, window=None, v_dim=vdim,
                            slopes=dev(slopes, torch.float32))
    want = plain_scores_attention(q[0], keys[0], values[0], n - 1, heads, 1.0, slopes).reshape(1, -1)
    without = plain_scores_attention(q[0], keys[0], values[0], n - 1, heads, 1.0, np.zeros(heads)).reshape(1, -1)
    assert np.abs(want - without).max() > 5.0, "the case does not show the slopes"
    close(f64(out), want, KERNEL_TOL[dtype], "far key")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,temp", [(6, 2, 32, 16, (0.5, 7)), (3, 3, 20, 28, None), (5, 1, 9, 3, (1.0, 1))])
def test_projection_bias_whole_row_norm_temperature_and_cache_write(dtype, heads, kv_heads, dim, vdim, temp):
    rng = np.random.default_rng(dim)
    positions = np.array([0, 5, 6, 7, 13, 14, 63, 64, 200], dtype=np.int32)
    T = len(positions)
    widths = (heads * dim, kv_heads * dim, kv_heads * vdim)
    rows = rng.normal(size=(T, sum(widths))).astype(np.float32)
    bias = rng.normal(size=sum(widths)).astype(np.float32)
    qw, kw = (1 + 0.2 * rng.normal(size=widths[0])).astype(np.float32), (1 + 0.2 * rng.normal(size=widths[1])).astype(np.float32)
    table = np.array([[2, 0, 3, 1]], dtype=np.int32)
    kc = torch.zeros((4, kv_heads, 64, dim), dtype=TORCH[dtype], device=DEV)
    vc = torch.zeros((4, kv_heads, vdim, 64), dtype=TORCH[dtype], device=DEV)
    q = torch.empty((T, widths[0]), dtype=TORCH[dtype], device=DEV)
    ops().qkv_prepare(dev(rows), dev(qw), dev(kw), 1e-4, None, None, dev(positions), dev(np.zeros(T, dtype=np.int32)), dev(table), q,
                      kc, vc, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, rotary_dim=0, interleaved=False,
                      write_cache=True, bias=dev(bias), v_dim=vdim, q_temp=temp)
    full = rows.astype(np.float64) + bias
    factors = np.array([pb.query_temperature(int(p), *temp) if temp else 1.0 for p in positions])
    close(f64(q), pb.rms_norm(full[:, :widths[0]], qw, 1e-4) * factors[:, None], KERNEL_TOL[dtype], "queries")
    want_k = pb.rms_norm(full[:, widths[0]:widths[0] + widths[1]], kw, 1e-4).reshape(T, kv_heads, dim)
    want_v = full[:, widths[0] + widths[1]:].reshape(T, kv_heads, vdim)
    got_k, got_v = f64(kc), f64(vc)
    for t, p in enumerate(positions):
        page, place = table[0, p // 64], p % 64
        close(got_k[page, :, place], want_k[t], KERNEL_TOL[dtype], f"key at {p}")
        close(got_v[page, :, :, place], want_v[t], KERNEL_TOL[dtype], f"value at {p}")
    # a layer without keys and values of its own: the row is the queries alone and the cache stays as it is
    before = kc.clone()
    ops().qkv_prepare(dev(rows[:, :widths[0]].copy()), dev(qw), None, 1e-4, None, None, dev(positions),
                      dev(np.zeros(T, dtype=np.int32)), dev(table), q, kc, vc, num_heads=heads, num_kv_heads=0, head_dim=dim,
                      rotary_dim=0, interleaved=False, write_cache=False, bias=dev(bias[:widths[0]].copy()), v_dim=vdim, q_temp=temp)
    close(f64(q), pb.rms_norm(full[:, :widths[0]], qw, 1e-4) * factors[:, None], KERNEL_TOL[dtype], "queries alone")
    assert torch.equal(before, kc)


def gla_case(rng, heads, dim, vdim, rank, width, tau, bias_shift):
    w = {"q": rng.normal(size=(heads * dim, width)) * 0.3, "k": rng.normal(size=(heads * dim, width)) * 0.3,
         "v": rng.normal(size=(heads * vdim, width)) * 0.3, "g": rng.normal(size=(heads * vdim, width)) * 0.3,
         "a1": rng.normal(size=(rank, width)) * 0.3, "a2": rng.normal(size=(heads * dim, rank)) * 0.5,
         "a2.b": rng.normal(size=heads * dim) + bias_shift, "norm": 1 + 0.2 * rng.normal(size=vdim),
         "o": np.eye(heads * vdim)}
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}
    return {"m." + k: v for k, v in w.items()}, mixer


@pytest.mark.parametrize("heads,dim,vdim,rank,tau,shift", [(2, 16, 24, 5, 4.0, 0.0), (3, 8, 8, 3, 1.0, -3.0), (1, 100, 33, 2, 16.0, 4.0),
                                                          (2, 128, 128, 16, 16.0, 2.0), (1, 200, 40, 4, 2.0, 0.0),
                                                          # states too large for one block: value columns in slices over blocks
                                                          (1, 130, 200, 9, 32.0, 1.0), (2, 256, 300, 4, 4.0, 0.0)])
def test_gated_linear_attention_scan_with_state_carried_between_calls(heads, dim, vdim, rank, tau, shift):
    rng = np.random.default_rng(dim + vdim)
    width = 48
    w, mixer = gla_case(rng, heads, dim, vdim, rank, width, tau, shift)
    lengths = [70, 1, 33]
    h = [rng.normal(size=(n, width)) for n in lengths]
    want, states = zip(*[pb.gla_mixer(x, w, "m.", mixer, 1e-5) for x in h])
    w_in = dev(np.concatenate([w["m.q"], w["m.k"], w["m.v"], w["m.g"], w["m.a1"]]), torch.float32)
    offsets = (0, heads * dim, 2 * heads * dim, 2 * heads * dim + heads * vdim, 2 * heads * dim + 2 * heads * vdim)
    state = torch.zeros((5, 2, heads, dim, vdim), dtype=torch.float32, device=DEV)
    slots = [3, 0, 4]
    done = [0, 0, 0]
    got = [[] for _ in lengths]
    # first all but the last 20 tokens of each (the one-token sequence whole), then the rest one token a call
    pieces = [[(b, 0, max(1, n - 20)) for b, n in enumerate(lengths)]]
    for step in range(20):
        pieces.append([(b, n - 20 + step, n - 20 + step + 1) for b, n in enumerate(lengths) if n > 20])
    for piece in pieces:
        rows = np.concatenate([h[b][lo:hi] for b, lo, hi in piece])
        proj = torch.mm(dev(rows, torch.float32), w_in.t())
        out = torch.empty((rows.shape[0], heads * vdim), dtype=torch.float32, device=DEV)
        cu = np.concatenate([[0], np.cumsum([hi - lo for _, lo, hi in piece])]).astype(np.int32)
        ops().gla_scan(proj, offsets, dev(w["m.a2"], torch.float32), dev(w["m.a2.b"], torch.float32), dev(w["m.norm"], torch.float32),
                       state, dev(np.array([slots[b] for b, _, _ in piece], dtype=np.int32)),
                       dev(np.array([lo for _, lo, _ in piece], dtype=np.int32)), dev(cu), out, heads=heads, dim=dim, vdim=vdim,
                       tau=tau, q_scale=dim ** -0.5, eps=1e-5)
        o = f64(out)
        for i, (b, lo, hi) in enumerate(piece):
            got[b].append(o[cu[i]:cu[i + 1]])
            done[b] = hi
    for b, n in enumerate(lengths):
        close(np.concatenate(got[b]), want[b], 2e-5, f"sequence {b}")
        close(f64(state[slots[b], n & 1]), states[b], 2e-5, f"state of sequence {b}")


@pytest.mark.parametrize("heads,dim,vdim,rank,tau", [(2, 16, 24, 5, 4.0), (1, 128, 128, 16, 16.0), (3, 40, 70, 3, 1.0),
                                                     (1, 300, 130, 4, 8.0)])
def test_gated_linear_attention_in_segments_side_by_side(heads, dim, vdim, rank, tau):
    """A first call leaves a state; the second call's tokens are cut into segments of 128, 50 and 1 tokens that
    run side by side: outputs and the new state equal the plain recurrence over all tokens."""
    rng = np.random.default_rng(dim * vdim)
    width = 32
    w, mixer = gla_case(rng, heads, dim, vdim, rank, width, tau, 1.0)
    first, second = [70, 3, 1], [300, 129, 1]
    h = [rng.normal(size=(a + b, width)) for a, b in zip(first, second)]
    want, states = zip(*[pb.gla_mixer(x, w, "m.", mixer, 1e-5) for x in h])
    w_in = dev(np.concatenate([w["m.q"], w["m.k"], w["m.v"], w["m.g"], w["m.a1"]]), torch.float32)
    offsets = (0, heads * dim, 2 * heads * dim, 2 * heads * dim + heads * vdim, 2 * heads * dim + 2 * heads * vdim)
    state = torch.zeros((4, 2, heads, dim, vdim), dtype=torch.float32, device=DEV)
    slots = dev(np.array([2, 0, 3], dtype=np.int32))
    tensors = (dev(w["m.a2"], torch.float32), dev(w["m.a2.b"], torch.float32), dev(w["m.norm"], torch.float32))
    sizes = dict(heads=heads, dim=dim, vdim=vdim, tau=tau, q_scale=dim ** -0.5, eps=1e-5)
    for call, lengths in enumerate((first, second)):
        begin = [0, 0, 0] if call == 0 else first
        rows = np.concatenate([x[b:b + n] for x, b, n in zip(h, begin, lengths)])
        proj = torch.mm(dev(rows, torch.float32), w_in.t())
        out = torch.empty((rows.shape[0], heads * vdim), dtype=torch.float32, device=DEV)
        cu = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
        segments = scratch = None
        if call == 1:
            for size in (128, 50, 1):
                seqs, lo, hi, firsts = [], [], [], [0]
                for b, n in enumerate(lengths):
                    for t in range(0, n, size):
                        seqs.append(b), lo.append(t), hi.append(min(t + size, n))
                    firsts.append(len(seqs))
                segments = tuple(dev(np.array(x, dtype=np.int32)) for x in (seqs, lo, hi, firsts))
                scratch = torch.full((ops().gla_scratch_floats(len(seqs), heads, dim, vdim),), float("nan"), device=DEV)
                kept = state.clone()
                ops().gla_scan(proj, offsets, *tensors, kept, slots, dev(np.array(begin, dtype=np.int32)), dev(cu), out,
                               segments=segments, scratch=scratch, **sizes)
                o = f64(out)
                for b, n in enumerate(lengths):
                    close(o[cu[b]:cu[b + 1]], want[b][begin[b]:], 3e-5, f"segments of {size}, sequence {b}")
                    close(f64(kept[int(slots[b]), (begin[b] + n) & 1]), states[b], 3e-5, f"segments of {size}, state {b}")
        else:
            ops().gla_scan(proj, offsets, *tensors, state, slots, dev(np.array(begin, dtype=np.int32)), dev(cu), out, **sizes)
            o = f64(out)
            for b, n in enumerate(lengths):
                close(o[cu[b]:cu[b + 1]], want[b][:n], 3e-5, f"first call, sequence {b}")


def test_gated_linear_attention_remembers_a_token_hundreds_of_steps_back():
    """With decays close to one the first token's value is still in the output 600 tokens later; with strong
    decays it is gone.  The first token alone carries a large key and value."""
    rng = np.random.default_rng(5)
    heads, dim, vdim, rank, width, n = 1, 16, 16, 2, 24, 600
    for shift, survives in ((9.0, True), (-2.0, False)):
        w, mixer = gla_case(rng, heads, dim, vdim, rank, width, 8.0, shift)
        w["m.norm"] = np.ones(vdim)
        h = rng.normal(size=(n, width)) * 0.05
        h[0] = rng.normal(size=width) * 4.0
        want, _ = pb.gla_mixer(h, w, "m.", mixer, 1e-5)
        blank = h.copy()
        blank[0] = 0.0
        other, _ = pb.gla_mixer(blank, w, "m.", mixer, 1e-5)
        assert (np.abs(want[-1] - other[-1]).max() > 0.5 * np.abs(want[-1]).max()) == survives
        w_in = dev(np.concatenate([w["m.q"], w["m.k"], w["m.v"], w["m.g"], w["m.a1"]]), torch.float32)
        proj = torch.mm(dev(h, torch.float32), w_in.t())
        out = torch.empty((n, vdim), dtype=torch.float32, device=DEV)
        state = torch.zeros((1, 2, heads, dim, vdim), dtype=torch.float32, device=DEV)
        ops().gla_scan(proj, (0, dim, 2 * dim, 2 * dim + vdim, 2 * dim + 2 * vdim), dev(w["m.a2"], torch.float32),
                       dev(w["m.a2.b"], torch.float32), dev(w["m.norm"], torch.float32), state, dev(np.zeros(1, dtype=np.int32)),
                       dev(np.zeros(1, dtype=np.int32)), dev(np.array([0, n], dtype=np.int32)), out, heads=heads, dim=dim,
                       vdim=vdim, tau=8.0, q_scale=dim ** -0.5, eps=1e-5)
        close(f64(out), want, 5e-5, f"decay bias {shift}")


def sloped_case(rng, heads, kv_heads, dim, seqs, far=None):
    """Pages, queries and the plain result for sequences (tokens in the cache before the step, new tokens); ``far``
    = (sequence, position) makes that key stand out for the first head of every group in the sequence's last query."""
    lengths = [start + n for start, n in seqs]
    keys, values, kc, vc, table = scrambled_pages(rng, len(seqs), lengths, kv_heads, dim, dim, "bfloat16")
    rows = [(b, p) for b, (start, n) in enumerate(seqs) for p in range(start, start + n)]
    q = rounded(rng.normal(size=(len(rows), heads, dim)) * 0.5, "bfloat16")
    if far is not None:
        b, position = far
        last = max(r for r, (bb, _) in enumerate(rows) if bb == b)
        for g in range(kv_heads):
            keys[b][position, g] = rounded(q[last, g * (heads // kv_heads)] * 12.0, "bfloat16")
            values[b][position, g] = 9.0
        page, place = table[b, position // 64], position % 64
        kc[page, :, place] = keys[b][position]
        vc[page, :, :, place] = values[b][position]
    slopes = pb.distance_slopes(heads)
    want = np.stack([plain_scores_attention(q[r], keys[b], values[b], p, heads, 0.2, slopes).reshape(-1)
                     for r, (b, p) in enumerate(rows)])
    return dict(q=dev(q.reshape(len(rows), -1), torch.bfloat16), kc=dev(kc, torch.bfloat16), vc=dev(vc, torch.bfloat16),
                table=dev(table), rows=rows, want=want, slopes=dev(slopes, torch.float32), seqs=seqs)


@pytest.mark.parametrize("heads,kv_heads,dim", [(6, 1, 128), (8, 8, 64), (32, 2, 32), (12, 2, 96), (4, 2, 64)])
@pytest.mark.parametrize("kernel", ["attention_decode_mma", "attention_decode_tma"])
def test_one_token_attention_on_tensor_cores_with_distance_slopes(heads, kv_heads, dim, kernel):
    if kernel == "attention_decode_tma" and dim not in (64, 128):
        pytest.skip("the TMA kernel takes head sizes 64 and 128")
    rng = np.random.default_rng(dim + heads)
    c = sloped_case(rng, heads, kv_heads, dim, [(999, 1), (256, 1), (63, 1), (0, 1), (512, 1)], far=(0, 17))
    positions = np.array([p for _, p in c["rows"]], dtype=np.int32)
    chunks = (int(positions.max()) + 256) // 256
    n = len(positions)
    part_o = torch.full((n, heads, chunks, dim), float("nan"), dtype=torch.float32, device=DEV)
    part_ml = torch.full((n, heads, chunks, 2), float("nan"), dtype=torch.float32, device=DEV)
    for extra in ([{}] if kernel == "attention_decode_mma" else [{}, {"chunks_per_block": 2}, {"chunks_per_block": 4}]):
        out = torch.full_like(c["q"], 7.0)
        getattr(ops(), kernel)(c["q"], c["kc"], c["vc"], c["table"], dev(positions), dev(np.arange(n, dtype=np.int32)), part_o,
                               part_ml, out, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, scale=0.2, window=None,
                               max_chunks=chunks, slopes=c["slopes"], **extra)
        ops().tc_status_check(DEV)
        close(f64(out), c["want"], 1.2e-2, f"{kernel} {extra}")


@pytest.mark.parametrize("heads,kv_heads,dim", [(6, 1, 128), (4, 4, 64), (8, 2, 32), (6, 2, 96)])
@pytest.mark.parametrize("kernel", ["attention_prefill_mma", "attention_prefill_tc"])
def test_many_token_attention_on_tensor_cores_with_distance_slopes(heads, kv_heads, dim, kernel):
    if kernel == "attention_prefill_tc" and dim not in (64, 128):
        pytest.skip("the tcgen05 kernel takes head sizes 64 and 128")
    rng = np.random.default_rng(3 * dim + heads)
    seqs = [(0, 300), (130, 17), (0, 1), (63, 200), (500, 129)]
    c = sloped_case(rng, heads, kv_heads, dim, seqs, far=(4, 9))
    tile = 128 if kernel == "attention_prefill_tc" else 16
    tile_seq = np.concatenate([np.full((n + tile - 1) // tile, b) for b, (_, n) in enumerate(seqs)]).astype(np.int32)
    tile_q0 = np.concatenate([np.arange(0, n, tile) for _, n in seqs]).astype(np.int32)
    q_lens = np.array([n for _, n in seqs], dtype=np.int32)
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    out = torch.full_like(c["q"], 7.0)
    getattr(ops(), kernel)(c["q"], c["kc"], c["vc"], c["table"], dev(tile_seq), dev(tile_q0), dev(np.arange(len(seqs), dtype=np.int32)),
                           dev(np.array([s for s, _ in seqs], dtype=np.int32)), dev(q_lens), dev(cu), out, num_heads=heads,
                           num_kv_heads=kv_heads, head_dim=dim, scale=0.2, window=None, slopes=c["slopes"])
    ops().tc_status_check(DEV)
    close(f64(out), c["want"], 1.2e-2, kernel)


# ------------------------------------------------------------------------------------------- whole models

_LOADED = {}


def loaded(name, dtype, record_steps=True):
    key = (name, dtype, record_steps)
    if key not in _LOADED:
        lm = fr.load(model_folder(name), dtype=dtype, max_tokens=4096, num_slots=8)
        lm.engine.record_steps = record_steps and lm.model.replayable
        _LOADED[key] = lm
    return _LOADED[key]


_PLAIN = {}


def plain_logits(name, length, seed):
    key = (name, length, seed)
    if key not in _PLAIN:
        config, weights = plain_weights(name)
        _PLAIN[key] = pb.forward(config, weights, request_tokens(name, length, seed))
    return _PLAIN[key]


def model_close(got, ref, dtype, what):
    """Row by row: the root mean square of the difference over the vocabulary (its mean taken off: a shift of all
    logits changes no probability) against the root mean square of the plain logits."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert np.isfinite(got).all(), what
    diff = got - ref
    diff = diff - diff.mean(axis=-1, keepdims=True)
    per_row = np.sqrt((diff ** 2).mean(axis=-1)) / np.sqrt(((ref - ref.mean()) ** 2).mean())
    bad = per_row > MODEL_TOL[dtype]
    assert not bad.any(), (f"{what}: relative error {per_row.max():.3e} > {MODEL_TOL[dtype]:.1e} ({dtype}); first wrong row "
                           f"{int(np.argmax(bad))} of {len(per_row)}")
    if dtype == "bfloat16" and len(per_row) >= 20:
        assert np.quantile(per_row, 0.9) <= BF16_MOST_ROWS, f"{what}: a tenth of the rows is off by more than {BF16_MOST_ROWS}"


def run_schedule(lm, requests, steps):
    """``steps``: lists of (request, first position, end position); every place is wanted.  A request gets its slot
    at its first step and gives it back after its last token.  Returns request -> logits [length, vocab]."""
    engine = lm.engine
    slots, rows_of = {}, {key: [] for key in requests}
    for step in steps:
        for key, lo, hi in step:
            if key not in slots:
                slots[key] = engine.new_sequence()
        out = engine.step([slots[k] for k, _, _ in step], [requests[k][lo:hi] for k, lo, hi in step],
                          [list(range(hi - lo)) for _, lo, hi in step]).float().cpu().numpy()
        at = 0
        for key, lo, hi in step:
            rows_of[key].append(out[at:at + hi - lo])
            at += hi - lo
            if hi == len(requests[key]):
                engine.release(slots.pop(key))
    engine.check()
    engine.cache.check()
    assert not slots
    return {key: np.concatenate(parts) for key, parts in rows_of.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts(name, dtype):
    lm = loaded(name, dtype)
    for length, seed in ((1, 0), (2, 1), (63, 2), (64, 3), (65, 4), (300, 5)):
        got = lm.logits(request_tokens(name, length, seed)).float().cpu().numpy()
        model_close(got, plain_logits(name, length, seed), dtype, f"model {name}, {length} tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_prompt_then_token_by_token(name, dtype):
    lm = loaded(name, dtype)
    length, tail = 150, 90                  # the decoded tokens cross the page border at 64 and at 128
    ids = request_tokens(name, length, 6)
    steps = [[("r", 0, length - tail)]] + [[("r", p, p + 1)] for p in range(length - tail, length)]
    got = run_schedule(lm, {"r": ids}, steps)["r"]
    model_close(got, plain_logits(name, length, 6), dtype, f"model {name}, last {tail} tokens one by one")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_sequence_decoded_from_its_first_token(dtype):
    lm = loaded("A", dtype)
    length = 140
    ids = request_tokens("A", length, 7)
    got = run_schedule(lm, {"r": ids}, [[("r", p, p + 1)] for p in range(length)])["r"]
    model_close(got, plain_logits("A", length, 7), dtype, "one token a step from the start")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
@pytest.mark.parametrize("portion", [2, 3, 17, 64, 65])
def test_prompts_in_portions(name, dtype, portion):
    lm = loaded(name, dtype)
    length = 135
    ids = request_tokens(name, length, 8)
    steps = [[("r", lo, min(lo + portion, length))] for lo in range(0, length, portion)]
    got = run_schedule(lm, {"r": ids}, steps)["r"]
    model_close(got, plain_logits(name, length, 8), dtype, f"model {name}, portions of {portion}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_requests_in_one_batch_then_decoded_together_over_reused_slots(name, dtype):
    lm = loaded(name, dtype)
    for turn in range(2):                 # the second turn takes the slots, pages and states the first gave back
        lengths = {"a": 1 + 30, "b": 70 + 30, "c": 200 + 30, "d": 64 + 12, "e": 129 + 5} if turn == 0 else \
                  {"a": 90 + 25, "b": 3 + 25, "c": 64 + 25}
        tails = {"a": 30, "b": 30, "c": 30, "d": 12, "e": 5} if turn == 0 else {"a": 25, "b": 25, "c": 25}
        requests = {k: request_tokens(name, n, 20 + turn * 10 + i) for i, (k, n) in enumerate(lengths.items())}
        steps = [[(k, 0, lengths[k] - tails[k]) for k in lengths]]
        for t in range(max(tails.values())):
            steps.append([(k, lengths[k] - tails[k] + t, lengths[k] - tails[k] + t + 1) for k in lengths if t < tails[k]])
        got = run_schedule(lm, requests, steps)
        for i, k in enumerate(lengths):
            model_close(got[k], plain_logits(name, lengths[k], 20 + turn * 10 + i), dtype,
                        f"model {name}, turn {turn}, request {k}")


@pytest.mark.parametrize("name", ["A", "C"])
def test_recorded_decode_steps_equal_direct_ones(name):
    """Five sequences decode in a recorded step of six rows, the last sequence twice: the recurrent state and the
    cache must come out as if it were there once."""
    results = []
    for record in (False, True):
        lm = loaded(name, "bfloat16", record_steps=record)
        engine = lm.engine
        prompts = [request_tokens(name, n, 40 + i) for i, n in enumerate((5, 64, 1, 30, 100))]
        slots = [engine.new_sequence() for _ in prompts]
        logits = engine.step(slots, prompts)
        rows = [logits.float().cpu().numpy()]
        for step in range(12):
            tokens = [[(7 * step + 3 * i) % ALL[name][0]["vocab"]] for i in range(len(slots))]
            rows.append(engine.step(slots, tokens).float().cpu().numpy())
        for slot in slots:
            engine.release(slot)
        if record:
            assert engine.steps_replayed > 0
        results.append(np.stack(rows))
    assert np.array_equal(results[0], results[1])


def test_greedy_generation_through_the_entry_point():
    name = "A"
    config, weights = plain_weights(name)
    lm = loaded(name, "float32")
    prompts = [request_tokens(name, n, 60 + i) for i, n in enumerate((9, 1, 70))]
    got = lm.generate_batch(prompts, max_tokens=14, ignore_eos=True)
    for prompt, tokens in zip(prompts, got):
        ids = list(prompt)
        for _ in range(14):
            row = pb.forward(config, weights, ids)[-1]
            top2 = np.sort(row)[-2:]
            assert top2[1] - top2[0] > 1e-4, "a near tie: the case does not pin the greedy choice"
            ids.append(int(np.argmax(row)))
        assert tokens == ids[len(prompt):]
    assert lm.generate(prompts[0], 5) == got[0][:5]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_trace_replayed_through_the_runner(tmp_path, dtype):
    """bin/trace_run as a user drives it: a batch of three prompts of unequal lengths (one of a single token, one of
    which nothing is wanted), decoded together while the shorter requests end, then another batch in the freed slots."""
    name = "B"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    vocab = ALL[name][0]["vocab"]
    lengths = {"p": 1 + 6, "q": 80 + 20, "r": 130 + 9, "s": 65 + 12}
    heads = {"p": 1, "q": 80, "r": 130, "s": 65}
    ids = {k: request_tokens(name, n, 70 + i) for i, (k, n) in enumerate(lengths.items())}
    steps, rows, step = [], {k: [] for k in ids}, 0
    for batch in (["p", "q", "r"], ["s"]):
        entries = []
        at = 0
        for k in batch:
            want = [] if k == "q" else ([0] if heads[k] == 1 else [0, heads[k] // 2, heads[k] - 1])
            entries.append({"id": k, "tokens": ids[k][:heads[k]], "want": want})
            for w in want:
                rows[k].append((step, at, w))
                at += 1
        steps.append({"step": step, "entries": entries, "end": []})
        step += 1
        for t in range(max(lengths[k] - heads[k] for k in batch)):
            live = [k for k in batch if heads[k] + t < lengths[k]]
            steps.append({"step": step, "entries": [{"id": k, "tokens": [ids[k][heads[k] + t]], "want": [0]} for k in live],
                          "end": [k for k in live if heads[k] + t == lengths[k] - 1]})
            for row, k in enumerate(live):
                rows[k].append((step, row, heads[k] + t))
            step += 1
    text = "".join(json.dumps(x) + "\n" for x in steps)
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model_folder(name), "--dtype", dtype,
                           "--out", str(tmp_path), "--max-tokens", "384"], input=text, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [line for line in proc.stdout.splitlines() if line.startswith("done ")] == [f"done {x['step']}" for x in steps]
    out = {}
    for x in steps:
        wanted = sum(len(e["want"]) for e in x["entries"])
        if wanted:
            out[x["step"]] = np.fromfile(os.path.join(tmp_path, f"{x['step']}.f32"), dtype="<f4").reshape(wanted, vocab)
    for i, (k, n) in enumerate(lengths.items()):
        plain = plain_logits(name, n, 70 + i)
        got = np.stack([out[s][row] for s, row, _ in rows[k]])
        model_close(got, plain[[pos for _, _, pos in rows[k]]], dtype, f"request {k}")


def test_command_line_generates_with_the_design(tmp_path):
    """`python -m fieldrun_b200 random` writes a model of the design from a config.json, and the command line
    generates from it what the plain model's greedy loop gives."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(ALL["B"][0]))
    folder = tmp_path / "model"
    made = subprocess.run([sys.executable, "-m", "fieldrun_b200", "random", "--config", str(config_path), "--seed", "9", "--std", "0.1",
                           "--bias-std", "0.3", "-o", str(folder)], capture_output=True, text=True, cwd=root, timeout=300)
    assert made.returncode == 0, made.stderr
    with open(folder / "config.json") as handle:
        config = json.load(handle)
    from fieldrun_b200.weights.safetensors_io import ModelFolder
    files = ModelFolder(str(folder))
    weights = {n: files.tensor(n).double().numpy() for n in files.entries}
    files.close()
    ids = request_tokens("B", 20, 90)
    (tmp_path / "ids.json").write_text(json.dumps(ids))
    run = subprocess.run([sys.executable, "-m", "fieldrun_b200", "--model", str(folder), "--ids", str(tmp_path / "ids.json"), "--ctx", "12",
                          "--generate", "6", "--dtype", "float32", "--eos", "none"], capture_output=True, text=True, cwd=root, timeout=600)
    assert run.returncode == 0, run.stderr
    want = ids[:12]
    for _ in range(6):
        want.append(int(np.argmax(pb.forward(config, weights, want)[-1])))
    assert " ".join(str(t) for t in want[12:]) in run.stdout, run.stdout
