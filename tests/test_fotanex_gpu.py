"""The Fotanex design in the engine against the plain implementation of ``plain_fotanex``: each mechanism's kernel
alone, then whole models through the step function, the cache, recorded decode steps and the entry point."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import fieldrun_b200 as fr
import plain_fotanex as pf
from fotanex_configs import ALL, model_folder, plain_weights, request_tokens

pytestmark = pytest.mark.gpu

DEV = "cuda"
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
KERNEL_TOL = {"float32": 5e-6, "bfloat16": 1.2e-2}
# see model_close: per row, against the spread of the plain logits.  bfloat16 runs compare with the plain model made to
# use the experts the engine used (the router is not continuous), so the limit holds on every row.
MODEL_TOL = {"float32": 3e-5, "bfloat16": 6e-2}
ROUTE_MARGIN = 5e-3          # the engine may pick other experts than the plain model only where the scores are this close


def ops():
    from fieldrun_b200.csrc import ops as o
    return o


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(DEV).contiguous()


def f32(a):
    return dev(np.asarray(a, dtype=np.float32))


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


class Tables:
    """A step's tables on the device, as the kernels read them: sequences in ``slots`` that continue at ``starts``
    with ``q_lens`` new tokens each."""

    def __init__(self, slots, starts, q_lens):
        cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
        self.num_seqs = len(slots)
        self.seq_slot = dev(np.asarray(slots, dtype=np.int32))
        self.seq_start = dev(np.asarray(starts, dtype=np.int32))
        self.cu_q_len = dev(cu)
        self.tok_seq = dev(np.repeat(np.arange(len(slots)), q_lens).astype(np.int32))
        self.rows = [(int(cu[b]), int(cu[b + 1])) for b in range(len(slots))]


def in_steps(lengths, portions):
    """Cuts sequences of ``lengths`` into steps: ``portions[b]`` lists the sizes of sequence b's portions; step s holds
    the s-th portion of every sequence that still has one.  Yields (sequences, starts, sizes)."""
    at = [0] * len(lengths)
    for s in range(max(len(p) for p in portions)):
        live = [b for b in range(len(lengths)) if s < len(portions[b])]
        yield live, [at[b] for b in live], [portions[b][s] for b in live]
        for b in live:
            at[b] += portions[b][s]
    assert at == list(lengths)


# ------------------------------------------------------------------------------------------- mechanisms alone

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [40, 257, 1100])
def test_dynamic_tanh_of_a_stream_with_updates_for_two_norms_at_once(dtype, width):
    rng = np.random.default_rng(width)
    rows, top = 9, 3
    x, d0, d1 = (rng.normal(size=(rows, width)) for _ in range(3))
    y = rng.normal(size=(rows * top, width))
    ew = rng.uniform(0.1, 1.0, size=(rows, top))
    rowmap = rng.permutation(rows * top).astype(np.int32)
    norms = [(rng.normal(1.0, 0.2, width), rng.normal(0.0, 0.3, width), np.array([a])) for a in (0.4, 0.9)]
    stream = f32(x)
    out1 = torch.empty((rows, width), dtype=TORCH[dtype], device=DEV)
    out2, out2_32 = torch.empty_like(out1), torch.empty((rows, width), dtype=torch.float32, device=DEV)
    triples = [tuple(f32(t) for t in n) for n in norms]
    ops().dyt_norm(stream, triples[0], out1, second=triples[1], out2=out2, out2_32=out2_32, deltas=(f32(d0), f32(d1)),
                   experts=(f32(y), f32(ew), dev(rowmap)), write_back=True)
    total = x.astype(np.float32).astype(np.float64) + d0 + d1 + np.einsum("tk,tkw->tw", ew, y[rowmap].reshape(rows, top, width))
    close(f64(stream), total, 5e-6, "the sum stored back")
    for out, (w, b, a) in ((out1, norms[0]), (out2, norms[1])):
        close(f64(out), pf.dynamic_tanh(total, w, b, a[0]), KERNEL_TOL[dtype], "dynamic tanh")
    close(f64(out2_32), pf.dynamic_tanh(total, norms[1][0], norms[1][1], norms[1][2][0]), 5e-6, "the float32 copy")
    # one norm of chosen rows, nothing stored back
    pick = np.array([7, 0, 3], dtype=np.int32)
    before = f64(stream).copy()
    few = torch.empty((3, width), dtype=TORCH[dtype], device=DEV)
    ops().dyt_norm(stream, triples[0], few, deltas=(f32(d0),), rows=dev(pick))
    close(f64(few), pf.dynamic_tanh(before[pick] + d0[pick], *norms[0][:2], norms[0][2][0]), KERNEL_TOL[dtype], "chosen rows")
    assert np.array_equal(f64(stream), before)


def test_two_outputs_blended_by_their_root_mean_squares_and_the_reentry_of_the_stream():
    rng = np.random.default_rng(2)
    rows, width = 11, 90
    a, b = rng.normal(size=(rows, width)) * 3.0, rng.normal(size=(rows, width)) * 0.01
    wa, wb = rng.normal(1.0, 0.3, width), rng.normal(1.0, 0.3, width)
    out = torch.empty((rows, width), dtype=torch.float32, device=DEV)
    ops().rms_blend(f32(a), f32(b), f32(wa), f32(wb), out, 1e-5, 0.5)
    close(f64(out), pf.parallel_mixer(None, a, b, wa, wb, 1e-5), 5e-6, "rms blend")
    for dtype in ("float32", "bfloat16"):
        both = torch.empty((rows, 2 * width), dtype=TORCH[dtype], device=DEV)
        ops().concat_rows(f32(a), f32(b), both, delta=f32(b))
        close(f64(both), np.concatenate([a + b, b], axis=1), KERNEL_TOL[dtype], "rows side by side")
    ops().add_row_vector(f32(a), f32(wa), out)
    close(f64(out), a + wa, 1e-6, "a vector on every row")


@pytest.mark.parametrize("taps", [1, 2, 4, 5])
@pytest.mark.parametrize("activation", [None, "silu"])
def test_causal_convolution_keeps_its_last_inputs_from_step_to_step(taps, activation):
    """Three sequences of unequal lengths in portions down to one token, in slots that an earlier sequence used: the
    inputs before a portion come from the state, also where a portion is shorter than the taps reach back."""
    rng = np.random.default_rng(taps)
    channels, stride, offset = 150, 170, 13
    lengths = [23, 1, 40]
    portions = [[2, 1, 3, 2, 1, 14], [1], [5, 1, 1, 2, 31]]
    weights, bias, in_bias = rng.normal(size=(channels, taps)), rng.normal(size=channels), rng.normal(size=channels)
    inputs = [rng.normal(size=(n, stride)) for n in lengths]
    state = torch.full((5, 2, 7 + (taps - 1) * channels), 9.0, dtype=torch.float32, device=DEV)     # what an earlier user left
    slots = [3, 0, 4]
    state[slots] = 0.0                                        # the cache zeroes a slot when it hands it out
    got = [np.zeros((n, channels)) for n in lengths]
    for live, starts, sizes in in_steps(lengths, portions):
        tables = Tables([slots[b] for b in live], starts, sizes)
        rows = np.concatenate([inputs[b][s:s + n] for b, s, n in zip(live, starts, sizes)])
        out32 = torch.empty((rows.shape[0], channels), dtype=torch.float32, device=DEV)
        typed = torch.empty((rows.shape[0], channels), dtype=torch.bfloat16, device=DEV)
        ops().causal_conv(f32(rows), offset, channels, f32(weights), f32(bias), tables, state, 7, out32, typed,
                          in_bias=f32(in_bias), activation=activation)
        close(f64(typed), f64(out32), 8e-3, "the copy in the model dtype")
        for b, s, n, (lo, hi) in zip(live, starts, sizes, tables.rows):
            got[b][s:s + n] = f64(out32[lo:hi])
    for b, n in enumerate(lengths):
        want = pf.causal_conv(inputs[b][:, offset:offset + channels].astype(np.float32) + in_bias, weights, bias)
        if activation == "silu":
            want = pf.silu(want)
        close(got[b], want, 5e-6, f"sequence {b}")
    assert float(state[slots][:, :, :7].abs().sum()) == 0.0                            # only its own part is written
    assert float(state[1].min()) == 9.0 and float(state[2].min()) == 9.0              # and only the step's slots


@pytest.mark.parametrize("inner,n", [(150, 8), (70, 24), (33, 40), (128, 100), (16, 300)])
def test_selective_scan_carries_its_state_and_remembers_far_tokens(inner, n):
    """Small steps and decays close to one: what the first tokens wrote is still most of the state six hundred tokens
    on, so a lost or doubly applied state, or a decay that lost its distance from one, shows."""
    rng = np.random.default_rng(inner + n)
    lengths = [600, 37]
    portions = [[300, 1, 1, 1, 64, 233], [36, 1]]
    dt_bias = rng.normal(-5.0, 1.0, inner)
    a_log = rng.normal(-1.0, 1.0, (inner, n))
    d = rng.normal(size=inner)
    data = [dict(x=rng.normal(size=(t, inner)), z=rng.normal(size=(t, inner)), dt=rng.normal(size=(t, inner)),
                 b=rng.normal(size=(t, n)), c=rng.normal(size=(t, n))) for t in lengths]
    data[0]["x"][3] *= 30.0                                   # a far token that stands out
    state = torch.zeros((3, 2, inner * n + 11), dtype=torch.float32, device=DEV)
    got = [np.zeros((t, inner)) for t in lengths]
    slots = [2, 0]
    for live, starts, sizes in in_steps(lengths, portions):
        tables = Tables([slots[b] for b in live], starts, sizes)
        cut = lambda key: np.concatenate([data[b][key][s:s + m] for b, s, m in zip(live, starts, sizes)])
        xz = np.concatenate([cut("x") * 0 + 5.0, cut("z")], axis=1)          # only z is read from this tensor
        low = np.concatenate([np.full((xz.shape[0], 2), 3.0), cut("b"), cut("c")], axis=1)
        out = torch.empty((xz.shape[0], inner), dtype=torch.float32, device=DEV)
        ops().selective_scan(f32(xz), inner, f32(cut("x")), f32(low), 2, 2 + n, f32(cut("dt")), f32(dt_bias), f32(a_log), f32(d),
                             tables, state, 0, out)
        for b, s, m, (lo, hi) in zip(live, starts, sizes, tables.rows):
            got[b][s:s + m] = f64(out[lo:hi])
    for b in range(2):
        r = {k: v.astype(np.float32).astype(np.float64) for k, v in data[b].items()}
        dt = pf.softplus(r["dt"] + dt_bias.astype(np.float32))
        want = pf.selective_recurrence(r["x"], dt, r["b"], r["c"], a_log.astype(np.float32), d.astype(np.float32)) * pf.silu(r["z"])
        close(got[b], want, 2e-5, f"sequence {b}")
    assert float(state[1].abs().sum()) == 0.0 and float(state[:, :, inner * n:].abs().sum()) == 0.0


def test_gated_recurrence_with_decays_close_to_one():
    """lam far below zero makes a = exp(-8 r softplus(lam)) differ from one by 1e-6 and less: over 1,500 tokens the
    state is a sum of everything so far, and a decay rounded to one would be off by thousandths."""
    rng = np.random.default_rng(5)
    blocks, bw = 3, 50
    width = blocks * bw
    lengths = [1500, 130]
    portions = [[700, 1, 1, 798], [129, 1]]
    lam = np.concatenate([rng.normal(-14.0, 1.0, width // 2), rng.normal(0.0, 2.0, width - width // 2)])
    a_bias, i_bias, y_bias = rng.normal(size=width), rng.normal(size=width), rng.normal(size=width)
    data = [dict(y=rng.normal(size=(t, width)), u=rng.normal(size=(t, width)), r=rng.normal(size=(t, width)),
                 i=rng.normal(size=(t, width))) for t in lengths]
    state = torch.zeros((2, 2, width + 5), dtype=torch.float32, device=DEV)
    got = [np.zeros((t, width)) for t in lengths]
    for live, starts, sizes in in_steps(lengths, portions):
        tables = Tables(live, starts, sizes)
        cut = lambda key: np.concatenate([data[b][key][s:s + m] for b, s, m in zip(live, starts, sizes)])
        rows = cut("y").shape[0]
        yx = np.concatenate([np.zeros((rows, 4)), cut("y")], axis=1)
        # the gates' rows lie block by block: [blocks, T, r of the block | i of the block]
        gates = np.concatenate([cut("r").reshape(rows, blocks, bw), cut("i").reshape(rows, blocks, bw)], axis=2).transpose(1, 0, 2)
        out = torch.empty((rows, width), dtype=torch.float32, device=DEV)
        ops().gated_recurrence(f32(yx), 4, f32(y_bias), f32(cut("u")), f32(gates), f32(a_bias), f32(i_bias), f32(lam), tables,
                               state, 0, out, block_width=bw, gate_constant=8.0,
                               prepared=torch.empty((3, rows, width), dtype=torch.float32, device=DEV))
        for b, s, m, (lo, hi) in zip(live, starts, sizes, tables.rows):
            got[b][s:s + m] = f64(out[lo:hi])
    for b in range(2):
        r = {k: v.astype(np.float32).astype(np.float64) for k, v in data[b].items()}
        states = pf.gated_recurrence(r["u"], pf.sigmoid(r["r"] + a_bias.astype(np.float32)), pf.sigmoid(r["i"] + i_bias.astype(np.float32)),
                                     lam.astype(np.float32))
        assert (8.0 * pf.softplus(lam[:width // 2]) < 1e-3).all(), "the case has no decay close to one"
        close(got[b], states * pf.gelu_tanh(r["y"] + y_bias.astype(np.float32)), 2e-5, f"sequence {b}")


@pytest.mark.parametrize("heads,vdim,n,groups,norm_groups", [(3, 20, 10, 1, 1), (4, 36, 70, 2, 4), (2, 64, 130, 2, 1), (6, 32, 300, 3, 2)])
def test_state_space_scan_and_the_norm_in_parts(heads, vdim, n, groups, norm_groups):
    rng = np.random.default_rng(heads * n)
    inner = heads * vdim
    lengths = [400, 9]
    portions = [[150, 1, 1, 2, 246], [8, 1]]
    dt_bias, a_log, d = rng.normal(-4.0, 1.0, heads), rng.normal(-1.0, 1.0, heads), rng.normal(size=heads)
    data = [dict(z=rng.normal(size=(t, inner)), x=rng.normal(size=(t, inner)), b=rng.normal(size=(t, groups * n)),
                 c=rng.normal(size=(t, groups * n)), dt=rng.normal(size=(t, heads))) for t in lengths]
    data[0]["x"][1] *= 20.0
    state = torch.zeros((2, 2, heads * n * vdim + 3), dtype=torch.float32, device=DEV)
    got = [np.zeros((t, inner)) for t in lengths]
    weight = rng.normal(1.0, 0.2, inner)
    for live, starts, sizes in in_steps(lengths, portions):
        tables = Tables(live, starts, sizes)
        cut = lambda key: np.concatenate([data[b][key][s:s + m] for b, s, m in zip(live, starts, sizes)])
        proj = np.concatenate([cut("z"), np.ones((cut("z").shape[0], 5)), cut("dt")], axis=1)
        xbc = np.concatenate([cut("x"), cut("b"), cut("c")], axis=1)
        y = torch.empty((proj.shape[0], inner), dtype=torch.float32, device=DEV)
        ops().state_space_scan(f32(proj), 0, inner + 5, f32(xbc), inner, inner + groups * n, f32(dt_bias), f32(a_log), f32(d), tables,
                               state, 0, y, heads=heads, vdim=vdim, n=n, groups=groups)
        out = torch.empty_like(y)
        ops().group_rms_norm(y, f32(weight), out, norm_groups, 1e-5)
        for b, s, m, (lo, hi) in zip(live, starts, sizes, tables.rows):
            got[b][s:s + m] = f64(out[lo:hi])
    for b in range(2):
        r = {k: v.astype(np.float32).astype(np.float64) for k, v in data[b].items()}
        t = lengths[b]
        y = pf.state_space_recurrence(r["x"].reshape(t, heads, vdim), r["b"].reshape(t, groups, n), r["c"].reshape(t, groups, n),
                                      pf.softplus(r["dt"] + dt_bias.astype(np.float32)), a_log.astype(np.float32), d.astype(np.float32))
        want = pf.group_rms(y.reshape(t, inner) * pf.silu(r["z"]), weight.astype(np.float32), norm_groups, 1e-5)
        close(got[b], want, 2e-5, f"sequence {b}")


def scrambled_pages(rng, lengths, kv_heads, dim, vdim, dtype, spare=3):
    """Keys [slot][T, G, dim], values [slot][T, G, vdim] laid into pages of 64 in a scrambled order."""
    per = [(n + 63) // 64 for n in lengths]
    pages = sum(per) + spare
    order = rng.permutation(pages)
    table = np.full((len(lengths), max(per) + 1), -1, dtype=np.int32)
    kc, vc = np.zeros((pages, kv_heads, 64, dim)), np.zeros((pages, kv_heads, vdim, 64))
    keys, values = [], []
    at = 0
    for s, n in enumerate(lengths):
        keys.append(rounded(rng.normal(size=(n, kv_heads, dim)), dtype))
        values.append(rounded(rng.normal(size=(n, kv_heads, vdim)), dtype))
        for i in range(per[s]):
            table[s, i] = order[at]
            at += 1
    return keys, values, kc, vc, table


def lay_into_pages(keys, values, kc, vc, table):
    for s in range(len(keys)):
        for j in range(keys[s].shape[0]):
            page = table[s, j // 64]
            kc[page, :, j % 64] = keys[s][j]
            vc[page, :, :, j % 64] = values[s][j]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,chunk", [(6, 2, 32, 16, 48), (3, 3, 24, 40, 100), (8, 1, 64, 64, 64), (2, 1, 100, 7, 7),
                                                            (4, 2, 16, 16, 1)])
def test_attention_in_chunks_with_sink_and_head_gate(dtype, heads, kv_heads, dim, vdim, chunk):
    rng = np.random.default_rng(heads * 100 + chunk)
    lengths = [300, 64, 65, 1]
    keys, values, kc, vc, table = scrambled_pages(rng, lengths, kv_heads, dim, vdim, dtype)
    lay_into_pages(keys, values, kc, vc, table)
    sink = rng.normal(0.0, 2.0, heads)
    # queries: the first and last position of chunks, page borders, the end of the long sequence
    places = sorted({0, 1, chunk - 1, chunk, chunk + 1, 2 * chunk - 1, 2 * chunk, 63, 64, 65, 127, 128, 255, 256, 299} & set(range(300)))
    rows = [(0, p) for p in places] + [(1, 0), (1, 63), (2, 64), (3, 0)]
    q = rounded(rng.normal(size=(len(rows), heads, dim)), dtype)
    gate = rng.normal(size=(len(rows), heads + 3))            # rows wider than the heads, as when they are part of a larger product
    out = torch.empty((len(rows), heads * vdim), dtype=TORCH[dtype], device=DEV)
    ops().attention_generic(dev(q, TORCH[dtype]), dev(kc, TORCH[dtype]), dev(vc, TORCH[dtype]), dev(table),
                            dev(np.array([p for _, p in rows], dtype=np.int32)), dev(np.array([s for s, _ in rows], dtype=np.int32)),
                            out, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, scale=0.17, window=None, v_dim=vdim,
                            chunk=chunk, sinks=f32(sink), gate=f32(gate))
    gate32 = gate.astype(np.float32).astype(np.float64)
    want = np.stack([pf.attend_in_chunks(q[r:r + 1], keys[s], values[s], sink.astype(np.float32), gate32[r:r + 1, :heads], 0.17, chunk,
                                         positions=[p])[0].reshape(-1) for r, (s, p) in enumerate(rows)])
    close(f64(out), want, KERNEL_TOL[dtype], "attention in chunks")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_key_just_outside_the_chunk_gets_nothing_and_one_just_inside_gets_nearly_all(dtype):
    """Two keys are made to stand out, the last one of a chunk and the first one of the next: the query sees only the one of
    its own chunk, however large the other's score would be; and a large sink takes most of the weight from all keys."""
    rng = np.random.default_rng(21)
    heads, kv_heads, dim, vdim, chunk, n = 4, 2, 32, 8, 96, 400
    keys, values, kc, vc, table = scrambled_pages(rng, [n], kv_heads, dim, vdim, dtype)
    q = rounded(rng.normal(size=(1, heads, dim)) * 0.1, dtype)
    edge = 3 * chunk                                          # the first position of the query's chunk (the query sits at 380)
    for g in range(kv_heads):
        for place, value in ((edge - 1, 70.0), (edge, -40.0)):
            keys[0][place, g] = rounded(q[0, g * 2] * 60.0, dtype)
            values[0][place, g] = value
    lay_into_pages(keys, values, kc, vc, table)
    for sink in (np.full(heads, -30.0), np.full(heads, 25.0)):
        out = torch.empty((1, heads * vdim), dtype=TORCH[dtype], device=DEV)
        ops().attention_generic(dev(q, TORCH[dtype]), dev(kc, TORCH[dtype]), dev(vc, TORCH[dtype]), dev(table),
                                dev(np.array([380], dtype=np.int32)), dev(np.array([0], dtype=np.int32)), out, num_heads=heads,
                                num_kv_heads=kv_heads, head_dim=dim, scale=1.0, window=None, v_dim=vdim, chunk=chunk, sinks=f32(sink))
        want = pf.attend_in_chunks(q, keys[0], values[0], sink, None, 1.0, chunk, positions=[380]).reshape(1, -1)
        whole = pf.attend_in_chunks(q, keys[0], values[0], sink, None, 1.0, None, positions=[380]).reshape(1, -1)
        if sink[0] < 0:
            assert np.abs(want - whole).max() > 20.0 and want.min() < -20.0, "the case does not show the chunk's edge"
        else:
            assert np.abs(want).max() < 1.0, "the case does not show the sink"
        close(f64(out), want, KERNEL_TOL[dtype], "chunk edge")


def chunked_case(rng, heads, kv_heads, dim, seqs, chunk):
    """Sequences (start, new tokens): keys and values of start + new positions in scrambled pages, a query for each new
    token, a sink per head, and what the plain implementation makes of them.  One early key of the last sequence is
    made to stand out: it counts only for the queries of its own chunk."""
    lengths = [start + n for start, n in seqs]
    keys, values, kc, vc, table = scrambled_pages(rng, lengths, kv_heads, dim, dim, "bfloat16")
    rows = [(s, start + i) for s, (start, n) in enumerate(seqs) for i in range(n)]
    q = rounded(rng.normal(size=(len(rows), heads, dim)), "bfloat16")
    last = len(seqs) - 1
    far = min(5, lengths[last] - 1)
    keys[last][far] = rounded(q[len(rows) - 1, ::heads // kv_heads] * 3.0, "bfloat16")
    values[last][far] = 9.0
    lay_into_pages(keys, values, kc, vc, table)
    sink = rng.normal(1.0, 2.0, heads)
    want = np.stack([pf.attend_in_chunks(q[r:r + 1], keys[s], values[s], sink.astype(np.float32), None, 0.2, chunk, positions=[p])[0].reshape(-1)
                     for r, (s, p) in enumerate(rows)])
    return dict(q=dev(q.reshape(len(rows), heads * dim), torch.bfloat16), kc=dev(kc, torch.bfloat16), vc=dev(vc, torch.bfloat16),
                table=dev(table), sink=f32(sink), rows=rows, want=want)


@pytest.mark.parametrize("heads,kv_heads,dim", [(6, 1, 128), (8, 8, 64), (32, 2, 32), (12, 2, 96), (4, 2, 64)])
@pytest.mark.parametrize("chunk", [64, 100, 640])
@pytest.mark.parametrize("kernel", ["attention_decode_mma", "attention_decode_tma"])
def test_one_token_attention_on_tensor_cores_in_chunks_with_sinks(heads, kv_heads, dim, chunk, kernel):
    if kernel == "attention_decode_tma" and dim not in (64, 128):
        pytest.skip("the TMA kernel takes head sizes 64 and 128")
    rng = np.random.default_rng(dim + heads + chunk)
    c = chunked_case(rng, heads, kv_heads, dim, [(999, 1), (256, 1), (63, 1), (0, 1), (512, 1), (chunk, 1), (chunk - 1, 1), (2 * chunk + 3, 1)], chunk)
    positions = np.array([p for _, p in c["rows"]], dtype=np.int32)
    chunks = (int(positions.max()) + 256) // 256
    n = len(positions)
    part_o = torch.full((n, heads, chunks, dim), float("nan"), dtype=torch.float32, device=DEV)
    part_ml = torch.full((n, heads, chunks, 2), float("nan"), dtype=torch.float32, device=DEV)
    for extra in ([{}] if kernel == "attention_decode_mma" else [{}, {"chunks_per_block": 2}, {"chunks_per_block": 4}]):
        out = torch.full_like(c["q"], 7.0)
        getattr(ops(), kernel)(c["q"], c["kc"], c["vc"], c["table"], dev(positions), dev(np.arange(n, dtype=np.int32)), part_o,
                               part_ml, out, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, scale=0.2, window=None,
                               max_chunks=chunks, chunk=chunk, sinks=c["sink"], **extra)
        ops().tc_status_check(DEV)
        close(f64(out), c["want"], 1.2e-2, f"{kernel} {extra}")


@pytest.mark.parametrize("heads,kv_heads,dim", [(6, 1, 128), (4, 4, 64), (8, 2, 32), (6, 2, 96)])
@pytest.mark.parametrize("chunk", [64, 100, 128, 640])
@pytest.mark.parametrize("kernel", ["attention_prefill_mma", "attention_prefill_tc"])
def test_many_token_attention_on_tensor_cores_in_chunks_with_sinks_and_the_head_gate(heads, kv_heads, dim, chunk, kernel):
    if kernel == "attention_prefill_tc" and dim not in (64, 128):
        pytest.skip("the tcgen05 kernel takes head sizes 64 and 128")
    rng = np.random.default_rng(3 * dim + heads + chunk)
    seqs = [(0, 300), (130, 17), (0, 1), (63, 200), (500, 129), (0, 700)]
    c = chunked_case(rng, heads, kv_heads, dim, seqs, chunk)
    tile = 128 if kernel == "attention_prefill_tc" else 16
    tile_seq = np.concatenate([np.full((n + tile - 1) // tile, b) for b, (_, n) in enumerate(seqs)]).astype(np.int32)
    tile_q0 = np.concatenate([np.arange(0, n, tile) for _, n in seqs]).astype(np.int32)
    q_lens = np.array([n for _, n in seqs], dtype=np.int32)
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    out = torch.full_like(c["q"], 7.0)
    getattr(ops(), kernel)(c["q"], c["kc"], c["vc"], c["table"], dev(tile_seq), dev(tile_q0), dev(np.arange(len(seqs), dtype=np.int32)),
                           dev(np.array([s for s, _ in seqs], dtype=np.int32)), dev(q_lens), dev(cu), out, num_heads=heads,
                           num_kv_heads=kv_heads, head_dim=dim, scale=0.2, window=None, chunk=chunk, sinks=c["sink"])
    ops().tc_status_check(DEV)
    close(f64(out), c["want"], 1.2e-2, kernel)
    gate = rng.normal(size=(len(c["rows"]), heads))
    ops().head_gate(out, f32(gate), heads, dim)
    gated = c["want"].reshape(len(c["rows"]), heads, dim) * pf.sigmoid(gate.astype(np.float32))[:, :, None]
    close(f64(out), gated.reshape(len(c["rows"]), -1), 1.6e-2, "head gate")


@pytest.mark.parametrize("experts,top", [(8, 3), (5, 1), (4, 4), (40, 6), (300, 2)])
def test_softmax_scores_and_the_floor_under_their_sum(experts, top):
    rng = np.random.default_rng(experts)
    tokens = 33
    logits = rng.normal(size=(tokens, experts)) * 3.0
    ids = torch.empty((tokens, top), dtype=torch.int32, device=DEV)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=DEV)
    o = ops()
    o.router_topk(f32(logits), None, top, 1 | o.ROUTE_SOFTMAX | o.ROUTE_FLOOR, 1.0, ids, weights)
    z = logits.astype(np.float32).astype(np.float64)
    s = np.exp(z - z.max(axis=1, keepdims=True))
    s /= s.sum(axis=1, keepdims=True)
    order = np.argsort(-s, axis=1, kind="stable")[:, :top]
    assert np.array_equal(ids.cpu().numpy(), order)
    picked = np.take_along_axis(s, order, axis=1)
    close(f64(weights), picked / (picked.sum(axis=1, keepdims=True) + 1e-20), 5e-6, "weights")


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


def plain_run(name, length, seed):
    """(logits, [(experts, margins) of every run with experts]) of the plain model."""
    key = (name, length, seed)
    if key not in _PLAIN:
        config, weights = plain_weights(name)
        picks = []
        _PLAIN[key] = (pf.forward(config, weights, request_tokens(name, length, seed), picks=picks), picks)
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


class Routes:
    """Collects the experts the engine uses, run by run, while steps run directly (``on_route`` is called by every
    routed feed-forward with the ids of the step's rows)."""

    def __init__(self, lm):
        self.parts = [block.feed_forward for block in lm.model.blocks if block.feed_forward is not None]
        self.step = []

    def __enter__(self):
        for part in self.parts:
            part.on_route = lambda ids: self.step.append(ids.cpu().numpy().copy())
        return self

    def __exit__(self, *exc):
        for part in self.parts:
            part.on_route = None
        return False


def run_schedule(lm, requests, steps, routes=None):
    """``steps``: lists of (request, first position, end position); every place is wanted.  A request gets its slot
    at its first step and gives it back after its last token.  Returns request -> logits [length, vocab] and, with
    ``routes``, request -> the experts used, per run [length, top]."""
    engine = lm.engine
    slots, rows_of, used = {}, {key: [] for key in requests}, {key: None for key in requests}
    for step in steps:
        for key, lo, hi in step:
            if key not in slots:
                slots[key] = engine.new_sequence()
        if routes is not None:
            routes.step.clear()
        out = engine.step([slots[k] for k, _, _ in step], [requests[k][lo:hi] for k, lo, hi in step],
                          [list(range(hi - lo)) for _, lo, hi in step]).float().cpu().numpy()
        at = 0
        for key, lo, hi in step:
            rows_of[key].append(out[at:at + hi - lo])
            if routes is not None:
                if used[key] is None:
                    used[key] = [[] for _ in routes.step]
                for run, ids in enumerate(routes.step):
                    used[key][run].append(ids[at:at + hi - lo])
            at += hi - lo
            if hi == len(requests[key]):
                engine.release(slots.pop(key))
    engine.check()
    engine.cache.check()
    assert not slots
    logits = {key: np.concatenate(parts) for key, parts in rows_of.items()}
    if routes is None:
        return logits, None
    return logits, {key: [np.concatenate(parts) for parts in runs] for key, runs in used.items()}


def check_request(name, dtype, length, seed, got, used, what):
    """float32: against the plain model as it is.  bfloat16: against the plain model made to use the experts the engine
    used, and the engine's experts against the plain model's own, which may differ only where the scores are close."""
    plain, picks = plain_run(name, length, seed)
    if dtype == "float32":
        model_close(got, plain, dtype, what)
        return
    config, weights = plain_weights(name)
    forced = pf.forward(config, weights, request_tokens(name, length, seed), forced=used)
    model_close(got, forced, dtype, what)
    for run, ((own, margins), theirs) in enumerate(zip(picks, used)):
        differs = (np.sort(own, axis=-1) != np.sort(theirs, axis=-1)).any(axis=-1)
        if run == 0:                          # later runs read a stream that an earlier run's other choice has changed
            assert not (differs & (margins > ROUTE_MARGIN)).any(), f"{what}: other experts than the plain model's where the scores are apart"


def through(name, dtype, requests, steps, seeds, what):
    lm = loaded(name, dtype, record_steps=dtype == "float32")
    if dtype == "float32":
        got, used = run_schedule(lm, requests, steps)
    else:
        with Routes(lm) as routes:
            got, used = run_schedule(lm, requests, steps, routes)
    for key, ids in requests.items():
        check_request(name, dtype, len(ids), seeds[key], got[key], used[key] if used else None, f"model {name}, {what}, request {key}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts(name, dtype):
    for length, seed in ((1, 0), (2, 1), (63, 2), (64, 3), (65, 4), (300, 5)):
        through(name, dtype, {"r": request_tokens(name, length, seed)}, [[("r", 0, length)]], {"r": seed}, f"{length} tokens whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_prompt_then_token_by_token(name, dtype):
    length, tail = 250, 120                 # the decoded tokens cross page borders (64) and the edges of every chunk size
    steps = [[("r", 0, length - tail)]] + [[("r", p, p + 1)] for p in range(length - tail, length)]
    through(name, dtype, {"r": request_tokens(name, length, 6)}, steps, {"r": 6}, f"last {tail} tokens one by one")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_a_sequence_decoded_from_its_first_token(name, dtype):
    length = 140
    through(name, dtype, {"r": request_tokens(name, length, 7)}, [[("r", p, p + 1)] for p in range(length)], {"r": 7},
            "one token a step from the start")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("portion", [2, 3, 17, 64, 65])
def test_prompts_in_portions(name, dtype, portion):
    length = 135
    steps = [[("r", lo, min(lo + portion, length))] for lo in range(0, length, portion)]
    through(name, dtype, {"r": request_tokens(name, length, 8)}, steps, {"r": 8}, f"portions of {portion}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_requests_in_one_batch_then_decoded_together_over_reused_slots(name, dtype):
    for turn in range(2):                 # the second turn takes the slots, pages and states the first gave back
        lengths = {"a": 1 + 30, "b": 70 + 30, "c": 200 + 30, "d": 64 + 12, "e": 129 + 5} if turn == 0 else \
                  {"a": 90 + 25, "b": 3 + 25, "c": 64 + 25}
        tails = {"a": 30, "b": 30, "c": 30, "d": 12, "e": 5} if turn == 0 else {"a": 25, "b": 25, "c": 25}
        seeds = {k: 20 + turn * 10 + i for i, k in enumerate(lengths)}
        requests = {k: request_tokens(name, n, seeds[k]) for k, n in lengths.items()}
        steps = [[(k, 0, lengths[k] - tails[k]) for k in lengths]]
        for t in range(max(tails.values())):
            steps.append([(k, lengths[k] - tails[k] + t, lengths[k] - tails[k] + t + 1) for k in lengths if t < tails[k]])
        through(name, dtype, requests, steps, seeds, f"batch, turn {turn}")


def test_a_long_sequence_decoded_for_hundreds_of_tokens():
    name, length, tail = "B", 700, 400
    steps = [[("r", 0, length - tail)]] + [[("r", p, p + 1)] for p in range(length - tail, length)]
    through(name, "float32", {"r": request_tokens(name, length, 9)}, steps, {"r": 9}, "four hundred tokens one by one")


@pytest.mark.parametrize("name", ["A", "C"])
def test_recorded_decode_steps_equal_direct_ones(name):
    """Five sequences decode in a recorded step of six rows, the last sequence twice: the states, the convolutions' last
    inputs and the cache must come out as if it were there once."""
    results = []
    for record in (False, True):
        lm = loaded(name, "bfloat16", record_steps=record)
        engine = lm.engine
        prompts = [request_tokens(name, n, 40 + i) for i, n in enumerate((5, 64, 1, 30, 100))]
        slots = [engine.new_sequence() for _ in prompts]
        rows = [engine.step(slots, prompts).float().cpu().numpy()]
        for step in range(12):
            tokens = [[(7 * step + 3 * i) % ALL[name][0]["vocab"]] for i in range(len(slots))]
            rows.append(engine.step(slots, tokens).float().cpu().numpy())
        for slot in slots:
            engine.release(slot)
        if record:
            assert engine.steps_replayed > 0
        results.append(np.stack(rows))
    assert np.array_equal(results[0], results[1])


def test_pages_before_the_current_chunk_go_back_to_the_pool():
    lm = loaded("C", "float32")                       # chunks of 128 and 192 positions
    engine = lm.engine
    slot = engine.new_sequence()
    engine.step([slot], [request_tokens("C", 700, 50)])
    held = {group.chunk: group.pool.num_held for group in engine.cache.groups}
    assert held == {128: (700 - 640 + 63) // 64, 192: (700 - 576 + 63) // 64}
    engine.release(slot)
    engine.cache.check()
    assert all(group.pool.num_held == 0 for group in engine.cache.groups)


def test_greedy_generation_through_the_entry_point():
    name = "A"
    config, weights = plain_weights(name)
    lm = loaded(name, "float32")
    prompts = [request_tokens(name, n, 60 + i) for i, n in enumerate((9, 1, 70))]
    got = lm.generate_batch(prompts, max_tokens=14, ignore_eos=True)
    for prompt, tokens in zip(prompts, got):
        ids = list(prompt)
        for _ in range(14):
            row = pf.forward(config, weights, ids)[-1]
            top2 = np.sort(row)[-2:]
            assert top2[1] - top2[0] > 1e-4, "a near tie: the case does not pin the greedy choice"
            ids.append(int(np.argmax(row)))
        assert tokens == ids[len(prompt):]
    assert lm.generate(prompts[0], 5) == got[0][:5]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_trace_replayed_through_the_runner(tmp_path, dtype):
    """bin/trace_run as a user drives it: a batch of three prompts of unequal lengths (one of a single token, one of
    which nothing is wanted), decoded together while the shorter requests end, then another batch in the freed slots."""
    name = "D"                            # no close call among its routers: both of its two experts are always used
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
        plain = plain_run(name, n, 70 + i)[0]
        got = np.stack([out[s][row] for s, row, _ in rows[k]])
        model_close(got, plain[[pos for _, _, pos in rows[k]]], dtype, f"request {k}")


def test_command_line_generates_with_the_design(tmp_path):
    """`python -m fieldrun_b200 random` writes a model of the design from a config.json, and the command line
    generates from it what the plain model's greedy loop gives."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(ALL["D"][0]))
    folder = tmp_path / "model"
    made = subprocess.run([sys.executable, "-m", "fieldrun_b200", "random", "--config", str(config_path), "--seed", "9", "--std", "0.2",
                           "--bias-std", "0.3", "-o", str(folder)], capture_output=True, text=True, cwd=root, timeout=300)
    assert made.returncode == 0, made.stderr
    with open(folder / "config.json") as handle:
        config = json.load(handle)
    from fieldrun_b200.weights.safetensors_io import ModelFolder
    files = ModelFolder(str(folder))
    weights = {n: files.tensor(n).double().numpy() for n in files.entries}
    files.close()
    ids = request_tokens("D", 20, 90)
    (tmp_path / "ids.json").write_text(json.dumps(ids))
    run = subprocess.run([sys.executable, "-m", "fieldrun_b200", "--model", str(folder), "--ids", str(tmp_path / "ids.json"), "--ctx", "12",
                          "--generate", "6", "--dtype", "float32", "--eos", "none"], capture_output=True, text=True, cwd=root, timeout=600)
    assert run.returncode == 0, run.stderr
    want = ids[:12]
    for _ in range(6):
        want.append(int(np.argmax(pf.forward(config, weights, want)[-1])))
    assert " ".join(str(t) for t in want[12:]) in run.stdout, run.stdout
