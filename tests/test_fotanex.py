"""The Fotanex design without a GPU: its configuration, its plan, the cache's chunks, and the plain implementation
against loops written out element by element."""
import numpy as np
import pytest

import plain_fotanex as pf
from fieldrun_b200.cache import CacheNeed, SequenceCache
from fieldrun_b200.config import ConfigError, FotanexConfig, architecture_for
from fieldrun_b200.engine.model import DecoderModel
from fieldrun_b200.models.fotanex import fotanex_plan
from fotanex_configs import ALL, CONFIG_A, CONFIG_B, CONFIG_D


@pytest.mark.parametrize("name", sorted(ALL))
def test_configuration_reads_back_from_what_it_writes(name):
    raw = ALL[name][0]
    assert architecture_for(raw).name == "Fotanex"
    cfg = FotanexConfig.from_dict(raw)
    assert FotanexConfig.from_dict(cfg.to_json_dict()) == cfg
    assert cfg.to_json_dict()["layers"] == raw["layers"]
    assert cfg.num_hidden_layers == len(raw["layers"])


def test_impossible_configurations_are_refused_by_key():
    def changed(path, value):
        raw = {**CONFIG_A, "layers": [dict(layer, mixer=dict(layer["mixer"])) for layer in CONFIG_A["layers"]], "loop": dict(CONFIG_A["loop"])}
        node = raw
        for piece in path[:-1]:
            node = node[piece]
        node[path[-1]] = value
        return raw
    for path, value, word in ((("loop", "stop"), 9, "loop"), (("loop", "times"), 0, "times"), (("layers", 0, "type"), "gru", "type"),
                              (("layers", 2, "mixer", "blocks"), 7, "blocks"), (("layers", 0, "mixer", "groups"), 2, "groups"),
                              (("norm",), {"eps": 0}, "eps"), (("vocab",), "many", "vocab")):
        with pytest.raises(ConfigError, match=word):
            FotanexConfig.from_dict(changed(path, value))
    plain = changed(("layers", 1, "mixer"), {"left": {"heads": 2, "dim": 8}, "right": dict(CONFIG_A["layers"][1]["mixer"]["right"])})
    left = FotanexConfig.from_dict(plain).layers[1].mixer.left
    assert (left.kv_heads, left.vdim, left.chunk, left.scale) == (2, 8, None, 8 ** -0.5)      # what a file may leave out
    raw = changed(("layers", 1, "mlp"), {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 2, "top": 3}})
    with pytest.raises(ConfigError, match="top"):
        FotanexConfig.from_dict(raw)


def test_plan_runs_the_loop_with_a_cache_line_per_run_and_a_connector_per_pass():
    plan = fotanex_plan(FotanexConfig.from_dict(CONFIG_A))
    assert [r.layer for r in plan.run_order] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [r.cache_line for r in plan.run_order] == list(range(8))
    assert [r.connector for r in plan.run_order] == [None, (0, 0), None, (0, 1), None, (0, 2), None, None]
    assert [c.kind for c in plan.connectors] == ["stream_reentry"]
    assert pf.run_order(CONFIG_A) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert plan.layers[2].feed_forward is None and plan.layers[2].feed_forward_norm is None
    flat = fotanex_plan(FotanexConfig.from_dict(CONFIG_B))
    assert flat.connectors == () and [r.layer for r in flat.run_order] == [0, 1, 2, 3]
    assert pf.run_order(CONFIG_D) == [(0, 0), (0, 1), (1, None)]


def test_model_names_its_tensors_and_its_cache_lines():
    model = DecoderModel(fotanex_plan(FotanexConfig.from_dict(CONFIG_A)), "float32")
    names = {need.name: tuple(need.shape) for need in model.tensor_needs()}
    assert names["loop.in"] == (96, 192) and names["loop.step"] == (3, 96)
    assert names["l0.norm1.alpha"] == () and names["final.norm.b"] == (96,)
    assert names["l1.mix.left.sink"] == (4,) and names["l1.mix.left.g"] == (4, 96) and names["l1.mix.right.out"] == (96,)
    assert names["l3.mix.right.A_log"] == (70, 40) and names["l3.mix.right.x"] == (3 + 80, 70) and names["l3.mix.right.dt"] == (70, 3)
    assert names["l2.mix.ra"] == (1, 64, 64) and names["l2.mix.conv"] == (64, 5)
    assert names["l0.mix.in"] == (2 * 60 + 2 * 10 + 3, 96) and names["l0.mix.conv"] == (60 + 20, 3)
    assert "l2.norm2" not in names and "l2.mlp.router" not in names
    assert names["l3.mlp.e7.down"] == (96, 56)
    needs = model.cache_needs()
    assert needs[0] == CacheNeed(state_shape=(2, 3 * 10 * 20 + 2 * 80))
    assert needs[1] == CacheNeed(kv_heads=4, head_dim=24, chunk=48, state_shape=(2, 112 * 8 + 112))
    assert needs[1] == needs[3] == needs[5] and needs[2] == needs[4] == CacheNeed(state_shape=(2, 64 + 4 * 64))
    assert needs[7].value_dim == 40 and needs[7].chunk == 100
    assert model.replayable and "scans" in model.kernel_groups() and "recurrent" not in model.kernel_groups()


def test_cache_gives_back_the_pages_before_the_current_chunk():
    cache = SequenceCache([CacheNeed(kv_heads=1, head_dim=8, chunk=100), CacheNeed(kv_heads=1, head_dim=8)], max_tokens=1024,
                          num_slots=2, allocate=False)
    slot = cache.alloc()
    chunked, whole = cache.groups
    at = 0
    for n in (90, 9, 1, 1, 150, 49, 1, 400):
        cache.begin_step([slot], [n])
        cache.end_step([slot], [n])
        at += n
        first_key = at // 100 * 100                   # the first key the next query can see
        assert int(chunked.first_page[slot]) == first_key // 64
        assert chunked.pool.num_held == (at + 63) // 64 - first_key // 64 and whole.pool.num_held == (at + 63) // 64
        cache.check()
    cache.free(slot)
    assert chunked.pool.num_held == 0 and whole.pool.num_held == 0


# ------------------------------------------------------------------------------------------- the plain implementation

def test_plain_convolution_against_loops():
    rng = np.random.default_rng(0)
    v, taps, bias = rng.normal(size=(9, 3)), rng.normal(size=(3, 4)), rng.normal(size=3)
    got = pf.causal_conv(v, taps, bias)
    for t in range(9):
        for c in range(3):
            want = bias[c] + sum(taps[c, k] * v[t - 3 + k, c] for k in range(4) if t - 3 + k >= 0)
            assert abs(got[t, c] - want) < 1e-12


def test_plain_attention_against_a_mask_written_out():
    rng = np.random.default_rng(1)
    count, heads, groups, dim, vdim, chunk = 23, 4, 2, 5, 3, 7
    q, k, v = rng.normal(size=(count, heads, dim)), rng.normal(size=(count, groups, dim)), rng.normal(size=(count, groups, vdim))
    sink, gate = rng.normal(size=heads), rng.normal(size=(count, heads))
    got = pf.attend_in_chunks(q, k, v, sink, gate, 0.3, chunk)
    for h in range(heads):
        g = h // 2
        for i in range(count):
            e = np.array([np.exp(0.3 * q[i, h] @ k[j, g]) if j <= i and j // chunk == i // chunk else 0.0 for j in range(count)])
            want = (e / (e.sum() + np.exp(sink[h]))) @ v[:, g] / (1.0 + np.exp(-gate[i, h]))
            assert np.abs(got[i, h] - want).max() < 1e-12
    assert np.abs(got[7] - pf.attend_in_chunks(q[7:], k[7:], v[7:], sink, gate[7:], 0.3, chunk)[0]).max() < 1e-12   # a chunk stands alone


def test_plain_recurrences_against_loops():
    rng = np.random.default_rng(2)
    count, inner, n = 6, 3, 4
    x, dt, d = rng.normal(size=(count, inner)), rng.uniform(0.1, 1.0, (count, inner)), rng.normal(size=inner)
    b, c, a_log = rng.normal(size=(count, n)), rng.normal(size=(count, n)), rng.normal(size=(inner, n))
    got = pf.selective_recurrence(x, dt, b, c, a_log, d)
    for ch in range(inner):
        s = np.zeros(n)
        for t in range(count):
            for j in range(n):
                s[j] = np.exp(-dt[t, ch] * np.exp(a_log[ch, j])) * s[j] + dt[t, ch] * x[t, ch] * b[t, j]
            assert abs(got[t, ch] - (s @ c[t] + d[ch] * x[t, ch])) < 1e-12
    u, r, i, lam = rng.normal(size=(count, inner)), rng.uniform(size=(count, inner)), rng.uniform(size=(count, inner)), rng.normal(size=inner)
    got = pf.gated_recurrence(u, r, i, lam)
    for ch in range(inner):
        s = 0.0
        for t in range(count):
            a = np.exp(-8.0 * r[t, ch] * np.log1p(np.exp(lam[ch])))
            s = a * s + np.sqrt(1.0 - a * a) * i[t, ch] * u[t, ch]
            assert abs(got[t, ch] - s) < 1e-12
    heads, vdim, groups = 4, 3, 2
    xs, bs, cs = rng.normal(size=(count, heads, vdim)), rng.normal(size=(count, groups, n)), rng.normal(size=(count, groups, n))
    dts, al, ds = rng.uniform(0.1, 1.0, (count, heads)), rng.normal(size=heads), rng.normal(size=heads)
    got = pf.state_space_recurrence(xs, bs, cs, dts, al, ds)
    for h in range(heads):
        s = np.zeros((n, vdim))
        for t in range(count):
            for j in range(n):
                for e in range(vdim):
                    s[j, e] = np.exp(-np.exp(al[h]) * dts[t, h]) * s[j, e] + dts[t, h] * bs[t, h // 2, j] * xs[t, h, e]
            for e in range(vdim):
                assert abs(got[t, h, e] - (sum(s[j, e] * cs[t, h // 2, j] for j in range(n)) + ds[h] * xs[t, h, e])) < 1e-12
    y, w = rng.normal(size=(5, 12)), rng.normal(size=12)
    got = pf.group_rms(y, w, 3, 1e-5)
    for t in range(5):
        for part in range(3):
            cols = slice(4 * part, 4 * part + 4)
            assert np.abs(got[t, cols] - y[t, cols] / np.sqrt((y[t, cols] ** 2).mean() + 1e-5) * w[cols]).max() < 1e-12


def test_plain_experts_and_forced_choices():
    rng = np.random.default_rng(3)
    h, router = rng.normal(size=(7, 6)), rng.normal(size=(5, 6))
    experts = [(rng.normal(size=(4, 6)), rng.normal(size=(4, 6)), rng.normal(size=(6, 4))) for _ in range(5)]
    out, picked, margins = pf.routed_experts(h, router, experts, 2)
    for t in range(7):
        z = router @ h[t]
        s = np.exp(z) / np.exp(z).sum()
        order = sorted(range(5), key=lambda e: -s[e])[:2]
        assert list(picked[t]) == order and abs(margins[t] - (s[order[1]] - sorted(s)[-3])) < 1e-12
        want = sum(s[e] / (s[order[0]] + s[order[1]] + 1e-20) * (experts[e][2] @ (pf.silu(experts[e][0] @ h[t]) * (experts[e][1] @ h[t])))
                   for e in order)
        assert np.abs(out[t] - want).max() < 1e-12
    again, used, _ = pf.routed_experts(h, router, experts, 2, forced=picked[:, ::-1])
    assert np.abs(again - out).max() < 1e-12 and np.array_equal(used, picked[:, ::-1])
    other, _, _ = pf.routed_experts(h, router, experts, 2, forced=(picked + 1) % 5)
    assert np.abs(other - out).max() > 1e-3
