"""The Bamasun design without a GPU: its configuration reader, its plan, and the plain implementation checked
against element-wise restatements of its equations."""
import json
import math

import numpy as np
import pytest

import fieldrun_b200 as fr
import plain_bamasun as pb
from bamasun_configs import ALL, CONFIG_A, CONFIG_B, model_folder, plain_weights
from fieldrun_b200.config import BamasunConfig, ConfigError, architecture_for, load_config
from fieldrun_b200.models.bamasun import bamasun_plan, distance_slopes


def test_config_round_trip_and_registry(tmp_path):
    for config, _ in ALL.values():
        cfg = BamasunConfig.from_dict(config)
        assert cfg.vocab_size == config["vocab"] and cfg.hidden_size == config["width"]
        assert cfg.num_hidden_layers == len(config["layers"])
        (tmp_path / "config.json").write_text(json.dumps(cfg.to_json_dict()))
        assert BamasunConfig.from_dict(json.loads((tmp_path / "config.json").read_text())) == cfg
        assert architecture_for(config).name == "Bamasun"
    cfg = BamasunConfig.from_dict(CONFIG_B)
    assert cfg.logit_softcap is None and cfg.layers[1].ff is None and cfg.layers[1].mixer.q_temp_coef is None


def test_config_refusals():
    def changed(path, value):
        raw = json.loads(json.dumps(CONFIG_A))
        node = raw
        for piece in path[:-1]:
            node = node[piece]
        node[path[-1]] = value
        return raw

    for path, value, match in [
        (("layers", 2, "mixer", "kv_from"), 2, "earlier"),
        (("layers", 2, "mixer", "kv_from"), 0, "attention layer"),
        (("layers", 2, "mixer", "vdim"), 24, "do not fit"),
        (("layers", 1, "mixer", "kv_heads"), 4, "multiple"),
        (("layers", 0, "type"), "conv", "'attention' and 'gla'"),
        (("layers", 0, "mlp", "kind"), "moe", "'dense'"),
        (("layers", 1, "mixer", "window"), 128, "does not have"),
        (("norm", "kind"), "rms", "does not have"),
        (("layers", 0, "mixer", "tau"), 0.0, "tau"),
    ]:
        with pytest.raises(ConfigError, match=match):
            BamasunConfig.from_dict(changed(path, value))
    # a note of the file's writer at the top level is no arithmetic: a warning, and the configuration reads as before
    assert BamasunConfig.from_dict(dict(CONFIG_A, seed=7)) == BamasunConfig.from_dict(CONFIG_A)
    # a layer cannot read the keys of a layer that itself reads another's
    raw = changed(("layers", 4, "mixer"), dict(CONFIG_A["layers"][2]["mixer"], kv_from=2))
    with pytest.raises(ConfigError, match="of its own"):
        BamasunConfig.from_dict(raw)


def test_plan_lines_tensors_and_constants():
    cfg = BamasunConfig.from_dict(CONFIG_A)
    plan = bamasun_plan(cfg)
    # the recurrent layers and the attention layers with keys of their own have a line each; layer 2 reads layer 1's
    assert [(r.layer, r.cache_line, r.writes_cache) for r in plan.run_order] == \
        [(0, 0, True), (1, 1, True), (2, 1, False), (3, 2, True), (4, 3, True)]
    assert plan.layers[1].feed_forward is None and plan.layers[1].feed_forward_norm is None
    shared = plan.layers[2].mixer
    assert shared.args["shares_kv"] and shared.args["query_temperature"] is None and shared.args["softmax_scale"] == 0.3
    model = fr.build_model(architecture_for(CONFIG_A), cfg, "float32")
    names = {n.name: tuple(n.shape) for n in model.tensor_needs()}
    assert "l2.mix.k" not in names and "l2.mix.v.b" not in names and "l2.mix.k.norm" not in names
    assert names["l2.mix.q"] == (192, 96) and names["l2.mix.q.norm"] == (192,) and names["l1.mix.v"] == (32, 96)
    assert names["l1.mix.o"] == (96, 96) and names["l4.mix.o"] == (96, 120)
    assert names["l0.mix.a1"] == (5, 96) and names["l0.mix.a2"] == (32, 5) and names["l0.mix.norm"] == (24,)
    assert "l1.norm2" not in names and names["l1.norm1.b"] == (96,) and names["final.norm.b"] == (96,)
    needs = model.cache_needs()
    assert needs[0].state_shape == (2, 2, 16, 24) and needs[1].kv_heads == 2 and needs[1].value_dim == 16
    assert needs[3].head_dim == 24 and needs[3].value_dim == 40
    slopes = distance_slopes(8)
    assert slopes[0] == 0.5 and slopes[-1] == 2.0 ** -8 and np.allclose(slopes, pb.distance_slopes(8))


def test_the_rank_of_the_decay_comes_from_the_tensor(tmp_path):
    folder = model_folder("B")
    raw = json.loads(open(folder + "/config.json").read())
    assert raw["layers"][2]["mixer"].pop("rank") == 2
    import shutil
    shutil.copy(folder + "/model.safetensors", tmp_path / "model.safetensors")
    (tmp_path / "config.json").write_text(json.dumps(raw))
    _, cfg = load_config(str(tmp_path))
    assert cfg.layers[2].mixer.rank == 2
    with pytest.raises(ConfigError, match="rank"):
        bamasun_plan(BamasunConfig.from_dict(raw))


# ---------------------------------------------------------------- the plain implementation against restatements

def test_plain_norms_and_temperature():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(3, 11)) * 2 + 1
    w, b = rng.normal(size=11), rng.normal(size=11)
    got = pb.layer_norm(x, w, b, 1e-3)
    for r in range(3):
        mean = sum(x[r]) / 11
        var = sum((v - mean) ** 2 for v in x[r]) / 11
        for c in range(11):
            assert abs(got[r, c] - ((x[r, c] - mean) / math.sqrt(var + 1e-3) * w[c] + b[c])) < 1e-12
    got = pb.rms_norm(x, w, 1e-3)
    for r in range(3):
        ms = sum(v * v for v in x[r]) / 11
        assert np.allclose(got[r], x[r] / math.sqrt(ms + 1e-3) * w)
    assert pb.query_temperature(0, 0.3, 128) == 1.0 and pb.query_temperature(126, 0.3, 128) == 1.0
    assert abs(pb.query_temperature(127, 0.3, 128) - (1 + 0.3 * math.log(2))) < 1e-15
    assert abs(pb.query_temperature(383, 0.3, 128) - (1 + 0.3 * math.log(4))) < 1e-15


def test_plain_attention_equals_loops():
    config, w = plain_weights("B")
    mixer = config["layers"][0]["mixer"]
    rng = np.random.default_rng(1)
    T = 9
    h = rng.normal(size=(T, config["width"]))
    got, (k, v) = pb.attention_mixer(h, w, "l0.mix.", mixer, 1e-6)
    H, G, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    q = h @ w["l0.mix.q"].T + w["l0.mix.q.b"]
    q = q / np.sqrt((q * q).mean(axis=1, keepdims=True) + 1e-6) * w["l0.mix.q.norm"]
    heads_out = np.zeros((T, H * vdim))
    for i in range(T):
        factor = 1 + mixer["q_temp"]["coef"] * math.log((i + 1) // mixer["q_temp"]["every"] + 1)
        for head in range(H):
            g = head // (H // G)
            qi = q[i, head * dim:(head + 1) * dim] * factor
            s = np.array([qi @ k[j, g] * mixer["scale"] - 2.0 ** (-8 * (head + 1) / H) * (i - j) for j in range(i + 1)])
            p = np.exp(s - s.max())
            p /= p.sum()
            heads_out[i, head * vdim:(head + 1) * vdim] = sum(p[j] * v[j, g] for j in range(i + 1))
    assert np.allclose(got, heads_out @ w["l0.mix.o"].T, atol=1e-10)


def test_plain_gla_equals_the_unrolled_sum_and_carries_its_state():
    config, w = plain_weights("A")
    mixer = config["layers"][0]["mixer"]
    rng = np.random.default_rng(2)
    T = 7
    h = rng.normal(size=(T, config["width"]))
    got, state = pb.gla_mixer(h, w, "l0.mix.", mixer, 1e-5)
    H, dim, vdim = mixer["heads"], mixer["dim"], mixer["vdim"]
    q = (h @ w["l0.mix.q"].T) / math.sqrt(dim)
    k, v = h @ w["l0.mix.k"].T, h @ w["l0.mix.v"].T
    z = (h @ w["l0.mix.a1"].T) @ w["l0.mix.a2"].T + w["l0.mix.a2.b"]
    alpha = (1 / (1 + np.exp(-z))) ** (1 / mixer["tau"])
    o = np.zeros((T, H, vdim))
    for t in range(T):
        for head in range(H):
            c = slice(head * dim, (head + 1) * dim)
            for j in range(t + 1):
                decay = np.prod(alpha[j + 1:t + 1, c], axis=0)            # the decays after token j, up to and with t
                o[t, head] += (q[t, c] * decay) @ k[j, c] * v[j, head * vdim:(head + 1) * vdim]
    o = o / np.sqrt((o * o).mean(axis=-1, keepdims=True) + 1e-5) * w["l0.mix.norm"]
    gate = h @ w["l0.mix.g"].T
    want = (o.reshape(T, -1) * gate / (1 + np.exp(-gate))) @ w["l0.mix.o"].T
    assert np.allclose(got, want, atol=1e-10)
    first, mid = pb.gla_mixer(h[:4], w, "l0.mix.", mixer, 1e-5)
    second, end = pb.gla_mixer(h[4:], w, "l0.mix.", mixer, 1e-5, state=mid)
    assert np.allclose(np.concatenate([first, second]), got) and np.allclose(end, state)


def test_plain_forward_is_causal_and_shares_keys():
    config, w = plain_weights("A")
    ids = list(range(40))
    full = pb.forward(config, w, ids)
    assert np.allclose(pb.forward(config, w, ids[:17]), full[:17], atol=1e-9)
    assert np.abs(full).max() <= config["logit_softcap"]
    # layer 2 reads layer 1's keys: changing layer 1's key projection changes what layer 2 sees
    other = dict(w)
    other["l1.mix.k"] = w["l1.mix.k"] * 1.5
    _, layers_a = pb.forward(config, w, ids, return_layers=True)
    _, layers_b = pb.forward(config, other, ids, return_layers=True)
    assert np.allclose(layers_a[0], layers_b[0]) and not np.allclose(layers_a[1], layers_b[1])
