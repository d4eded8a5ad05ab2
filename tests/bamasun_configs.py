"""Small configurations of the Bamasun design for the tests, with random weights of a spread that makes every
mechanism matter.  They differ from one another in every size, in the order of the layers and in every constant:
a recurrent layer first or in the middle, key and value heads of unequal sizes, groups of one, two and three
query heads per key head, a layer without feed-forward, a layer that reads another layer's keys and values with
a scale and a temperature of its own, temperatures that step every 7 or 64 positions or are absent, logits with and
without a cap.  ``C`` has sizes that the tensor-core attention kernels take."""
import functools
import json
import os
import tempfile

import numpy as np

import fieldrun_b200 as fr
from fieldrun_b200 import RandomInit
from fieldrun_b200.weights.safetensors_io import ModelFolder


def attention(heads, kv_heads, dim, vdim, scale, q_temp=None, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if q_temp is not None:
        mixer["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return mixer


def layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


CONFIG_A = {
    "architecture": "Bamasun", "vocab": 131, "width": 96, "embedding": {"scale": 3.5}, "norm": {"eps": 1e-5},
    "logit_softcap": 12.0,
    "layers": [
        layer("gla", {"heads": 2, "dim": 16, "vdim": 24, "tau": 4.0, "rank": 5}, 160),
        layer("attention", attention(6, 2, 32, 16, 0.21, q_temp=(0.5, 7)), None),
        layer("attention", attention(6, 2, 32, 16, 0.3, kv_from=1), 64),
        layer("gla", {"heads": 3, "dim": 8, "vdim": 8, "tau": 1.0, "rank": 3}, 100),
        layer("attention", attention(3, 3, 24, 40, 0.2, q_temp=(0.25, 64)), 72),
    ],
}
INIT_A = RandomInit(seed=3, matrix_std=0.08, norm_std=0.2, bias_std=0.3)

CONFIG_B = {
    "architecture": "Bamasun", "vocab": 77, "width": 40, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
    "layers": [
        layer("attention", attention(4, 1, 12, 20, 0.4, q_temp=(1.0, 3)), 56),
        layer("attention", attention(2, 1, 12, 20, 0.25, kv_from=0), None),
        layer("gla", {"heads": 1, "dim": 20, "vdim": 12, "tau": 8.0, "rank": 2}, None),
        layer("attention", attention(4, 1, 12, 20, 0.4, q_temp=(0.1, 50), kv_from=0), 48),
    ],
}
INIT_B = RandomInit(seed=4, matrix_std=0.15, norm_std=0.1, bias_std=0.5)

CONFIG_C = {
    "architecture": "Bamasun", "vocab": 200, "width": 128, "embedding": {"scale": 6.0}, "norm": {"eps": 1e-6},
    "logit_softcap": 25.0,
    "layers": [
        layer("attention", attention(4, 2, 64, 64, 0.125, q_temp=(0.3, 32)), 192),
        layer("gla", {"heads": 2, "dim": 64, "vdim": 64, "tau": 16.0, "rank": 8}, 192),
        layer("attention", attention(4, 2, 64, 64, 0.11, q_temp=(0.3, 32), kv_from=0), 128),
        layer("attention", attention(2, 1, 128, 128, 0.09), 128),
    ],
}
INIT_C = RandomInit(seed=5, matrix_std=0.06, norm_std=0.1, bias_std=0.2)

ALL = {"A": (CONFIG_A, INIT_A), "B": (CONFIG_B, INIT_B), "C": (CONFIG_C, INIT_C)}

_ROOT = tempfile.mkdtemp(prefix="fieldrun_b200_bamasun_")


@functools.lru_cache(maxsize=None)
def model_folder(name: str) -> str:
    config, init = ALL[name]
    folder = os.path.join(_ROOT, name)
    fr.write_random_model(folder, config, init)
    return folder


@functools.lru_cache(maxsize=None)
def plain_weights(name: str):
    """(config.json as a dictionary, tensors as float64 arrays by name) of the written folder."""
    folder = model_folder(name)
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as handle:
        config = json.load(handle)
    files = ModelFolder(folder)
    try:
        weights = {n: files.tensor(n).double().numpy() for n in files.entries}
    finally:
        files.close()
    return config, weights


def request_tokens(name: str, length: int, seed: int) -> list[int]:
    vocab = ALL[name][0]["vocab"]
    return np.random.default_rng(7919 * seed + length).integers(0, vocab, size=length).tolist()
