"""Small configurations of the Fotanex design for the tests, with random weights of a spread that makes every
mechanism matter.  They differ from one another in every size, in the order of the layers and in every constant:
a loop over the middle layers, over the first ones, a loop that runs once, and no loop; one block or several in the
recurrent unit; a convolution of one tap (no convolution state) up to five; states smaller and larger than what one
thread keeps; value sizes that are no multiple of 32; one, two and four groups; key heads shared by one, two or three
query heads; chunks of 48, 100 and 128 positions (pages hold 64); one expert of five, all four of four, two of eight;
a layer without feed-forward.  ``C`` has sizes that the tensor-core kernels take."""
import functools
import json
import os
import tempfile

import numpy as np

import fieldrun_b200 as fr
from fieldrun_b200 import RandomInit
from fieldrun_b200.weights.safetensors_io import ModelFolder


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def rglru(width, blocks, conv, mlp):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}, "mlp": mlp}


def mamba2(heads, vdim, state, groups, norm_groups, conv, mlp):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups,
                                        "norm_groups": norm_groups, "conv": conv}, "mlp": mlp}


def parallel(heads, kv_heads, dim, vdim, scale, chunk, inner, state, dt_rank, conv, mlp):
    return {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": chunk}},
        "right": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}, "mlp": mlp}


CONFIG_A = {
    "architecture": "Fotanex", "vocab": 131, "width": 96, "norm": {"eps": 1e-5},
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        mamba2(3, 20, 10, 1, 1, 3, moe(5, 1, 48)),
        parallel(4, 4, 24, 24, 0.2, 48, 112, 8, 5, 2, moe(4, 4, 40)),
        rglru(64, 1, 5, None),
        parallel(6, 2, 16, 40, 0.3, 100, 70, 40, 3, 4, moe(8, 2, 56)),
    ],
}
INIT_A = RandomInit(seed=13, matrix_std=0.09, norm_std=0.2, bias_std=0.4)

CONFIG_B = {
    "architecture": "Fotanex", "vocab": 77, "width": 40, "norm": {"eps": 1e-6},
    "layers": [
        rglru(40, 5, 1, moe(3, 2, 24)),
        mamba2(4, 36, 70, 2, 4, 4, moe(6, 3, 16)),
        parallel(3, 1, 20, 12, 0.35, 64, 48, 17, 2, 3, None),
        rglru(88, 4, 2, moe(2, 1, 64)),
    ],
}
INIT_B = RandomInit(seed=14, matrix_std=0.15, norm_std=0.1, bias_std=0.6)

CONFIG_C = {
    "architecture": "Fotanex", "vocab": 200, "width": 128, "norm": {"eps": 1e-6},
    "loop": {"start": 0, "stop": 2, "times": 1},
    "layers": [
        parallel(4, 2, 64, 64, 0.125, 128, 256, 16, 8, 4, moe(8, 2, 128)),
        mamba2(4, 64, 128, 4, 2, 4, moe(8, 2, 128)),
        parallel(2, 1, 128, 128, 0.09, 192, 128, 16, 4, 4, moe(4, 2, 256)),
    ],
}
INIT_C = RandomInit(seed=15, matrix_std=0.06, norm_std=0.1, bias_std=0.3)

CONFIG_D = {
    "architecture": "Fotanex", "vocab": 64, "width": 32, "norm": {"eps": 1e-5},
    "loop": {"start": 0, "stop": 1, "times": 2},
    "layers": [
        parallel(2, 2, 8, 8, 0.4, 7, 32, 4, 1, 4, moe(2, 2, 16)),
        mamba2(1, 32, 5, 1, 1, 2, None),
    ],
}
INIT_D = RandomInit(seed=16, matrix_std=0.2, norm_std=0.1, bias_std=0.5)

ALL = {"A": (CONFIG_A, INIT_A), "B": (CONFIG_B, INIT_B), "C": (CONFIG_C, INIT_C), "D": (CONFIG_D, INIT_D)}

_ROOT = tempfile.mkdtemp(prefix="fieldrun_b200_fotanex_")


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
    return np.random.default_rng(6151 * seed + length).integers(0, vocab, size=length).tolist()
