"""Small configurations of the Depelix design for the tests, with random weights of a spread that makes every mechanism
matter.  They differ from one another in every size, in the order of the layers and in every constant: windows of 5,
33, 50, 64 and 130 positions (pages hold 64); a layer that reads another layer's latents through a window of its own,
narrower or wider than the writer's; two readers of one line; a rotation over a part of the rotated entries only; one head; one expert of five, all four of four, two of six; a layer without feed-forward; a
model without pair table and one without token input.  ``C`` has sizes that the tensor-core kernel takes."""
import functools
import json
import os
import tempfile

import numpy as np

import fieldrun_b200 as fr
from fieldrun_b200 import RandomInit
from fieldrun_b200.weights.safetensors_io import ModelFolder


def moe(experts, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def mixer(heads, dim, rot_dim, vdim, kv_rank, q_rank, base, scale, window=None, kv_from=None, rot_dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def windowed(mlp, *args, **kwargs):
    return {"type": "latent_attention", "mixer": mixer(*args, **kwargs), "mlp": mlp}


def causal(mlp, *args, **kwargs):
    return {"type": "latent_attention_2", "mixer": mixer(*args, **kwargs), "mlp": mlp}


CONFIG_A = {
    "architecture": "Depelix", "vocab": 131, "width": 96, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 61, "mul_prev": 5, "mul_cur": 11}}, "token_side": {"dim": 8},
    "layers": [
        windowed(moe(5, 1, 48, 0.7), 3, 24, 8, 20, 40, 48, 10000.0, 0.2, window=50),
        windowed(dense(72), 5, 16, 8, 12, 40, 36, 10000.0, 0.25, window=33, kv_from=0),
        causal(None, 2, 16, 12, 28, 24, 30, 500.0, 0.3),
        windowed(moe(6, 2, 40, 1.5), 3, 8, 8, 20, 40, 20, 10000.0, 0.3, window=130, kv_from=0),
        causal(moe(4, 4, 24, 0.4), 4, 12, 6, 10, 18, 44, 30000.0, 0.22, rot_dims=4),
    ],
}
INIT_A = RandomInit(seed=23, matrix_std=0.07, norm_std=0.2, bias_std=0.4)

CONFIG_B = {
    "architecture": "Depelix", "vocab": 77, "width": 40, "norm": {"eps": 1e-6},
    "token_side": {"dim": 5},
    "layers": [
        causal(dense(56), 1, 20, 10, 36, 33, 24, 100.0, 0.18),
        windowed(moe(3, 2, 24, 2.0), 4, 8, 16, 12, 20, 28, 2000.0, 0.25, window=5),
        windowed(None, 2, 12, 4, 16, 20, 16, 2000.0, 0.25, window=64),
    ],
}
INIT_B = RandomInit(seed=24, matrix_std=0.09, norm_std=0.1, bias_std=0.5)

CONFIG_C = {
    "architecture": "Depelix", "vocab": 200, "width": 128, "norm": {"eps": 1e-6},
    "embedding": {"bigram": {"buckets": 1021, "mul_prev": 100003, "mul_cur": 7919}},
    "layers": [
        causal(moe(8, 2, 128, 1.0), 8, 32, 32, 32, 64, 64, 10000.0, 0.125),
        windowed(dense(256), 16, 64, 64, 64, 128, 96, 10000.0, 0.09, window=100),
        windowed(moe(4, 1, 256, 3.0), 4, 32, 64, 48, 128, 64, 10000.0, 0.1, window=256, kv_from=1),
        causal(dense(128), 2, 16, 16, 16, 32, 32, 50000.0, 0.18),
    ],
}
INIT_C = RandomInit(seed=25, matrix_std=0.07, norm_std=0.1, bias_std=0.3)

ALL = {"A": (CONFIG_A, INIT_A), "B": (CONFIG_B, INIT_B), "C": (CONFIG_C, INIT_C)}

_ROOT = tempfile.mkdtemp(prefix="fieldrun_b200_depelix_")


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
    return np.random.default_rng(7219 * seed + length).integers(0, vocab, size=length).tolist()
