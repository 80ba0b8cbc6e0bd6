"""Small configurations of the Bakasun design for the tests, with random weights of a spread that makes every
mechanism matter.  They differ from one another in every size, in the order of the layers and in every constant:
windows of 5 to 200 keys over pages of 64; rotations over a part of a head and over all of it, with and without scaled
angles; caps of 3 to 30 on the scores, and none; key heads shared by one, two, three and four query heads; key and value
sizes that differ; delta-rule heads of 8 x 12 up to 128 x 64 with one to five taps; experts in one group, in groups of
which one or several stay, groups of a single expert; one expert of six, all four of four; layers with a dense unit,
with experts without a shared one, and without feed-forward.  ``C`` has sizes that the tensor-core kernels take."""
import functools
import json
import os
import tempfile

import numpy as np

import fieldrun_b200 as fr
from fieldrun_b200 import RandomInit
from fieldrun_b200.weights.safetensors_io import ModelFolder


def rot(base, dims, factor=None):
    out = {"base": base, "dims": dims}
    if factor is not None:
        out["scaling"] = {"factor": factor}
    return out


def attn(heads, kv_heads, dim, vdim, scale, window=None, rotation=None, softcap=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        out["mask"] = {"size": window}
    if rotation is not None:
        out["rot"] = rotation
    if softcap is not None:
        out["softcap"] = softcap
    return out


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def attention(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def parallel(left, right, left_scale, right_scale, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=None, keep=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups, "keep": keep}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


CONFIG_A = {
    "architecture": "Bakasun", "vocab": 131, "width": 96, "norm": {"eps": 1e-5},
    "layers": [
        parallel(attn(4, 2, 24, 40, 0.21, 33, rot(5000.0, 16, 2.5), 6.0), delta(4, 2, 20, 12, 3), 0.7, 0.4, moe(6, 2, 40, 3, 2, 24)),
        attention(attn(6, 2, 16, 16, 0.3, 100, rot(10000.0, 16)), dense(80)),
        attention(attn(3, 3, 32, 8, 0.17, 64, rot(300.0, 8)), moe(4, 4, 48)),
        parallel(attn(3, 1, 20, 20, 0.25, 5, rot(20000.0, 20, 8.0), 3.0), delta(3, 3, 8, 16, 5), 1.2, 0.9, None),
    ],
}
INIT_A = RandomInit(seed=31, matrix_std=0.1, norm_std=0.2, bias_std=0.4)

CONFIG_B = {
    "architecture": "Bakasun", "vocab": 77, "width": 40, "norm": {"eps": 1e-6},
    "layers": [
        attention(attn(4, 1, 12, 20, 0.3, 130, rot(1000.0, 12)), moe(6, 1, 24, 6, 3, 16)),
        parallel(attn(2, 2, 36, 12, 0.16, 65, None, 30.0), delta(2, 1, 40, 36, 1), 0.5, 1.5, moe(8, 3, 16, 4, 2)),
        attention(attn(5, 5, 8, 8, 0.4), None),
        parallel(attn(8, 2, 10, 14, 0.33, 200, rot(777.0, 10, 1.5)), delta(1, 1, 12, 8, 2), 1.0, 1.0, dense(56)),
    ],
}
INIT_B = RandomInit(seed=32, matrix_std=0.16, norm_std=0.1, bias_std=0.6)

CONFIG_C = {
    "architecture": "Bakasun", "vocab": 200, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        attention(attn(4, 2, 64, 64, 0.125, 100, rot(10000.0, 64)), moe(8, 2, 128, 4, 2, 128)),
        parallel(attn(4, 1, 128, 128, 0.09, 192, rot(50000.0, 64, 4.0), 10.0), delta(2, 1, 128, 64, 4), 0.6, 0.5, dense(256)),
        parallel(attn(2, 2, 64, 64, 0.125, 70, rot(10000.0, 32), 20.0), delta(4, 2, 64, 128, 4), 0.8, 0.3, moe(4, 2, 128, 2, 1, 256)),
        attention(attn(8, 2, 32, 32, 0.18, 136, rot(10000.0, 32)), dense(128)),
    ],
}
INIT_C = RandomInit(seed=33, matrix_std=0.07, norm_std=0.1, bias_std=0.3)

CONFIG_D = {
    "architecture": "Bakasun", "vocab": 64, "width": 32, "norm": {"eps": 1e-5},
    "layers": [
        parallel(attn(2, 2, 8, 8, 0.4, 7, rot(100.0, 8), 4.0), delta(2, 2, 8, 8, 4), 0.6, 0.5, moe(2, 2, 16, None, None, 8)),
        attention(attn(2, 1, 16, 8, 0.3, 48, rot(100.0, 4)), dense(24)),
    ],
}
INIT_D = RandomInit(seed=34, matrix_std=0.2, norm_std=0.1, bias_std=0.5)

ALL = {"A": (CONFIG_A, INIT_A), "B": (CONFIG_B, INIT_B), "C": (CONFIG_C, INIT_C), "D": (CONFIG_D, INIT_D)}

_ROOT = tempfile.mkdtemp(prefix="fieldrun_b200_bakasun_")


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
    return np.random.default_rng(7321 * seed + length).integers(0, vocab, size=length).tolist()
