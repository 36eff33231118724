"""Small Venizen configurations for the tests (sizes of their own, each unlike the
others in head counts, head sizes, windows, rotation, loop and layer order) and
helpers to write them as model folders with random weights."""
from __future__ import annotations

import functools
import os
import tempfile

import torch


def parallel_layer(left: dict, right: dict, ff, left_scale=0.7, right_scale=1.3) -> dict:
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale,
                                          "right_scale": right_scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta_layer(heads: int, dim: int, rank: int, ff) -> dict:
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def attention(heads, kv_heads, dim, vdim, window, keep_first, rot_dims, base=10000.0, scale=None) -> dict:
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "mask": {"size": window, "keep_first": keep_first}, "rot": {"base": base, "dims": rot_dims},
            "scale": scale if scale is not None else dim ** -0.5}


def retention(heads, dim, vdim, decay, rot_dims, base=10000.0) -> dict:
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": {"base": base, "dims": rot_dims}}


CONFIGS = {
    # a delta layer first, a span of two layers run three times from layer 0, value heads
    # narrower and wider than key heads, partial rotation, a window shorter than what it keeps
    "P": {"architecture": "Venizen", "vocab": 300, "width": 64, "norm": {"eps": 1e-5},
          "layers": [delta_layer(2, 16, 8, 96),
                     parallel_layer(attention(4, 4, 16, 24, 20, 3, 8, scale=0.9),
                                    retention(3, 16, 8, [0.9, 0.99, 0.5], 16), None),
                     parallel_layer(attention(4, 1, 32, 32, 7, 9, 32, base=500.0, scale=0.6),
                                    retention(1, 48, 40, [0.97], 0), 72, left_scale=1.0, right_scale=0.25)],
          "loop": {"start": 0, "stop": 2, "times": 3}},
    # no loop, two delta layers in a row (one with a key size that is no power of two), windows on
    # page borders, one head
    "Q": {"architecture": "Venizen", "vocab": 257, "width": 96, "norm": {"eps": 3e-6},
          "layers": [parallel_layer(attention(2, 2, 8, 8, 16, 1, 4, scale=1.5),
                                    retention(2, 8, 8, [1.0, 0.75], 8, base=77.0), 40),
                     delta_layer(1, 40, 5, None),
                     delta_layer(3, 8, 16, 200),
                     parallel_layer(attention(6, 2, 16, 16, 32, 16, 16, scale=0.8),
                                    retention(2, 64, 16, [0.999, 0.9], 32), None)],
          "loop": {"start": 2, "stop": 3, "times": 1}},
    # head sizes of 64 and 128, the loop over the last layers, a long window
    "R": {"architecture": "Venizen", "vocab": 512, "width": 128, "norm": {"eps": 1e-6},
          "layers": [parallel_layer(attention(4, 2, 64, 64, 100, 4, 64, base=1e6, scale=0.4),
                                    retention(2, 64, 64, [0.95, 0.999], 64, base=1e5), 256),
                     delta_layer(2, 64, 32, None),
                     parallel_layer(attention(2, 1, 128, 64, 48, 0, 32, scale=0.3),
                                    retention(1, 128, 128, [0.99], 64), 192),
                     delta_layer(1, 128, 16, 128)],
          "loop": {"start": 2, "stop": 4, "times": 2}},
    # sizes that fit no vector width: an odd vocabulary, a width that is no multiple of 8, head
    # sizes of 6, 5, 10 and 3, three heads on one key/value head
    "S": {"architecture": "Venizen", "vocab": 101, "width": 100, "norm": {"eps": 2e-5},
          "layers": [parallel_layer(attention(3, 1, 6, 5, 9, 2, 2, scale=0.7), retention(1, 10, 3, [0.8], 6), 50),
                     delta_layer(2, 6, 3, None)],
          "loop": {"start": 0, "stop": 2, "times": 2}},
    # four key/value heads of 128: in 32-bit a tile's keys and values of all of them do not fit in
    # shared memory at once, so the attention walks them in passes
    "T": {"architecture": "Venizen", "vocab": 128, "width": 64, "norm": {"eps": 1e-6},
          "layers": [parallel_layer(attention(4, 4, 128, 128, 40, 2, 128, scale=0.2), retention(1, 16, 16, [0.9], 16), None)],
          "loop": {"start": 0, "stop": 0, "times": 1}},
}
INIT = {"P": dict(seed=3, sigma=0.15, norm_jitter=0.2), "Q": dict(seed=5, sigma=0.12, norm_jitter=0.1),
        "R": dict(seed=9, sigma=0.08, norm_jitter=0.15), "S": dict(seed=12, sigma=0.2, norm_jitter=0.1),
        "T": dict(seed=14, sigma=0.1, norm_jitter=0.1)}

_tmp = tempfile.TemporaryDirectory(prefix="kipp_b200_venizen_")


def write_folder(folder: str, cfg: dict, init: dict, dtype=torch.float32) -> str:
    from kipp_b200.config import config_from_dict
    from kipp_b200.weights import write_random_model
    return write_random_model(folder, config_from_dict(cfg), init["seed"], sigma=init["sigma"],
                              norm_jitter=init["norm_jitter"], dtype=dtype)


@functools.lru_cache(maxsize=None)
def model_folder(name: str) -> str:
    return write_folder(os.path.join(_tmp.name, name), CONFIGS[name], INIT[name])


def random_tokens(vocab: int, n: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
