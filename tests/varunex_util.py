"""Small Varunex configurations for the tests (sizes of their own, each unlike the
others in head counts, head sizes, windows, rotation and layer order) and helpers
to write them as model folders with random weights."""
from __future__ import annotations

import functools
import os
import tempfile

import torch


def ff(n):
    return {"kind": "dense", "ff": n} if n else None


def memory_layer(heads, dim, vdim, cap, mlp) -> dict:
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": ff(mlp)}


def latent_layer(heads, dim, rot_dim, vdim, kv_rank, q_rank, mlp, base=10000.0, scale=None) -> dict:
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "rot": {"base": base, "dims": rot_dim},
                      "scale": scale if scale is not None else (dim + rot_dim) ** -0.5},
            "mlp": ff(mlp)}


def diff_layer(heads, kv_heads, dim, vdim, window, rot_dims, mlp, diff=0.4, base=10000.0, scaling=None, scale=None) -> dict:
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "rot": rot,
             "scale": scale if scale is not None else dim ** -0.5}
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "attention", "mixer": mixer, "mlp": ff(mlp)}


CONFIGS = {
    # attention layers first, two key/value heads under four heads, a rotation of half of every map
    # with all three zones of the stretched wavelengths, a layer without a feed-forward, a
    # differential layer without a window, a memory whose values are wider than its keys
    "A": {"architecture": "Varunex", "vocab": 300, "width": 64, "norm": {"eps": 1e-5},
          "layers": [latent_layer(4, 16, 8, 24, 32, 40, 96),
                     diff_layer(4, 2, 16, 24, 20, 8, None, diff=0.3, scaling=(8.0, 1.0, 4.0, 64)),
                     memory_layer(2, 16, 40, 10.0, 72),
                     diff_layer(2, 2, 8, 8, 0, 8, 48, diff=0.6, base=500.0),
                     latent_layer(2, 8, 16, 8, 16, 24, None, base=300.0, scale=0.5),
                     memory_layer(3, 8, 8, 4.0, None)]},
    # sizes that fit no vector width: an odd vocabulary, a width that is no multiple of 8, three
    # heads on one key/value head, head sizes of 6, 10, 5, 7 and 12, a window of 7
    "B": {"architecture": "Varunex", "vocab": 101, "width": 100, "norm": {"eps": 2e-5},
          "layers": [memory_layer(1, 12, 7, 9.0, 50),
                     diff_layer(3, 1, 10, 6, 7, 4, 30, diff=0.5, scaling=(2.0, 1.0, 2.0, 16)),
                     latent_layer(3, 6, 4, 5, 12, 10, 36, scale=0.8)]},
    # head sizes of 32, 64 and 128, as many key/value heads as heads, a long window, a memory of
    # 64 x 128 per head (several slices of value columns, several threads per column)
    "C": {"architecture": "Varunex", "vocab": 512, "width": 128, "norm": {"eps": 1e-6},
          "layers": [diff_layer(4, 4, 64, 64, 100, 32, 256, diff=0.2, base=2e5, scaling=(4.0, 2.0, 8.0, 256), scale=0.2),
                     latent_layer(4, 32, 16, 32, 64, 48, 192, base=1e5),
                     memory_layer(2, 64, 128, 15.0, None),
                     latent_layer(2, 64, 64, 128, 128, 96, 128, base=1e4, scale=0.1)]},
    # every count that can be 1 is 1, and sizes that can be equal are equal (an odd vocabulary on a
    # width the tensor-core products take)
    "D": {"architecture": "Varunex", "vocab": 67, "width": 32, "norm": {"eps": 1e-5},
          "layers": [latent_layer(1, 16, 16, 16, 16, 16, 32),
                     diff_layer(1, 1, 16, 16, 16, 16, 32, diff=0.5),
                     memory_layer(1, 16, 16, 1.0, 32)]},
    # a width the tensor-core products take around inner sizes that fit no vector width: products
    # with 86, 30 or 50 features, rows of activations that start at odd addresses
    "E": {"architecture": "Varunex", "vocab": 67, "width": 64, "norm": {"eps": 1e-5},
          "layers": [diff_layer(3, 1, 10, 6, 9, 6, 50, diff=0.45),
                     latent_layer(3, 6, 4, 5, 12, 10, 36, scale=0.8),
                     memory_layer(1, 12, 7, 9.0, None),
                     latent_layer(5, 8, 8, 8, 24, 20, 30)]},
    # more heads than one block of the tensor-core kernels holds: 20 heads on one latent (two groups
    # of 16 rows, the second partly empty), 40 score maps on 5 key/value heads (dealt out to blocks)
    "F": {"architecture": "Varunex", "vocab": 120, "width": 64, "norm": {"eps": 1e-5},
          "layers": [latent_layer(20, 8, 8, 8, 24, 16, 64),
                     diff_layer(20, 5, 16, 16, 50, 8, None, diff=0.25)]},
}
INIT = {"A": dict(seed=3, sigma=0.15, norm_jitter=0.2), "B": dict(seed=5, sigma=0.2, norm_jitter=0.1),
        "C": dict(seed=9, sigma=0.08, norm_jitter=0.15), "D": dict(seed=12, sigma=0.2, norm_jitter=0.1), "E": dict(seed=15, sigma=0.2, norm_jitter=0.1),
        "F": dict(seed=17, sigma=0.15, norm_jitter=0.1)}

_tmp = tempfile.TemporaryDirectory(prefix="kipp_b200_varunex_")


def write_folder(folder: str, cfg: dict, init: dict, dtype=torch.float32, override=None) -> str:
    """A model folder with random weights; ``override(name, tensor) -> tensor or None``
    replaces tensors before they are written."""
    from kipp_b200.config import config_from_dict
    from kipp_b200.weights import write_random_model
    out = write_random_model(folder, config_from_dict(cfg), init["seed"], sigma=init["sigma"],
                             norm_jitter=init["norm_jitter"], dtype=dtype)
    if override is not None:
        from tiny import read_weights
        from kipp_b200.weights.safetensors_io import write_safetensors
        w = read_weights(out)
        for k in list(w):
            new = override(k, w[k])
            if new is not None:
                w[k] = new.to(w[k].dtype)
        write_safetensors(os.path.join(out, "model.safetensors"), list(w.items()))
    return out


@functools.lru_cache(maxsize=None)
def model_folder(name: str) -> str:
    return write_folder(os.path.join(_tmp.name, name), CONFIGS[name], INIT[name])


def random_tokens(vocab: int, n: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
