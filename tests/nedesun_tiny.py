"""Tiny Nedesun configurations of the tests and helpers around them.

N has sizes no kernel likes (nothing a multiple of 8, keys and values of different sizes, a rotation over part of a
head, windows and chunks shorter than a page and not a multiple of one, kept first tokens that end inside a page,
three and five taps, layers without feed-forward, an attention layer that blends no values between blending ones).
P has sizes the fast kernels take.  Q makes things equal or 1 that the others keep apart (one key/value head, one
head of state, as many key/value heads as heads, one tap, a window of one page, a chunk of one page, no kept tokens,
a residual multiplier and an embedding scale of 1, a blend whose source is the model's last attention layer but one).
"""
import copy
import json
import os

import torch

from prelude_b200.weights.random_init import random_tensors, write_random_model
from prelude_b200.weights.safetensors_io import write_safetensors


def _ff(ff):
    return None if ff is None else {"kind": "dense", "ff": ff}


def attention(heads, kv, dim, vdim, scale, chunk, rot_dims, base, softcap, v_mix, ff):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": chunk},
         "rot": {"dims": rot_dims, "base": base}, "softcap": softcap, "v_mix": v_mix}
    return {"type": "attention", "mixer": m, "mlp": _ff(ff)}


def wkv(heads, dim, ff=None):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}, "mlp": _ff(ff)}


def left(heads, kv, dim, vdim, scale, window, keep_first):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window, "keep_first": keep_first}}


def right(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def parallel(l, r, ff):
    return {"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": _ff(ff)}


NEDESUN_N = {
    "architecture": "Nedesun", "vocab": 101, "width": 44, "norm": {"eps": 1e-5}, "residual_mult": 0.45, "embedding": {"scale": 1.7},
    "layers": [
        parallel(left(4, 2, 12, 20, 0.3, 7, 3), right(4, 2, 10, 6, 3), 24),
        attention(3, 1, 10, 14, 0.32, 9, 6, 50.0, 5.0, True, 56),
        wkv(3, 12),
        attention(2, 2, 12, 6, 0.3, 13, 12, 30.0, 2.5, False, None),
        attention(2, 1, 8, 14, 0.35, 5, 4, 90.0, 3.0, True, 18),
        parallel(left(2, 1, 10, 6, 0.35, 19, 6), right(3, 3, 9, 11, 5), None),
        wkv(2, 22, 30),
    ],
}

NEDESUN_P = {
    "architecture": "Nedesun", "vocab": 211, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.6, "embedding": {"scale": 0.8},
    "layers": [
        attention(8, 2, 64, 64, 0.125, 48, 64, 10000.0, 30.0, True, 256),
        wkv(4, 32),
        parallel(left(8, 2, 64, 64, 0.125, 50, 5), right(4, 2, 64, 32, 4), 192),
        wkv(2, 64, 96),
        attention(4, 2, 32, 64, 0.18, 64, 16, 500.0, 15.0, True, None),
        parallel(left(4, 4, 32, 32, 0.17, 33, 16), right(8, 4, 32, 16, 4), 96),
    ],
}

NEDESUN_Q = {
    "architecture": "Nedesun", "vocab": 50, "width": 32, "norm": {"eps": 1e-6}, "residual_mult": 1.0, "embedding": {"scale": 1.0},
    "layers": [
        wkv(1, 32, 32),
        parallel(left(2, 1, 16, 16, 0.25, 8, 0), right(1, 1, 16, 16, 1), 32),
        attention(1, 1, 16, 16, 0.25, 8, 16, 20.0, 8.0, True, 32),
        parallel(left(4, 4, 8, 8, 0.3, 1, 1), right(4, 4, 8, 24, 2), 40),
        attention(2, 1, 8, 16, 0.3, 1, 2, 20.0, 50.0, True, 24),
    ],
}

# configuration, random-weight options, page size
PARAMS = {"N": (NEDESUN_N, dict(seed=41, std=0.25, norm_jitter=0.3), 4),
          "P": (NEDESUN_P, dict(seed=42, std=0.12, norm_jitter=0.2), 16),
          "Q": (NEDESUN_Q, dict(seed=43, std=0.2, norm_jitter=0.2), 8)}


def make_folder(tmp_path, which: str, dtype=torch.float32, config=None, **overrides):
    cfg, init, _ = PARAMS[which]
    cfg = copy.deepcopy(config or cfg)
    init = dict(init, **overrides)
    d = os.path.join(str(tmp_path), f"nedesun_{which}_{str(dtype).split('.')[-1]}_{abs(hash(str(cfg) + str(init))) % 10**8}")
    return write_random_model(d, cfg, dtype=dtype, **init)


def make_folder_from_tensors(tmp_path, name: str, cfg: dict, tensors: dict) -> str:
    """A folder with the given tensors (made or changed by a test so that a fault would show)."""
    d = os.path.join(str(tmp_path), name)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors, {"format": "pt"})
    return d


__all__ = ["NEDESUN_N", "NEDESUN_P", "NEDESUN_Q", "PARAMS", "make_folder", "make_folder_from_tensors", "random_tensors"]
