"""Tiny Pepolorn configurations of the tests and helpers around them.

A has sizes no kernel likes (nothing a multiple of 8, keys and values of different sizes, a rotation over part of a
head with and without rescaled rates, chunks shorter than a page and not a multiple of one, three and five taps, a
layer without feed-forward, experts in groups and without, two layers that run another layer's weights).
B has sizes the fast kernels take.  C makes things equal or 1 that the others keep apart (as many key/value heads as
heads, one head of state, one group, one tap, a chunk of one page and of one token, a rotation over the whole head
with a factor of 1, a decay of 1, scales of 1, one expert per group, all groups kept, one expert per token, the first
layer run again as the last).
"""
import copy
import json
import os

import torch

from prelude_b200.weights.random_init import random_tensors
from prelude_b200.weights.safetensors_io import write_safetensors


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def left(heads, kv, dim, vdim, scale, chunk, rot_dims=None, base=None, scaling=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rot_dims is not None:
        m["rot"] = {"dims": rot_dims, "base": base}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return m


def right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def parallel(l, r, scales, mlp):
    return {"type": "parallel", "mixer": {"left": l, "right": r, "left_scale": scales[0], "right_scale": scales[1]}, "mlp": mlp}


def mamba2(heads, groups, state, vdim, conv, norm_groups, mlp):
    return {"type": "mamba2", "mixer": {"heads": heads, "groups": groups, "state": state, "vdim": vdim, "conv": conv,
                                        "norm_groups": norm_groups}, "mlp": mlp}


def again(layer, source):
    return dict(copy.deepcopy(layer), weights_of=source)


_A0 = parallel(left(4, 2, 12, 20, 0.3, 7, 6, 50.0, (4.0, 64, 8.0, 2.0)), right(3, 10, 6, (0.5, 0.9, 0.99)), (0.7, 1.3), moe(6, 2, 10, (3, 2)))
_A3 = mamba2(3, 1, 9, 11, 5, 1, None)
PEPOLORN_A = {
    "architecture": "Pepolorn", "vocab": 101, "width": 44, "norm": {"eps": 1e-5},
    "layers": [
        _A0,
        mamba2(4, 2, 10, 6, 3, 3, dense(24)),
        again(_A0, 0),
        _A3,
        parallel(left(2, 1, 10, 6, 0.35, 13, 10, 30.0), right(2, 9, 11, (0.8, 0.97)), (1.2, 0.6), moe(5, 3, 14)),
        again(_A3, 3),
    ],
}

_B1 = parallel(left(8, 2, 64, 64, 0.25, 48, 32, 10000.0, (16.0, 128, 16.0, 1.0)), right(2, 128, 64, (0.9, 0.995)), (0.9, 1.1), moe(8, 4, 64, (4, 2)))
PEPOLORN_B = {
    "architecture": "Pepolorn", "vocab": 211, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        mamba2(4, 1, 64, 32, 4, 1, dense(192)),
        _B1,
        mamba2(8, 4, 32, 16, 4, 2, moe(16, 2, 32, (2, 1))),
        again(_B1, 1),
        parallel(left(4, 4, 32, 64, 0.3, 64, 16, 500.0), right(8, 32, 16, (0.3, 0.5, 0.7, 0.8, 0.9, 0.95, 0.98, 0.999)), (1.0, 0.5), dense(96)),
    ],
}

_C0 = parallel(left(2, 2, 16, 16, 0.4, 8, 16, 20.0, (1.0, 32, 4.0, 1.0)), right(1, 16, 16, (1.0,)), (1.0, 1.0), moe(4, 1, 8, (4, 4)))
PEPOLORN_C = {
    "architecture": "Pepolorn", "vocab": 50, "width": 32, "norm": {"eps": 1e-6},
    "layers": [
        _C0,
        mamba2(1, 1, 8, 16, 1, 1, moe(2, 1, 16, (2, 1))),
        parallel(left(4, 4, 8, 8, 0.5, 1), right(4, 8, 24, (0.6, 0.7, 0.8, 0.9)), (1.0, 1.0), dense(40)),
        mamba2(2, 2, 16, 8, 2, 2, None),
        again(_C0, 0),
    ],
}

# configuration, random-weight options, page size
PARAMS = {"A": (PEPOLORN_A, dict(seed=61, std=0.25, norm_jitter=0.3), 4),
          "B": (PEPOLORN_B, dict(seed=62, std=0.12, norm_jitter=0.2), 16),
          "C": (PEPOLORN_C, dict(seed=63, std=0.2, norm_jitter=0.2), 8)}


ROUTER_SCALE = 0.2      # router logits of order one: scores that are not all 0 or 1, so that choices differ from token to token


def tensors_of(cfg: dict, dtype=torch.float32, **init):
    """Random tensors of a configuration, the routers scaled down."""
    tensors = random_tensors(cfg, dtype=torch.float32, **init)
    return {k: (v * ROUTER_SCALE if k.endswith(".router") else v).to(dtype) for k, v in tensors.items()}


def make_folder(tmp_path, which: str, dtype=torch.float32, config=None, **overrides):
    cfg, init, _ = PARAMS[which]
    cfg = copy.deepcopy(config or cfg)
    init = dict(init, **overrides)
    name = f"pepolorn_{which}_{str(dtype).split('.')[-1]}_{abs(hash(str(cfg) + str(init))) % 10**8}"
    return make_folder_from_tensors(tmp_path, name, cfg, tensors_of(cfg, dtype, **init))


def make_folder_from_tensors(tmp_path, name: str, cfg: dict, tensors: dict) -> str:
    """A folder with the given tensors (made or changed by a test so that a fault would show)."""
    d = os.path.join(str(tmp_path), name)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors, {"format": "pt"})
    return d


__all__ = ["PEPOLORN_A", "PEPOLORN_B", "PEPOLORN_C", "PARAMS", "make_folder", "make_folder_from_tensors", "random_tensors", "tensors_of"]
