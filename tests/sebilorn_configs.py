"""Small Sebilorn configurations for the tests, unlike each other in every size: layer order, heads
against key/value heads, key against value sizes, windows (one of a single key, one wider than any
test sequence, one shorter than a page), kept first tokens (none, fewer and more than the window,
more than a page), layers that read another layer's keys and values with a mask of their own,
rotary share of a head, frequency rescaling, soft caps present and absent, ranks, decays up to 1,
layers without a feed-forward.  Weights come from ``plain_sebilorn.random_weights``."""

from __future__ import annotations

import os

import torch

import plain_sebilorn as ps


def _rot(dims, base, scaling=None):
    out = {"dims": dims, "base": base}
    if scaling is not None:
        out["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return out


def _attention(heads, kv_heads, dim, vdim, scale, size, keep, rot, softcap=None, kv_from=None,
               ff=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
             "mask": {"size": size, "keep_first": keep}, "rot": rot}
    if softcap is not None:
        mixer["softcap"] = softcap
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer,
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _parallel(left, right, scales, ff=None):
    heads, kv_heads, dim, vdim, scale, rot = left
    rheads, rdim, rank = right
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                               "scale": scale, "rot": rot},
                      "right": {"heads": rheads, "dim": rdim, "rank": rank},
                      "left_scale": scales[0], "right_scale": scales[1]},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _lightning(heads, dim, vdim, decay, ff=None):
    return {"type": "lightning",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


SEBI_A = {
    "architecture": "Sebilorn", "vocab": 97, "width": 64, "norm": {"eps": 1e-5},
    "embedding": {"scale": 3.0}, "logit_softcap": 9.0,
    "layers": [
        _attention(4, 2, 16, 24, 0.3, 20, 3, _rot(8, 3000.0, (3.0, 1.0, 3.0, 40)), 12.0, ff=96),
        _attention(4, 2, 16, 24, 0.2, 9, 5, _rot(8, 3000.0, (3.0, 1.0, 3.0, 40)), 30.0, 0),
        _parallel((4, 1, 24, 16, 0.25, _rot(12, 500.0)), (2, 20, 6), (0.7, 0.4), 80),
        _lightning(3, 12, 20, [0.9, 1.0, 0.5]),
    ],
}

SEBI_B = {
    "architecture": "Sebilorn", "vocab": 75, "width": 42, "norm": {"eps": 1e-6},
    "embedding": {"scale": 1.0},
    "layers": [
        _lightning(1, 22, 6, [0.97], 30),
        _parallel((3, 3, 10, 6, 0.4, _rot(10, 77.0)), (1, 34, 3), (1.0, 1.5)),
        _attention(3, 3, 10, 6, 0.35, 1, 0, _rot(4, 10000.0), None, ff=50),
        _attention(2, 1, 6, 14, 0.5, 500, 2, _rot(0, 10.0), 5.0, ff=None),
        _attention(6, 3, 10, 6, 0.3, 7, 0, _rot(4, 10000.0), 8.0, 2, 20),
    ],
}

# sizes whose rows are whole 16-byte pieces (the kernels that load them so, and the one for steps
# of single tokens), eight query heads a key/value head, more kept tokens than a page and than the
# window, two layers with keys and values that each have a reader
SEBI_C = {
    "architecture": "Sebilorn", "vocab": 130, "width": 128, "norm": {"eps": 1e-6},
    "embedding": {"scale": 8.0}, "logit_softcap": 20.0,
    "layers": [
        _attention(8, 1, 32, 64, 0.18, 16, 40, _rot(32, 250000.0, (4.0, 1.0, 4.0, 64)), 15.0,
                   ff=128),
        _parallel((4, 2, 64, 32, 0.125, _rot(32, 10000.0)), (2, 32, 8), (0.6, 0.5), 128),
        _attention(8, 1, 32, 64, 0.2, 33, 1, _rot(32, 250000.0, (4.0, 1.0, 4.0, 64)), 15.0, 0,
                   64),
        _attention(4, 4, 16, 16, 0.25, 24, 17, _rot(16, 1000.0), None, ff=64),
        _lightning(4, 32, 32, [0.6, 0.88, 0.97, 0.999]),
        _attention(8, 4, 16, 16, 0.25, 50, 0, _rot(16, 1000.0), 10.0, 3),
    ],
}

# many heads of whole 16-byte rows: a prompt of a thousand tokens has so many rows that the
# attention takes tiles of 64 rows and the products a thousand rows and more
SEBI_WIDE = {
    "architecture": "Sebilorn", "vocab": 300, "width": 256, "norm": {"eps": 1e-6},
    "embedding": {"scale": 4.0}, "logit_softcap": 30.0,
    "layers": [
        _attention(24, 4, 32, 32, 0.18, 300, 5, _rot(32, 250000.0, (4.0, 1.0, 4.0, 256)), 20.0,
                   ff=512),
        _parallel((24, 4, 32, 16, 0.18, _rot(16, 10000.0)), (4, 64, 16), (0.6, 0.5), 512),
        _attention(24, 4, 32, 32, 0.18, 1000, 0, _rot(32, 250000.0, (4.0, 1.0, 4.0, 256)), None,
                   0),
        _lightning(4, 32, 64, [0.9, 0.99, 0.999, 0.97]),
    ],
}

ALL = {"sebi_a": SEBI_A, "sebi_b": SEBI_B, "sebi_c": SEBI_C, "sebi_wide": SEBI_WIDE}
SEEDS = {"sebi_a": 15, "sebi_b": 16, "sebi_c": 17, "sebi_wide": 18}
PAGES = {"sebi_a": 16, "sebi_b": 8, "sebi_c": 16, "sebi_wide": 16}


def write_folder(config: dict, folder: str, weights: dict) -> str:
    import json
    from distengine_b200.weights import save_tensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(config, handle)
    save_tensors(os.path.join(folder, "model.safetensors"),
                 {k: v.to(torch.bfloat16) for k, v in weights.items()})
    return folder


def make_folder(name: str, root: str, weights: "dict | None" = None) -> "tuple[str, dict]":
    """Write the model folder (bfloat16 tensors); returns (folder, weights)."""
    config = ALL[name]
    if weights is None:
        weights = ps.random_weights(config, SEEDS[name])
    return write_folder(config, os.path.join(root, name), weights), weights


def tokens(name: str, length: int, index: int = 0) -> list[int]:
    import numpy as np
    rng = np.random.default_rng(100 * SEEDS[name] + 7 * index + length)
    return [int(t) for t in rng.integers(0, ALL[name]["vocab"], size=length)]
