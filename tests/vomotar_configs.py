"""Small Vomotar configurations for the tests, unlike each other in every size: layer order, heads
against key/value heads, key against value sizes, taps, ranks, chunk lengths (one shorter than a
page, one that no page size divides), rotary share of a head, norm groups, a layer without a
feed-forward, a single head.  Weights come from ``plain_vomotar.random_weights``."""

from __future__ import annotations

import os

import torch

import plain_vomotar as pv


def _delta(heads, kv_heads, dim, vdim, conv, rank, ff):
    return {"type": "channel_delta",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                      "conv": conv, "rank": rank},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _parallel(left, right, ff):
    heads, kv_heads, dim, vdim, scale, size = left
    rheads, rdim, rvdim, decay, dims, base = right
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                               "scale": scale, "mask": {"size": size}},
                      "right": {"heads": rheads, "dim": rdim, "vdim": rvdim, "decay": decay,
                                "rot": {"dims": dims, "base": base}}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


VOMO_A = {
    "architecture": "Vomotar", "vocab": 101, "width": 64, "norm": {"eps": 1e-5, "groups": 4},
    "layers": [
        _delta(4, 2, 16, 24, 3, 8, 96),
        _parallel((4, 2, 32, 16, 0.2, 24), (2, 16, 32, [0.9, 0.99], 8, 100.0), 96),
        _delta(4, 2, 16, 24, 3, 8, None),
    ],
}

VOMO_B = {
    "architecture": "Vomotar", "vocab": 77, "width": 96, "norm": {"eps": 1e-6, "groups": 1},
    "layers": [
        _parallel((3, 3, 20, 40, 0.31, 7), (3, 40, 8, [1.0, 0.5, 0.97], 40, 10000.0), 40),
        _delta(1, 1, 40, 72, 2, 5, 40),
        _parallel((6, 1, 12, 12, 0.5, 50), (1, 36, 36, [0.995], 18, 500.0), None),
    ],
}

VOMO_C = {
    "architecture": "Vomotar", "vocab": 130, "width": 48, "norm": {"eps": 1e-6, "groups": 3},
    "layers": [
        _delta(2, 2, 68, 20, 5, 16, 64),
        _delta(6, 3, 8, 8, 1, 3, 24),
    ],
}

# heads of 64 and 128 features, rows that are whole 16-byte pieces: the sizes at which prompts of a
# thousand tokens and more take the tensor-core products, the wide attention tiles and 16-byte copies
VOMO_WIDE = {
    "architecture": "Vomotar", "vocab": 300, "width": 256, "norm": {"eps": 2e-6, "groups": 8},
    "layers": [
        _parallel((4, 2, 128, 64, 0.1, 300), (2, 64, 128, [0.999, 0.95], 32, 10000.0), 512),
        _delta(4, 4, 64, 64, 4, 32, 512),
    ],
}

ALL = {"vomo_a": VOMO_A, "vomo_b": VOMO_B, "vomo_c": VOMO_C, "vomo_wide": VOMO_WIDE}
SEEDS = {"vomo_a": 5, "vomo_b": 6, "vomo_c": 7, "vomo_wide": 8}
PAGES = {"vomo_a": 16, "vomo_b": 8, "vomo_c": 32, "vomo_wide": 16}


def make_folder(name: str, root: str, weights: "dict | None" = None) -> "tuple[str, dict]":
    """Write the model folder (bfloat16 tensors); returns (folder, float32 weights)."""
    import json
    from distengine_b200.weights import save_tensors
    config = ALL[name]
    if weights is None:
        weights = pv.random_weights(config, SEEDS[name])
    folder = os.path.join(root, name)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(config, handle)
    save_tensors(os.path.join(folder, "model.safetensors"),
                 {k: v.to(torch.bfloat16) for k, v in weights.items()})
    return folder, weights


def tokens(name: str, length: int, index: int = 0) -> list[int]:
    import numpy as np
    rng = np.random.default_rng(100 * SEEDS[name] + 7 * index + length)
    return [int(t) for t in rng.integers(0, ALL[name]["vocab"], size=length)]
