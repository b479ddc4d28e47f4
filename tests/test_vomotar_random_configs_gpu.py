"""Vomotar models of random sizes through the engine against the plain implementation: layer
orders, groups, heads a key/value head (also more than the single-token attention kernel takes),
key and value sizes that are and are not whole 16-byte pieces, 1 to 5 taps, ranks down to 1,
chunks of 1 to 1,000 positions, rotation of none, some or all of a head, layers without a
feed-forward; mixed batches on a small pool (freed pages poisoned), with and without CUDA graphs.

The 32-bit bound of a position is the usual one or, where the design itself is touchy there (a
read-out divided by its own root mean square where that is tiny), four times what the plain
implementation loses between 64-bit and 32-bit at that position."""

import json
import os
import tempfile

import numpy as np
import pytest
import torch

import plain_vomotar as pv
import trace_helpers as th
from gpu_helpers import F32_REL

pytestmark = pytest.mark.gpu


def random_config(rng) -> dict:
    groups = int(rng.choice([1, 2, 3, 4, 6]))
    width = groups * int(rng.choice([8, 12, 20, 32, 44, 64]))
    layers = []
    for _ in range(int(rng.integers(1, 4))):
        ff = None if rng.random() < 0.2 else int(rng.choice([24, 40, 100, 136]))
        mlp = None if ff is None else {"kind": "dense", "ff": ff}
        kv = int(rng.choice([1, 2, 3]))
        if rng.random() < 0.5:
            rep = int(rng.choice([1, 2, 4]))
            mixer = {"heads": kv * rep, "kv_heads": kv,
                     "dim": int(rng.choice([4, 8, 12, 24, 32, 40, 64, 100, 128])),
                     "vdim": int(rng.choice([4, 8, 20, 32, 48, 64, 72])),
                     "conv": int(rng.integers(1, 6)), "rank": int(rng.choice([1, 3, 8, 16, 24, 40]))}
            layers.append({"type": "channel_delta", "mixer": mixer, "mlp": mlp})
        else:
            rep = int(rng.choice([1, 2, 4, 8, 12]))
            rdk, rh = int(rng.choice([4, 8, 16, 24, 64, 128])), int(rng.choice([1, 2, 5]))
            left = {"heads": kv * rep, "kv_heads": kv,
                    "dim": int(rng.choice([4, 8, 12, 24, 32, 64, 96, 128])),
                    "vdim": int(rng.choice([4, 8, 16, 40, 64, 96, 128])),
                    "scale": float(rng.uniform(0.05, 0.5)),
                    "mask": {"size": int(rng.choice([1, 3, 16, 17, 50, 64, 1000]))}}
            right = {"heads": rh, "dim": rdk, "vdim": int(rng.choice([4, 8, 24, 32, 64])),
                     "decay": [float(x) for x in rng.uniform(0.8, 1.0, size=rh)],
                     "rot": {"dims": int(rng.choice([0, 2, rdk // 2, rdk])) // 2 * 2,
                             "base": float(rng.choice([100.0, 1e4, 1e6]))}}
            layers.append({"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp})
    return {"architecture": "Vomotar", "vocab": int(rng.choice([50, 97, 130])), "width": width,
            "norm": {"eps": float(rng.choice([1e-6, 1e-5])), "groups": groups}, "layers": layers}


@pytest.mark.parametrize("seed", range(8))
def test_random_configuration(seed):
    from distengine_b200.engine.replay import build_runner
    from distengine_b200.weights import save_tensors
    rng = np.random.default_rng(1000 + seed)
    config = random_config(rng)
    weights = pv.random_weights(config, seed)
    requests = {f"r{i}": [int(t) for t in rng.integers(0, config["vocab"], size=n)]
                for i, n in enumerate([70, 33, 100, 5, 1, 48])}
    page = int(rng.choice([8, 16, 32]))
    exact = {r: pv.forward(config, weights, t).numpy() for r, t in requests.items()}
    single = {r: pv.forward(config, weights, t, dtype=torch.float32).double().numpy()
              for r, t in requests.items()}
    rounded = {r: pv.forward(config, weights, t, act=torch.bfloat16).numpy()
               for r, t in requests.items()}
    steps = th.schedule_mixed(requests, 320, seed=seed)
    with tempfile.TemporaryDirectory() as root:
        with open(os.path.join(root, "config.json"), "w") as handle:
            json.dump(config, handle)
        save_tensors(os.path.join(root, "model.safetensors"),
                     {k: v.to(torch.bfloat16) for k, v in weights.items()})
        for dtype in ("float32", "bfloat16"):
            runner = build_runner(root, dtype, 320, page_size=page, poison_freed_pages=True,
                                  live_requests=4, use_graphs=seed % 2 == 0)
            with tempfile.TemporaryDirectory() as out:
                th.replay_in_process(runner, steps, out)
                rows = th.collect(steps, out, config["vocab"])
            runner.cache.check_invariants()
            assert rows and not runner.cache.live
            for (r, p), got in rows.items():
                assert np.isfinite(got).all(), f"{config}: {dtype} {r}@{p} is not finite"
                if dtype == "float32":
                    want = exact[r][p]
                    bound = max(F32_REL * max(1.0, np.abs(want).max()),
                                4 * np.abs(single[r][p] - want).max())
                else:
                    want = rounded[r][p]
                    bound = 8e-2 * np.abs(want).max()
                assert np.abs(got - want).max() <= bound, (
                    f"{config}: {dtype} {r}@{p}: max error {np.abs(got - want).max():.3e} > "
                    f"{bound:.3e}")
