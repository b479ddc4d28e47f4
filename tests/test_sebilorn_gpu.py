"""The Sebilorn architecture through the engine against the plain implementation
(``plain_sebilorn``): whole prompts, prefill against token-by-token decoding, portions down to two
tokens, mixed batches on pools so small that pages and slots are used again (freed pages
poisoned), long decoding across many window edges, CUDA graphs, models of random sizes, and greedy
generation through ``Engine`` and the command line."""

import tempfile

import numpy as np
import pytest
import torch

import plain_sebilorn as ps
import sebilorn_configs as sc
import trace_helpers as th
from gpu_helpers import assert_close

pytestmark = pytest.mark.gpu
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
LENGTHS = [70, 33, 100, 5, 64, 17, 90, 48, 1, 2]

_cache: dict = {}


def _model(name, model_root):
    if name not in _cache:
        folder, weights = sc.make_folder(name, model_root)
        requests = {f"r{i}": sc.tokens(name, n, i) for i, n in enumerate(LENGTHS)}
        # bfloat16 is compared with the plain implementation rounding where the engine rounds
        reference = {dtype: {rid: ps.forward(sc.ALL[name], weights, t, act=act)
                             .to(torch.float32).numpy() for rid, t in requests.items()}
                     for dtype, act in (("float32", None), ("bfloat16", torch.bfloat16))}
        _cache[name] = (folder, weights, requests, reference)
    return _cache[name]


def _schedules(requests):
    return {
        "whole": (th.schedule_whole(requests), 128),
        "tail": (th.schedule_tail(requests, 32), 128),
        "portions": (th.schedule_portions(requests), 128),
        "pairs": (th.schedule_portions(requests, sizes=(2,)), 128),
        "mixed": (th.schedule_mixed(requests, 320, seed=3), 320),
        "mixed_tight": (th.schedule_mixed(requests, 192, seed=11, decode_tail=32), 192),
    }


# bfloat16 bounds of this file, as shares of a position's largest logit; the 32-bit runs are the
# sharp test (gpu_helpers.F32_REL).  The engine and the plain implementation's rounding model sum
# in different orders, and a head's read-out divided by its own root mean square passes small
# differences on at full size where the read-out is small.
BF16_MAX, BF16_RMS = 8e-2, 2e-2


def _compare(rows, reference, dtype, what):
    assert rows, "the replay wrote nothing"
    for (rid, position), got in rows.items():
        want = reference[rid][position]
        if dtype == torch.float32:
            assert_close(got, want, dtype, f"{what} {rid}@{position}")
            continue
        assert np.isfinite(got).all(), f"{what} {rid}@{position}: not finite"
        err, scale = np.abs(got - want), np.abs(want).max()
        assert err.max() <= BF16_MAX * scale and np.sqrt((err ** 2).mean()) <= BF16_RMS * scale, (
            f"{what} {rid}@{position}: max {err.max():.3e}, rms {np.sqrt((err ** 2).mean()):.3e}, "
            f"largest logit {scale:.3e}")


@pytest.mark.parametrize("name", ["sebi_a", "sebi_b", "sebi_c"])
@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", ["whole", "tail", "portions", "pairs", "mixed", "mixed_tight"])
def test_replay_matches_plain(name, dtype_name, schedule, model_root):
    from distengine_b200.engine.replay import build_runner
    folder, _, requests, reference = _model(name, model_root)
    steps, max_tokens = _schedules(requests)[schedule]
    runner = build_runner(folder, dtype_name, max_tokens, page_size=sc.PAGES[name],
                          poison_freed_pages=True, live_requests=4)
    with tempfile.TemporaryDirectory() as out:
        th.replay_in_process(runner, steps, out)
        rows = th.collect(steps, out, sc.ALL[name]["vocab"])
    runner.cache.check_invariants()
    assert not runner.cache.live
    wanted = sum(len(e["want"]) for s in steps for e in s["entries"])
    assert len(rows) == wanted
    _compare(rows, reference[dtype_name], DTYPES[dtype_name], f"{name} {schedule}")


@pytest.mark.parametrize("name", ["sebi_a", "sebi_c"])
def test_float32_cuts_agree_closely(name, model_root):
    """However a request is cut, its 32-bit logits agree far inside the tolerance."""
    from distengine_b200.engine.replay import build_runner
    folder, _, requests, _ = _model(name, model_root)
    got = {}
    for schedule in ("whole", "tail", "pairs", "mixed"):
        steps, max_tokens = _schedules(requests)[schedule]
        runner = build_runner(folder, "float32", max_tokens, page_size=sc.PAGES[name])
        with tempfile.TemporaryDirectory() as out:
            th.replay_in_process(runner, steps, out)
            got[schedule] = th.collect(steps, out, sc.ALL[name]["vocab"])
    for schedule in ("tail", "pairs", "mixed"):
        for key, row in got[schedule].items():
            np.testing.assert_allclose(row, got["whole"][key], rtol=0, atol=2e-5,
                                       err_msg=f"{schedule} {key}")


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["sebi_a", "sebi_c"])
def test_long_decoding_with_graphs(name, dtype_name, model_root):
    """A short prompt, then 220 tokens one by one, also replayed as CUDA graphs: every window
    passes over decoded tokens many times and pages behind the windows are given back, while the
    pages of the kept first tokens stay."""
    from distengine_b200.engine.replay import build_runner
    folder, weights = sc.make_folder(name, model_root)
    ids = sc.tokens(name, 230, 77)
    act = None if dtype_name == "float32" else torch.bfloat16
    want = ps.forward(sc.ALL[name], weights, ids, act=act).to(torch.float32).numpy()
    steps = th.schedule_tail({"long": ids}, 220)
    for graphs in (False, True):
        runner = build_runner(folder, dtype_name, 256, page_size=16, use_graphs=graphs,
                              poison_freed_pages=True)
        with tempfile.TemporaryDirectory() as out:
            th.replay_in_process(runner, steps, out)
            rows = th.collect(steps, out, sc.ALL[name]["vocab"])
        assert (not graphs) or runner.graph_replays > 100
        _compare(rows, {"long": want}, DTYPES[dtype_name], f"long decode graphs={graphs}")


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_a_long_prompt_at_wide_sizes(dtype_name, model_root):
    """1,100 tokens in one step (products of a thousand rows and more, attention tiles of 64 rows,
    windows of 300 and 1,000 keys passing), then tokens one by one, then the same prompt in two
    uneven portions."""
    from distengine_b200.engine.replay import build_runner
    from distengine_b200.kernels import recurrent as rk
    name = "sebi_wide"
    folder, weights = sc.make_folder(name, model_root)
    ids = sc.tokens(name, 1112, 3)
    assert rk.long_portion_rows(np.array([1100], dtype=np.int32), 24, 4) >= 48
    act = None if dtype_name == "float32" else torch.bfloat16
    want = ps.forward(sc.ALL[name], weights, ids, act=act).to(torch.float32).numpy()
    picked = [0, 1, 4, 5, 299, 300, 301, 304, 305, 306, 599, 999, 1000, 1001, 1099]
    head = {"step": 0, "end": [], "entries": [{"id": "w", "tokens": ids[:1100], "want": picked}]}
    tail = [{"step": 1 + i, "end": ["w"] if i == 11 else [],
             "entries": [{"id": "w", "tokens": [ids[1100 + i]], "want": [0]}]} for i in range(12)]
    cut = [{"step": 13, "end": [], "entries": [{"id": "c", "tokens": ids[:1027], "want": [1026]}]},
           {"step": 14, "end": ["c"], "entries": [{"id": "c", "tokens": ids[1027:],
                                                    "want": [0, 84]}]}]
    steps = [head] + tail + cut
    runner = build_runner(folder, dtype_name, 1152, page_size=16, poison_freed_pages=True)
    with tempfile.TemporaryDirectory() as out:
        th.replay_in_process(runner, steps, out)
        rows = th.collect(steps, out, sc.ALL[name]["vocab"])
    assert len(rows) == len(picked) + 12 + 3
    _compare(rows, {"w": want, "c": want}, DTYPES[dtype_name], f"wide {dtype_name}")


def test_pages_behind_a_window_come_back_but_the_first_stay(model_root):
    """After 200 tokens the windowed groups hold the pages of their kept first tokens and of the
    window only; the group that sees everything holds all."""
    from distengine_b200.engine.replay import build_runner
    from distengine_b200.engine.step import StepEntry
    folder, _ = sc.make_folder("sebi_c", model_root)
    runner = build_runner(folder, "float32", 256, page_size=16)
    ids = sc.tokens("sebi_c", 200, 5)
    runner.step([StepEntry("a", ids[:150], [])])
    for t in ids[150:]:
        runner.step([StepEntry("a", [t], [0])])
    runner.check_status()
    held = {}
    for group in runner.cache.paged:
        table = group.tables["a"]
        held[(group.spec.window, group.spec.keep_first)] = [p for p, x in enumerate(table) if x >= 0]
    assert held[(None, 0)] == list(range(13))
    # window 33 and 40 kept tokens: pages 0..2 stay, then from position 200 - 33 + 1 on
    assert held[(33, 40)] == [0, 1, 2] + list(range((200 - 33 + 1) // 16, 13))
    assert held[(50, 17)] == [0, 1] + list(range((200 - 50 + 1) // 16, 13))
    runner.release("a")
    runner.cache.check_invariants()


def test_batch_of_unequal_requests_against_each_alone(model_root):
    """Four unequal requests in one step give what each gives alone (32-bit: to rounding)."""
    from distengine_b200.engine.replay import build_runner
    from distengine_b200.engine.step import StepEntry
    name = "sebi_b"
    folder, _, requests, reference = _model(name, model_root)
    picked = ["r0", "r3", "r8", "r5"]
    runner = build_runner(folder, "float32", 512, page_size=8)
    entries = [StepEntry(r, requests[r], list(range(len(requests[r])))) for r in picked]
    logits = runner.step(entries).cpu().numpy()
    runner.check_status()
    at = 0
    for r in picked:
        n = len(requests[r])
        assert_close(logits[at: at + n], reference["float32"][r], torch.float32, f"batched {r}")
        at += n


def _random_config(rng) -> dict:
    """A model of random sizes: every kind of layer at least once, in random order."""
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    width = int(pick(24, 40, 56, 72))
    layers, owners = [], []
    kinds = ["attention", "parallel", "lightning", "attention", pick("attention", "lightning"),
             pick("attention", "parallel")]
    rng.shuffle(kinds)
    for i, kind in enumerate(kinds):
        ff = None if rng.random() < 0.3 else int(pick(16, 48, 72))
        if kind == "attention":
            if owners and rng.random() < 0.5:
                j = int(pick(*owners))
                src = layers[j]["mixer"]
                heads = src["kv_heads"] * int(pick(1, 2))
                layers.append(sc._attention(heads, src["kv_heads"], src["dim"], src["vdim"],
                                            float(pick(0.2, 0.3)), int(pick(1, 5, 16, 40, 300)),
                                            int(pick(0, 1, 4, 20)), src["rot"],
                                            pick(None, 6.0, 25.0), j, ff))
                continue
            kv = int(pick(1, 2, 3))
            heads = kv * int(pick(1, 2, 4))
            dim, vdim = int(pick(4, 8, 10, 16, 24)), int(pick(2, 6, 8, 16, 32))
            dims = int(pick(0, 2, dim // 2 * 2, dim // 4 * 2))
            scaling = pick(None, (2.0, 1.0, 4.0, 16), (8.0, 0.5, 2.0, 100))
            layers.append(sc._attention(heads, kv, dim, vdim, float(pick(0.2, 0.35)),
                                        int(pick(1, 3, 16, 17, 64, 300)), int(pick(0, 1, 7, 33)),
                                        sc._rot(dims, float(pick(50.0, 10000.0)), scaling),
                                        pick(None, 4.0, 30.0), None, ff))
            if rng.random() < 0.2:
                del layers[-1]["mixer"]["mask"]          # every earlier token is seen
            owners.append(i)
        elif kind == "parallel":
            kv = int(pick(1, 2))
            dim = int(pick(6, 8, 16))
            layers.append(sc._parallel(
                (kv * int(pick(1, 3)), kv, dim, int(pick(4, 8, 10)), float(pick(0.25, 0.4)),
                 sc._rot(int(pick(0, 2, dim)), float(pick(100.0, 500000.0)))),
                (int(pick(1, 2, 3)), int(pick(4, 9, 16, 32)), int(pick(1, 4, 8))),
                (float(pick(1.0, 0.6)), float(pick(1.0, 0.5))), ff))
        else:
            heads = int(pick(1, 2, 5))
            layers.append(sc._lightning(heads, int(pick(3, 8, 16)), int(pick(5, 8, 16)),
                                        [float(pick(1.0, 0.99, 0.7, 0.3)) for _ in range(heads)],
                                        ff))
    config = {"architecture": "Sebilorn", "vocab": int(pick(50, 111)), "width": width,
              "norm": {"eps": float(pick(1e-5, 1e-6))},
              "embedding": {"scale": float(pick(1.0, 4.0, 6.5))}, "layers": layers}
    if rng.random() < 0.7:
        config["logit_softcap"] = float(pick(5.0, 30.0))
    return config


@pytest.mark.parametrize("seed", range(6))
def test_models_of_random_sizes_under_a_mixed_schedule(seed, model_root):
    from distengine_b200.engine.replay import build_runner
    import os
    rng = np.random.default_rng(1000 + seed)
    config = _random_config(rng)
    weights = ps.random_weights(config, 50 + seed)
    folder = sc.write_folder(config, os.path.join(model_root, f"sebi_random_{seed}"), weights)
    requests = {f"q{i}": [int(t) for t in rng.integers(0, config["vocab"], size=n)]
                for i, n in enumerate((61, 9, 80, 2, 35, 50))}
    want = {rid: ps.forward(config, weights, t).to(torch.float32).numpy()
            for rid, t in requests.items()}
    steps = th.schedule_mixed(requests, 256, seed=seed, decode_tail=20)
    for graphs in (False, True):
        runner = build_runner(folder, "float32", 256, page_size=int(rng.choice([4, 8, 16])),
                              poison_freed_pages=True, use_graphs=graphs)
        with tempfile.TemporaryDirectory() as out:
            th.replay_in_process(runner, steps, out)
            rows = th.collect(steps, out, config["vocab"])
        runner.cache.check_invariants()
        _compare(rows, want, torch.float32, f"random model {seed} graphs={graphs}")


def test_greedy_generation_through_the_engine(model_root):
    """``Engine.generate`` (scheduler, portions of prompts under a small token budget, sampling,
    step-ahead decoding) gives the plain implementation's greedy tokens in 32-bit."""
    from distengine_b200 import Engine, EngineConfig
    name = "sebi_a"
    folder, weights = sc.make_folder(name, model_root)
    prompts = [sc.tokens(name, n, 40 + i) for i, n in enumerate((3, 29, 50, 11, 1))]
    new = 12

    def plain_greedy(prompt):
        ids = list(prompt)
        for _ in range(new):
            ids.append(int(ps.forward(sc.ALL[name], weights, ids)[-1].argmax()))
        return ids[len(prompt):]

    want = [plain_greedy(p) for p in prompts]
    engine = Engine(folder, EngineConfig(dtype="float32", block_size=16, num_blocks=24,
                                         decode_batch_size=3, max_batch_tokens=32,
                                         max_model_len=128))
    assert engine.generate(prompts, new) == want
    engine.cache.check_invariants()
    # bfloat16: the first generated token is the plain implementation's unless two are nearly tied
    engine = Engine(folder, EngineConfig(dtype="bfloat16", block_size=16, num_blocks=24,
                                         decode_batch_size=3, max_batch_tokens=32,
                                         max_model_len=128))
    got = engine.generate(prompts, new)
    for prompt, tokens in zip(prompts, got):
        logits = ps.forward(sc.ALL[name], weights, prompt)[-1]
        gap = (logits.max() - logits[tokens[0]]).item()
        assert gap <= 4e-2 * logits.abs().max().item()


def test_preempted_requests_are_recomputed(model_root):
    """So few pages that running requests are preempted: they give back pages and slot, and their
    states are built again from their tokens; the greedy tokens stay the plain implementation's."""
    from distengine_b200 import Engine, EngineConfig
    name = "sebi_a"
    folder, weights = sc.make_folder(name, model_root)
    prompts = [sc.tokens(name, n, 60 + i) for i, n in enumerate((30, 27, 33))]
    new = 24

    def plain_greedy(prompt):
        ids = list(prompt)
        for _ in range(new):
            ids.append(int(ps.forward(sc.ALL[name], weights, ids)[-1].argmax()))
        return ids[len(prompt):]

    engine = Engine(folder, EngineConfig(dtype="float32", block_size=16, num_blocks=5,
                                         decode_batch_size=3, max_batch_tokens=48,
                                         max_model_len=64))
    assert engine.generate(prompts, new) == [plain_greedy(p) for p in prompts]
    assert engine.scheduler.num_preemptions > 0
    engine.cache.check_invariants()
    assert not engine.cache.live


def test_the_command_line_generates(model_root):
    import os
    import subprocess
    import sys
    folder, _ = sc.make_folder("sebi_b", model_root)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    result = subprocess.run([sys.executable, "-m", "distengine_b200", "generate", "--model", folder,
                             "--prompt-ids", "5 17 3", "--max-new-tokens", "4", "--dtype",
                             "float32", "--num-blocks", "16", "--decode-batch-size", "2"],
                            cwd=root, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr[-2000:]
    assert "Generated token IDs" in result.stdout
