"""Host side of the Vomotar architecture: its config.json, the tensors it expects, sizes that only
a weight file gives, and what its mixers ask of the cache manager (a paged group and a state
group for one layer; pages given back behind a chunk)."""

import copy
import json
import os

import pytest
import torch

import plain_vomotar as pv
import vomotar_configs as vc
from distengine_b200.cache.manager import CacheManager
from distengine_b200.config import ConfigError, VomotarConfig
from distengine_b200.models.decoder import expected_tensors
from distengine_b200.parts import PagedKVSpec, StateSpec
from distengine_b200.registry import resolve
from distengine_b200.weights import WeightMismatchError, load_checked, save_tensors


@pytest.mark.parametrize("name", sorted(vc.ALL))
def test_config_round_trip_and_tensor_names(name):
    architecture, config = resolve(vc.ALL[name])
    assert architecture.name == "Vomotar" and isinstance(config, VomotarConfig)
    assert config.to_json() == vc.ALL[name]
    assert resolve(config.to_json())[1] == config
    expected, vectors, optional = expected_tensors(config)
    assert expected == {k: tuple(v) for k, v in pv.tensor_shapes(vc.ALL[name]).items()}
    assert not optional and "final.norm" in vectors


def test_a_rank_comes_from_the_weight_file(tmp_path):
    data = copy.deepcopy(vc.VOMO_C)
    for layer in data["layers"]:
        del layer["mixer"]["rank"]
    _, config = resolve(data)
    expected, _, _ = expected_tensors(config)
    assert expected["l0.mix.a1"] == (-1, 48) and expected["l0.mix.g2"] == (2 * 20, -1)
    weights = pv.random_weights(vc.VOMO_C, 1)
    save_tensors(str(tmp_path / "model.safetensors"), weights)
    loaded = load_checked(str(tmp_path), expected, set(), torch.float32)
    assert loaded["l0.mix.a1"].shape == (16, 48) and loaded["l1.mix.a2"].shape == (6 * 8, 3)
    weights["l0.mix.q"] = weights["l0.mix.q"][:-1]
    save_tensors(str(tmp_path / "model.safetensors"), weights)
    with pytest.raises(WeightMismatchError) as error:
        load_checked(str(tmp_path), expected, set(), torch.float32)
    assert [w[0] for w in error.value.wrong_shape] == ["l0.mix.q"]


@pytest.mark.parametrize("change,word", [
    (lambda d: d["layers"][0].__setitem__("type", "other"), "type"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda d: d["layers"][1]["mixer"]["right"].__setitem__("decay", [0.5]), "decay"),
    (lambda d: d["layers"][1]["mixer"]["right"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"]["left"].pop("scale"), "scale"),
    (lambda d: d["layers"][1]["mixer"]["left"]["mask"].__setitem__("size", 0), "size"),
    (lambda d: d["norm"].__setitem__("groups", 5), "groups"),
    (lambda d: d["layers"][0]["mlp"].__setitem__("kind", "routed"), "mlp"),
    (lambda d: d.pop("vocab"), "vocab"),
])
def test_what_the_configuration_refuses(change, word):
    data = copy.deepcopy(vc.VOMO_A)
    change(data)
    with pytest.raises(ConfigError) as error:
        resolve(data)
    assert word in str(error.value)


def test_layers_become_parts():
    _, config = resolve(vc.VOMO_A)
    specs = config.layer_specs()
    assert [s.mixer.kind for s in specs] == ["gated_delta_rule", "parallel", "gated_delta_rule"]
    assert specs[2].feed_forward is None and specs[0].feed_forward.kind == "gated_mlp"
    assert specs[0].norm.params["groups"] == 4 and specs[0].prefix("mixer") == "l0.mix."
    left, right = (spec for _, spec in specs[1].mixer.params["branches"])
    assert left.kind == "chunk_attention" and left.params["chunk"] == 24
    assert right.kind == "retention" and right.params["decay"] == (0.9, 0.99)


def _manager(specs, pages=12, page=4, slots=3):
    return CacheManager(specs, [None] * len(specs), page, pages, slots, 64, torch.float32, "cpu")


def test_a_layer_with_pages_and_a_state_gets_both():
    paged = PagedKVSpec(2, 6, None, value_dim=10, chunk=8)
    specs = [StateSpec((5,)), (paged, StateSpec((7,))), StateSpec((5,)), (paged, StateSpec((7,)))]
    cache = _manager(specs)
    bindings = cache.bindings()
    assert bindings[0].kind == "state" and bindings[0].state.shape == (3, 5)
    assert bindings[1].kind == "parts" and [b.kind for b in bindings[1].parts] == ["paged", "state"]
    left, right = bindings[3].parts
    assert left.k_pages.shape == (12, 2, 4, 6) and left.v_pages.shape == (12, 2, 4, 10)
    assert right.state.shape == (3, 7)
    # two layers of a kind share a group, each with a tensor of its own
    assert left.k_pages.data_ptr() != bindings[1].parts[0].k_pages.data_ptr()
    assert left.block_table is bindings[1].parts[0].block_table
    assert CacheManager.bytes_per_page(specs, 4, torch.float32) == 2 * 2 * 4 * (6 + 10) * 4
    cache.admit("a")
    right.state[cache.slot("a")] = 3.0
    cache.release("a")
    cache.admit("b")                                    # the slot comes back zeroed
    assert float(right.state[cache.slot("b")].abs().sum()) == 0.0


def test_pages_behind_the_chunk_are_given_back():
    cache = _manager([PagedKVSpec(1, 4, None, chunk=10)], pages=8, page=4)
    cache.admit("a")
    cache.reserve([("a", 23)])                          # a portion over two chunk edges
    assert cache.num_free_pages() == 8 - 6
    cache.commit("a", 23)                               # the next token reads from position 20 on
    assert cache.paged[0].tables["a"][:5] == [-1] * 5 and cache.num_free_pages() == 8 - 1
    cache.check_invariants()
    for length in range(24, 41):                        # token by token over the edges at 30, 40
        cache.reserve([("a", length)])
        cache.commit("a", length)
        table = cache.paged[0].tables["a"]
        first = (length // 10 * 10) // 4
        assert all(p < 0 for p in table[:first]) and all(p >= 0 for p in table[first:])
        cache.check_invariants()
    # a tentative step gives nothing back until it is confirmed
    cache.reserve([("a", 50)])
    held = cache.num_free_pages()
    cache.commit("a", 50, tentative=True)
    assert cache.num_free_pages() == held
    cache.confirm("a")
    assert cache.num_free_pages() > held
    cache.release("a")
    assert cache.num_free_pages() == 8
    cache.check_invariants()


def test_random_weights_mode_writes_a_model(tmp_path):
    from distengine_b200.weights import write_random_model
    folder = write_random_model(vc.VOMO_B, str(tmp_path / "m"), seed=3, dtype="bfloat16")
    with open(os.path.join(folder, "config.json")) as handle:
        written = json.load(handle)
    _, config = resolve(written)
    expected, _, _ = expected_tensors(config)
    assert set(load_checked(folder, expected, set(), torch.bfloat16)) == set(expected)
    data = copy.deepcopy(vc.VOMO_B)
    del data["layers"][1]["mixer"]["rank"]
    with pytest.raises(ValueError):
        write_random_model(data, str(tmp_path / "n"), seed=3)
