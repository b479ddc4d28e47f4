"""The Sebilorn configuration on the CPU: round trip, what it refuses, tensor names and shapes,
the plan of layers that read another layer's keys and values, the cache specs of such a group, and
the cache manager keeping the pages of a window's kept first tokens."""

import copy

import pytest
import torch

import plain_sebilorn as ps
import sebilorn_configs as sc
from distengine_b200.cache.manager import CacheManager
from distengine_b200.config.model import ConfigError
from distengine_b200.models.decoder import expected_tensors
from distengine_b200.parts.base import PagedKVSpec, StateSpec
from distengine_b200.registry import resolve


@pytest.mark.parametrize("name", sorted(sc.ALL))
def test_round_trip_and_tensor_names(name):
    config = sc.ALL[name]
    _, parsed = resolve(config)
    assert resolve(parsed.to_json())[1] == parsed
    expected, vectors, optional = expected_tensors(parsed)
    shapes = ps.tensor_shapes(config)
    assert set(expected) == set(shapes) and not optional
    for tensor, shape in shapes.items():
        assert all(a in (b, -1) for a, b in zip(expected[tensor], shape)), tensor
    assert "final.norm" in vectors and "final.norm.b" not in vectors


def test_a_reader_has_no_key_and_value_tensors_and_reads_the_owners_cache():
    _, parsed = resolve(sc.SEBI_C)
    expected, _, _ = expected_tensors(parsed)
    assert "l2.mix.q" in expected and "l2.mix.k" not in expected and "l2.mix.v" not in expected
    assert [(e.layer, e.reads_cache_of) for e in parsed.plan()] == [
        (0, None), (1, None), (2, 0), (3, None), (4, None), (5, 3)]
    arch, _ = resolve(sc.SEBI_C)
    specs = arch.build_model(parsed, torch.float32, "meta").cache_specs()
    # the pages keep the widest window and the most kept tokens among owner and readers
    assert specs[0] == PagedKVSpec(1, 32, 33, value_dim=64, keep_first=40) and specs[2] is None
    assert specs[3] == PagedKVSpec(4, 16, 50, value_dim=16, keep_first=17) and specs[5] is None
    assert specs[1] == (PagedKVSpec(2, 64, None, value_dim=32), StateSpec((2 * 32 * 32,)))
    assert specs[4] == StateSpec((4 * 32 * 32,))


def _broken(change):
    config = copy.deepcopy(sc.SEBI_A)
    change(config)
    return config


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=7), "vdim"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "size"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda c: c["layers"][0]["mixer"].update(softcap=0), "softcap"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][1]["mixer"].update(dim=8), "equal"),
    (lambda c: c["layers"][3]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][2]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][2].update(mlp={"kind": "routed"}), "mlp"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
    (lambda c: c["norm"].update(eps=0), "eps"),
    (lambda c: c.pop("layers"), "layers"),
])
def test_refusals_name_the_key(change, word):
    with pytest.raises(ConfigError) as error:
        resolve(_broken(change))
    assert word in str(error.value)


def test_a_reader_of_a_reader_is_refused():
    config = copy.deepcopy(sc.SEBI_A)
    config["layers"].insert(2, copy.deepcopy(config["layers"][1]))
    config["layers"][2]["mixer"]["kv_from"] = 1
    with pytest.raises(ConfigError):
        resolve(config)


def test_defaults_where_the_file_is_silent():
    config = copy.deepcopy(sc.SEBI_B)
    del config["embedding"]
    _, parsed = resolve(config)
    assert parsed.embedding_scale == 1.0 and parsed.logit_softcap is None
    _, full = resolve(sc.SEBI_A)
    assert full.embedding_scale == 3.0 and full.logit_softcap == 9.0


def test_an_attention_layer_without_a_mask_sees_everything():
    config = copy.deepcopy(sc.SEBI_C)
    del config["layers"][2]["mixer"]["mask"]             # a reader of layer 0 without a window
    del config["layers"][3]["mixer"]["vdim"]
    arch, parsed = resolve(config)
    assert resolve(parsed.to_json())[1] == parsed
    specs = arch.build_model(parsed, torch.float32, "meta").cache_specs()
    assert specs[0] == PagedKVSpec(1, 32, None, value_dim=64)       # nothing may be given back
    assert specs[3].value_dim == 16


def test_the_pages_of_kept_first_tokens_are_never_given_back():
    spec = PagedKVSpec(2, 8, window=20, value_dim=4, keep_first=9)
    plain = PagedKVSpec(2, 8, window=20, value_dim=4)
    cache = CacheManager([spec, plain], [None, None], 4, 64, 2, 256, torch.float32, "cpu")
    cache.admit("a")
    length = 0
    for grow in (30, 1, 1, 50, 1, 17):
        cache.reserve([("a", length + grow)])
        length += grow
        cache.commit("a", length)
        cache.check_invariants()
    first = (length - 20 + 1) // 4
    last = (length + 3) // 4
    kept, windowed = (g.tables["a"] for g in cache.paged)
    assert [p for p, x in enumerate(kept) if x >= 0] == [0, 1, 2] + list(range(first, last))
    assert [p for p, x in enumerate(windowed) if x >= 0] == list(range(first, last))
    cache.release("a")
    cache.check_invariants()
    assert all(g.pool.num_free == 64 for g in cache.paged)
