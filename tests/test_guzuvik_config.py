"""Configuration, tensor list and cache book-keeping of the Guzuvik decoder (no GPU)."""
import copy

import pytest

from guzuvik_cases import CASES, random_config, tensor_shapes


def _spec(raw):
    from xeno_rt_b200.config import config_from_dict
    arch, config = config_from_dict(raw)
    return arch, config, arch.build_spec(config)


@pytest.mark.parametrize("name", list(CASES))
def test_the_spec_expects_exactly_the_tensors_of_the_design(name):
    raw = CASES[name][0]
    arch, config, spec = _spec(raw)
    assert arch.name == "Guzuvik"
    spec.validate()
    got = {e.name: tuple(e.shape) for e in spec.expected_tensors()}
    assert got == {k: tuple(v) for k, v in tensor_shapes(raw).items()}
    assert config.to_dict() == raw and _spec(config.to_dict())[1] == config


def test_random_configurations_give_their_tensors_too():
    import numpy as np
    for seed in range(30):
        raw = random_config(np.random.default_rng(seed))
        raw = copy.deepcopy(raw)
        for layer in raw["layers"]:
            if layer["type"] == "attention":
                layer["mixer"]["scale"] = float(layer["mixer"]["scale"])
        spec = _spec(raw)[2]
        assert {e.name: tuple(e.shape) for e in spec.expected_tensors()} == {k: tuple(v) for k, v in tensor_shapes(raw).items()}


def test_every_bad_key_is_reported_in_one_error():
    from xeno_rt_b200.core import ConfigError
    raw = copy.deepcopy(CASES["mixed"][0])
    raw["width"] = 0
    raw["layers"][0]["mixer"]["kv_heads"] = 3          # 4 heads are no multiple
    raw["layers"][0]["mixer"]["mask"].pop("size")
    raw["layers"][1]["mixer"]["norm_groups"] = 5        # 24 channels are no multiple
    raw["layers"][1]["mlp"] = {"kind": "swiglu"}
    raw["layers"][3]["mlp"]["router"]["top"] = 9
    raw["layers"][2]["type"] = "conv"
    raw["embedding"]["bigram"]["buckets"] = -1
    with pytest.raises(ConfigError) as err:
        _spec(raw)
    text = str(err.value)
    for piece in ("width", "kv_heads", "mask.size", "norm_groups", "swiglu", "top 9", "'conv'", "buckets"):
        assert piece in text, piece


def test_layers_that_blend_values_must_agree_on_their_size():
    from xeno_rt_b200.core import ConfigError
    raw = copy.deepcopy(CASES["mixed"][0])
    raw["layers"][2]["mixer"]["vdim"] = 32
    with pytest.raises(ConfigError):
        _spec(raw)


def test_a_windowed_group_gives_blocks_back_but_keeps_those_of_the_first_tokens():
    from xeno_rt_b200.cache import Cache, KVNeed
    from xeno_rt_b200.core import DType
    needs = [KVNeed(2, 16, 100, 70), KVNeed(2, 16, 100, 0), KVNeed(2, 16, None, 0), KVNeed(1, 16, 30, 64)]
    cache = Cache(needs, 64 * 40, 1 << 20, DType.F32, "cpu", max_slots=4)
    slot = cache.open_slot()
    cache.reserve(slot, 500)
    cache.advance(slot, 500)
    cache.check()
    held = {(g.need.window, g.need.keep_first): g.held_blocks(slot, 8) for g in cache.kv_groups}
    # a token at 500 sees keys from 401 on (block 6 on), or from 471 on (block 7 on)
    assert held[(100, 70)] == [0, 1, 6, 7] and held[(100, 0)] == [6, 7] and held[(None, 0)] == list(range(8))
    assert held[(30, 64)] == [0, 7]
    for _ in range(200):
        cache.reserve(slot, 1)
        cache.advance(slot, 1)
    cache.check()
    assert cache.kv_groups[0].held_blocks(slot, 11) == [0, 1, 9, 10]
    other = cache.open_slot()   # blocks that were given back are handed out again
    cache.reserve(other, 64 * 20)
    cache.advance(other, 64 * 20)
    cache.check()
    cache.close_slot(slot)
    cache.close_slot(other)
    cache.check()
    assert cache.blocks_free() == cache.n_blocks
