"""The Givopel configuration, its order of layers and its tensors (no GPU), and the plain implementation against itself."""
import copy

import numpy as np
import pytest

from givopel_cases import CASES, random_weights, tensor_shapes


def _typed(raw):
    from xeno_rt_b200.config import config_from_dict
    return config_from_dict(raw)


@pytest.mark.parametrize("name", list(CASES))
def test_the_spec_asks_for_the_designs_tensors(name):
    raw, ranks, _ = CASES[name]
    shapes = tensor_shapes(raw, ranks)
    arch, cfg = _typed(raw)
    assert arch.name == "Givopel"
    from xeno_rt_b200.core import ConfigError
    with pytest.raises(ConfigError):  # the ranks are sizes of tensors only
        arch.build_spec(cfg)
    spec = arch.build_spec(cfg.with_tensor_shapes(shapes))
    spec.validate()
    assert {e.name: tuple(e.shape) for e in spec.expected_tensors()} == {k: tuple(v) for k, v in shapes.items()}
    # written back and read again it is the same configuration
    assert _typed(cfg.to_dict())[1] == cfg


def test_order_of_layers_and_where_a_pass_begins():
    arch, cfg = _typed(CASES["loop-middle"][0])
    assert cfg.order() == [(0, False), (1, True), (2, False), (1, True), (2, False), (1, True), (2, False)]
    spec = arch.build_spec(cfg.with_tensor_shapes(tensor_shapes(*CASES["loop-middle"][:2])))
    assert [(p.layer, p.before, p.cache_from) for p in spec.schedule] == \
        [(0, None, None)] + [(1, "loop_in", None), (2, None, None)] * 3
    arch, cfg = _typed(CASES["no-loop"][0])
    assert cfg.order() == [(0, False), (1, False)]
    assert arch.build_spec(cfg.with_tensor_shapes(tensor_shapes(*CASES["no-loop"][:2]))).stream_parts == {}
    raw = copy.deepcopy(CASES["loop-middle"][0])
    raw["loop"] = {"start": 0, "stop": 2, "times": 1}
    assert _typed(raw)[1].order() == [(0, True), (1, False), (2, False)]


@pytest.mark.parametrize("change,word", [
    (lambda r: r["layers"][0].update(type="window"), "type"),
    (lambda r: r["layers"][1]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda r: r["layers"][1]["mixer"]["left"]["rot"].update(dims=34), "rot.dims"),
    (lambda r: r["layers"][1]["mixer"]["right"].pop("conv"), "conv"),
    (lambda r: r["loop"].update(stop=9), "loop"),
    (lambda r: r["layers"][0]["mlp"].update(kind="routed"), "mlp.kind"),
    (lambda r: r.pop("width"), "width"),
    (lambda r: r["norm"].pop("eps"), "eps"),
    (lambda r: r["layers"][0]["mixer"].update(tau=0), "tau"),
])
def test_a_bad_configuration_is_refused_with_its_key(change, word):
    from xeno_rt_b200.core import ConfigError
    raw = copy.deepcopy(CASES["loop-middle"][0])
    change(raw)
    with pytest.raises(ConfigError, match=word):
        _typed(raw)


def test_the_plain_model_is_causal_and_its_mechanisms_matter():
    from plain import givopel
    raw, ranks, seed = CASES["loop-middle"]
    w = random_weights(raw, ranks, seed)
    tokens = np.random.default_rng(0).integers(0, raw["vocab"], size=40).tolist()
    full = givopel.forward(raw, w, tokens)
    assert np.abs(givopel.forward(raw, w, tokens[:25]) - full[:25]).max() < 1e-9
    for change in (lambda r: r["layers"][1]["mixer"]["left"].pop("rot"),
                   lambda r: r["layers"][1]["mixer"]["left"]["rot"].pop("scaling"),
                   lambda r: r["loop"].update(times=2),
                   lambda r: r["layers"][0]["mixer"].update(tau=50.0),
                   lambda r: r.update(logit_softcap=3.0)):
        other = copy.deepcopy(raw)
        change(other)
        assert np.abs(givopel.forward(other, w, tokens) - full).max() > 1e-2 * np.abs(full).max()
