"""The Buguzen configuration, its model's tensor names and schedule, and the cache it asks for (no GPU)."""
import copy

import pytest
import torch

import buguzen_tiny as bt
import plain_buguzen as plain
from alpacca_b200.config import BuguzenConfig, ConfigError, config_from_dict
from alpacca_b200.engine.loading import build_model
from alpacca_b200.parts import KVSpec, StateSpec


@pytest.mark.parametrize("name", list(bt.CONFIGS))
def test_tensor_names_and_shapes(name):
    cfg = config_from_dict(bt.CONFIGS[name])
    assert isinstance(cfg, BuguzenConfig) and cfg.max_positions is None
    model = build_model(cfg, "float32", "cpu", 128)
    specs = {s.name: tuple(s.shape) for s in model.param_specs()}
    assert specs == bt.tensor_shapes(bt.CONFIGS[name])


@pytest.mark.parametrize("name", list(bt.CONFIGS))
def test_schedule_and_cache_entries(name):
    """A layer inside the loop runs once per pass, each run with a cache entry of its own; the pass offset enters
    before the first layer of every pass and nowhere else."""
    raw = bt.CONFIGS[name]
    cfg = config_from_dict(raw)
    model = build_model(cfg, "float32", "cpu", 128)
    order = plain.run_order(raw)
    assert cfg.run_order() == order
    assert [r.layer for r in model.spec.schedule] == [i for i, _ in order]
    for r, (i, t) in zip(model.spec.schedule, order):
        first = t is not None and i == raw["loop"]["start"]
        assert (r.enter is not None) == first
        if first:
            assert r.enter[1] == t
    specs = model.cache_entry_specs()
    assert len(specs) == len(order)
    for spec, (i, _) in zip(specs, order):
        layer = raw["layers"][i]
        mx = layer["mixer"]
        if layer["type"] == "lightning":
            assert spec == StateSpec((mx["heads"], mx["dim"], mx["vdim"]), torch.float32)
        elif layer["type"] == "attention":
            assert spec == KVSpec(2 * mx["kv_heads"], mx["dim"], mx["mask"]["size"], value_heads=mx["kv_heads"],
                                  value_dim=mx["vdim"])
        else:
            assert spec == KVSpec(mx["kv_heads"], mx["dim"], mx["mask"]["size"], value_heads=mx["kv_heads"],
                                  value_dim=mx["dim"])


def test_values_of_their_own_size_in_the_cache():
    from alpacca_b200.cache import SequenceCache
    cache = SequenceCache([KVSpec(4, 16, 9, value_heads=2, value_dim=24), KVSpec(2, 16)], 256, 2, 256, torch.float32, "cpu")
    g = cache.kv_groups[0]
    assert tuple(g.k.shape[2:]) == (4, 64, 16) and tuple(g.v.shape[2:]) == (2, 64, 24)
    assert g.bytes_per_token == (4 * 16 + 2 * 24) * 4 and cache.kv_groups[1].bytes_per_token == 2 * 2 * 16 * 4


def _broken(change):
    raw = copy.deepcopy(bt.TINY_U)
    change(raw)
    return raw


@pytest.mark.parametrize("change,words", [
    (lambda c: c["layers"][0].update(type="convolution"), "not supported"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5, 0.9]), "decay"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5, 0.9, 1.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "cannot share"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("high"), "high"),
    (lambda c: c["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][0]["mixer"]["mask"].pop("size"), "size"),
    (lambda c: c["loop"].update(stop=4), "loop"),
    (lambda c: c["loop"].update(start=2), "loop"),
    (lambda c: c["token_side"].pop("dim"), "dim"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "dense"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_faults_are_named(change, words):
    with pytest.raises(ConfigError) as e:
        config_from_dict(_broken(change))
    assert words in str(e.value)


def test_optional_parts_may_be_left_out():
    raw = copy.deepcopy(bt.TINY_U)
    del raw["loop"], raw["token_side"]
    del raw["layers"][0]["mixer"]["rot"]["scaling"]
    cfg = config_from_dict(raw)
    model = build_model(cfg, "float32", "cpu", 64)
    names = {s.name for s in model.param_specs()}
    assert "loop.step" not in names and "side.embed" not in names and not any(".side." in n for n in names)
    assert cfg.to_dict()["layers"] == raw["layers"] and "loop" not in cfg.to_dict()


def test_a_rotation_over_no_dims_is_no_rotation():
    raw = copy.deepcopy(bt.TINY_U)
    raw["layers"][0]["mixer"]["rot"]["dims"] = 0
    model = build_model(config_from_dict(raw), "float32", "cpu", 64)
    assert model.spec.layers[0].mixer.position is None and model.spec.layers[2].mixer.position is not None


def test_frequency_scaling_of_the_rotation():
    """The package's table of angles against the plain frequencies, for a scaling whose blended range is hit."""
    from alpacca_b200.models.buguzen import _scaling
    from alpacca_b200.parts import scaled_inv_freq
    for rot in (bt.TINY_U["layers"][2]["mixer"]["rot"], bt.TINY_W["layers"][1]["mixer"]["rot"],
                bt.TINY_U["layers"][0]["mixer"]["rot"], bt.TINY_X["layers"][0]["mixer"]["rot"]):
        got = scaled_inv_freq(rot["dims"], rot["base"], _scaling(rot.get("scaling"))).numpy()
        assert abs(got - plain.frequencies(rot)).max() <= 1e-15
