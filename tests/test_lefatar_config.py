"""The Lefatar configuration, its place in the registry, its tensors and what it asks of the cache (no GPU), and
the plain implementation's own consistency (a state that is carried equals a whole sequence)."""
import copy
import json

import numpy as np
import pytest

import lefatar_tiny as lt
import plain_lefatar as plain
from alpacca_b200.config import ConfigError, LefatarConfig, config_from_dict, load_config
from alpacca_b200.engine.loading import build_model, write_random_model_dir
from alpacca_b200.parts import KVSpec, StateSpec
from alpacca_b200.weights import FolderSource
from alpacca_b200.weights.loader import check_names


def test_registry_reads_the_architecture_key():
    cfg = config_from_dict(copy.deepcopy(lt.TINY_P))
    assert isinstance(cfg, LefatarConfig) and cfg.vocab == 97 and cfg.eps == 1e-5
    assert cfg.max_positions is None and cfg.stop_tokens == () and len(cfg.layers) == 4
    assert cfg.to_dict()["architecture"] == "Lefatar" and cfg.to_dict()["layers"] == lt.TINY_P["layers"]


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1].__setitem__("type", "conv"), "not supported"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("count", 4), "equal groups"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 5), "cannot be chosen"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 14), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("gate_cap", 0), "gate_cap"),
    (lambda c: c.__setitem__("norm", {}), "norm.eps"),
    (lambda c: c.__setitem__("layers", []), "at least one layer"),
    (lambda c: c["layers"][0].__setitem__("mlp", {"kind": "conv"}), "kind"),
])
def test_faults_are_named(edit, word):
    c = copy.deepcopy(lt.TINY_P)
    edit(c)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(c)


@pytest.mark.parametrize("name", list(lt.CONFIGS))
def test_tensors_and_cache_entries(name, tmp_path):
    cfg = lt.CONFIGS[name]
    model = build_model(copy.deepcopy(cfg), "float32", "cpu", 128)
    table = {n: ("BF16", s) for n, s in lt.tensor_shapes(cfg).items()}
    check_names(model.param_specs(), table)
    specs = model.cache_entry_specs()
    assert len(specs) == len(cfg["layers"])
    for layer, spec in zip(cfg["layers"], specs):
        mx = layer["mixer"]
        if layer["type"] == "mlstm":
            assert isinstance(spec, StateSpec) and spec.shape[0] == mx["heads"]
            assert spec.shape[1] >= mx["dim"] * mx["vdim"] + mx["dim"] + 1
        else:
            assert spec == KVSpec(1, mx["kv_rank"] + mx["rot_dim"], None, values=False)
    # the random-weights mode writes a folder that loads again under the same names
    d = write_random_model_dir(tmp_path / name, copy.deepcopy(cfg), seed=1)
    assert json.loads((d / "config.json").read_text())["layers"] == cfg["layers"]
    assert isinstance(load_config(d), LefatarConfig)
    src = FolderSource(d)
    check_names(model.param_specs(), src.table())
    src.close()


def test_a_latent_group_keeps_one_tensor():
    import torch
    from alpacca_b200.cache import SequenceCache
    cache = SequenceCache([KVSpec(1, 24, None, values=False), KVSpec(2, 16)], 256, 2, 256, torch.float32, "cpu")
    latent = cache.entry_view(0, [None, None])
    assert latent.v is None and tuple(latent.k.shape) == (4, 1, 64, 24)
    assert cache.kv_groups[0].bytes_per_token == 24 * 4 and cache.kv_groups[1].bytes_per_token == 2 * 2 * 16 * 4
    assert "key/value group" in cache.describe()


def test_plain_matrix_memory_carries_its_state():
    rng = np.random.default_rng(0)
    mx = {"heads": 2, "dim": 8, "vdim": 12, "gate_cap": 10.0}
    w = {"q": rng.normal(0, .3, (16, 20)), "k": rng.normal(0, .3, (16, 20)), "v": rng.normal(0, .3, (24, 20)),
         "g": rng.normal(0, .3, (24, 20)), "o": rng.normal(0, .3, (20, 24)), "norm": 1 + rng.normal(0, .1, 24),
         "i": rng.normal(0, .3, (2, 20)), "i.b": rng.normal(0, 1, 2), "f": rng.normal(0, .3, (2, 20)),
         "f.b": rng.normal(3, 1, 2)}
    h = rng.normal(0, 1, (30, 20))
    whole, _ = plain.mlstm(h, w, mx, 1e-6)
    a, st = plain.mlstm(h[:11], w, mx, 1e-6)
    b, _ = plain.mlstm(h[11:], w, mx, 1e-6, state=st)
    assert np.abs(np.concatenate([a, b]) - whole).max() < 1e-12


def test_plain_router_by_hand():
    rt = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 2}}
    z = np.log(np.array([[0.05, 0.30, 0.25, 0.02, 0.28, 0.10]]))      # groups (0,1) (2,3) (4,5): best two are 0 and 2
    idx, w = plain.route(z, np.eye(6), rt)
    assert idx.tolist() == [[1, 4]]
    assert np.allclose(w, 2.0 * np.array([[0.30, 0.28]]) / 0.58)


def test_plain_sink_by_hand():
    p = plain.softmax_with_sink(np.array([[0.0, 0.0]]), 0.0)
    assert np.allclose(p, [[1 / 3, 1 / 3]])


def test_show_command_reads_a_lefatar_folder(tmp_path, capsys):
    from alpacca_b200.cli import main
    d = write_random_model_dir(tmp_path / "m", copy.deepcopy(lt.TINY_Q), seed=2)
    assert main(["show", str(d), "--tensors"]) == 0
    out = capsys.readouterr().out
    assert "Lefatar: 3 layers" in out and "no limit on positions" in out and "l1.mix.dkv.norm" in out
