"""Logozen on the host: configuration, plan, tensor names, the random-weights writer, and the plain implementation's
own consistency (prompt against token-by-token recurrences)."""
import copy
import json
import os

import pytest
import torch

import logozen_models as zoo
import plain_logozen
from mini_engine_b200.config.model_config import ConfigError, LogozenConfig
from mini_engine_b200.config.registry import get_architecture, load_model_config
from mini_engine_b200.parts import DecoderModel, KVCacheNeed, StateNeed
from mini_engine_b200.weights import write_random_model
from mini_engine_b200.weights.loader import expected_disk_tensors


def _model(cfg_dict):
    cfg = LogozenConfig.from_dict(cfg_dict)
    return cfg, DecoderModel(get_architecture("Logozen").plan(cfg))


@pytest.mark.parametrize("name", sorted(zoo.ALL))
def test_the_plan_declares_the_tensors_of_the_design(name):
    cfg_dict, seed, _ = zoo.ALL[name]
    cfg, model = _model(cfg_dict)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.streams, cfg.canon_taps) == (cfg_dict["vocab"], cfg_dict["width"],
                                                                              cfg_dict["streams"], cfg_dict["canon"]["taps"])
    want = {k: tuple(v.shape) for k, v in zoo.tensors(cfg_dict, seed).items()}
    got = {k: e.shape for k, e in expected_disk_tensors(model).items()}
    assert got == want


def test_cache_needs_follow_the_layers():
    _, model = _model(zoo.P)
    m0, m1 = zoo.P["layers"][0]["mixer"], zoo.P["layers"][1]["mixer"]
    assert KVCacheNeed(1, m0["kv_rank"] + m0["rot_dim"], None, planes=1) in model.slot_needs[0]
    assert {n.name for n in model.slot_needs[0] if isinstance(n, StateNeed)} == {"canon1", "canon2"}
    names = {n.name: n.shape for n in model.slot_needs[1] if isinstance(n, StateNeed)}
    assert names == {"S": (m1["heads"], m1["dim"], m1["vdim"]), "n": (m1["heads"], m1["dim"]), "m": (m1["heads"],),
                     "canon1": (zoo.P["canon"]["taps"] - 1, zoo.P["width"])}          # layer 1 has no feed-forward
    _, one_tap = _model(zoo.Q)
    assert not [n for n in one_tap.slot_needs[0] if isinstance(n, StateNeed)]          # one tap keeps no inputs


def test_config_is_found_by_its_architecture_key(tmp_path):
    with open(tmp_path / "config.json", "w") as f:
        json.dump(zoo.S, f)
    cfg = load_model_config(str(tmp_path))
    assert isinstance(cfg, LogozenConfig) and cfg.num_hidden_layers == 2 and cfg.layers[0]["mixer"]["kv_rank"] == 136
    assert LogozenConfig.from_dict(cfg.to_json_dict()).layers == cfg.layers


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0].update(mlp={"kind": "routed", "ff": 8}), "dense"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].update(gate_cap=0.0), "gate_cap"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(streams=17), "streams"),
    (lambda c: c["canon"].update(taps=0), "canon_taps"),
])
def test_what_the_engine_cannot_honour_is_refused(change, text):
    c = copy.deepcopy(zoo.P)
    change(c)
    with pytest.raises(ConfigError, match=text):
        LogozenConfig.from_dict(c)


def test_random_weights_writer_makes_a_model_the_plain_implementation_runs(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), zoo.R, seed=3, matrix_std=0.1)
    cfg, w = plain_logozen.load_folder(folder)
    assert set(w) == set(zoo.tensors(zoo.R, 0))
    assert abs(float(w["l0.hc1.mix"].diagonal().mean()) - 1.0) < 0.3                 # mixing matrices start near the identity
    logits = plain_logozen.forward(cfg, w, [1, 2, 3, 4, 5])
    assert logits.shape == (5, zoo.R["vocab"]) and torch.isfinite(logits).all()


def test_plain_model_is_causal_and_layer_outputs_have_the_models_shape():
    cfg, w = plain_logozen.load_folder(zoo.folder("P"))
    ids = torch.randint(0, cfg["vocab"], (30,), generator=torch.Generator().manual_seed(0)).tolist()
    full, layers = plain_logozen.forward(cfg, w, ids, return_layers=True)
    assert layers.shape == (len(cfg["layers"]), 30, cfg["width"])
    part = plain_logozen.forward(cfg, w, ids[:17])
    assert torch.allclose(full[:17], part, atol=1e-9)
