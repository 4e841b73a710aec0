"""Pugadra's configuration and plan on the CPU: what is read, what is refused, which tensors the model asks for."""
import copy

import pytest

import pugadra_models as zoo
from mini_engine_b200.config import ConfigError, PugadraConfig
from mini_engine_b200.config.registry import get_architecture
from mini_engine_b200.engine.model_runner import plan_cache_groups
from mini_engine_b200.parts import StateNeed
from mini_engine_b200.weights.loader import expected_disk_tensors
from mini_engine_b200.weights.random_init import build_model_from_config_dict


@pytest.mark.parametrize("name", sorted(zoo.ALL))
def test_the_model_asks_for_the_designs_tensors(name):
    cfg, seed, _ = zoo.ALL[name]
    _, model = build_model_from_config_dict(cfg)
    want = {k: tuple(v.shape) for k, v in zoo.tensors(cfg, seed).items()}
    got = {k: tuple(e.shape) for k, e in expected_disk_tensors(model).items()}
    assert got == want


def test_every_number_comes_from_the_file():
    c = PugadraConfig.from_dict(zoo.A)
    assert (c.vocab_size, c.hidden_size, c.norm_eps, c.residual_mult, c.side_dim) == (101, 64, 1e-6, 0.5, 8)
    plan = get_architecture("Pugadra").plan(c)
    m0, m1, m2 = (plan.blocks[i].mixer.args for i in range(3))
    assert (m0["num_heads"], m0["num_kv_heads"], m0["dim"], m0["vdim"], m0["conv_taps"], m0["window"]) == (4, 2, 16, 24, 3, 40)
    assert m1["own_kv"] is False and m1["window"] == 24 and m0["cache_window"] == 40
    assert m2["window"] is None and m2["cache_window"] is None
    assert plan.schedule[1].kv_slot == 0 and plan.schedule[3].kv_slot == 2 and plan.schedule[0].kv_slot is None
    assert plan.blocks[2].feed_forward is None and plan.blocks[1].feed_forward.kind == "routed_experts"
    assert plan.blocks[1].args["side"]["first"] == 8 and plan.tables["token_side"] == ("side.embed", 101, 32)
    assert plan.tie_word_embeddings


def test_cache_groups_keep_the_widest_window_of_their_readers():
    _, model = build_model_from_config_dict(zoo.C)
    groups, location, states = plan_cache_groups(model)
    assert [(g.window, g.num_kv_heads, g.head_dim, g.planes) for g in groups] == [(128, 2, 64, 2), (None, 4, 64, 2)]
    assert sorted(location) == [0, 2]                       # the layer that borrows keys has no pages of its own
    assert states[1] == [StateNeed((2, 8 * 64), "float32", "conv")]        # ... and a state for its queries only
    assert states[0] == [StateNeed((2, 8 * 64 + 2 * 128), "float32", "conv")]


def test_a_model_without_convolution_has_no_state():
    cfg = copy.deepcopy(zoo.D)
    _, model = build_model_from_config_dict(cfg)
    assert plan_cache_groups(model)[2] == {}


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].update(type="recurrence"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), "differ"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "router.top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c["layers"][0]["mlp"].update(limit=-1.0), "limit"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.pop("width"), "width"),
])
def test_what_is_refused(edit, text):
    c = copy.deepcopy(zoo.A)
    edit(c)
    with pytest.raises(ConfigError, match=text):
        PugadraConfig.from_dict(c)
