"""Reravik without a device: the typed configuration, the model specification's tensor names, lanes and per-sequence
state, the schedule of a repeated group, and identities of the plain implementation's mechanisms."""
import copy

import pytest
import torch

from cpmcu_b200.config.base import ConfigError, architecture_name
from cpmcu_b200.config.reravik import ReravikConfig
from cpmcu_b200.models.model import Model
from cpmcu_b200.registry import architecture
from tests import reravik_cases as cases
from tests.plain import reravik_plain as plain


@pytest.mark.parametrize("name", sorted(cases.CONFIGS))
def test_specification_declares_exactly_the_checkpoint_tensors(name):
    cfgd = cases.CONFIGS[name]()
    arch = architecture(architecture_name(cfgd))
    cfg = arch.config_class.from_dict(cfgd)
    assert cfg.to_dict() == cfgd
    model = Model(arch.model_spec(cfg), None)
    specs = {k: tuple(v.shape) for k, v in model.weight_specs().items()}
    assert specs == cases.tensor_shapes(cfgd)


def test_schedule_of_a_repeated_group_and_its_lanes():
    cfg = ReravikConfig.from_dict(cases.config_a())
    assert cfg.runs() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert plain.run_order(cases.config_a()) == cfg.runs()
    model = Model(architecture("Reravik").model_spec(cfg), None)
    assert [e.lane for e in model.schedule] == list(range(8))            # every run has a cache lane of its own
    needs = model.cache_needs()
    assert [n.kv_heads for n in needs] == [0, 1, 0, 1, 0, 1, 0, 1]
    assert needs[1].head_dim == 48 and needs[1].window == 37 and needs[1].values is False
    assert needs[7].head_dim == 64 and needs[7].window == 70
    assert set(needs[0].state) == {"gru_state", "shift_prev"} and set(needs[1].state) == {"shift_prev"}
    assert needs[0].state["gru_state"][0] == (80,) and needs[2].state["gru_state"][0] == (72,)
    no_loop = ReravikConfig.from_dict(cases.config_c())
    assert no_loop.runs() == [(0, None), (1, None), (2, None)]
    spec = architecture("Reravik").model_spec(no_loop)
    assert spec.pass_entry is None and "loop.step" not in Model(spec, None).weight_specs()


def test_configuration_errors_are_collected():
    bad = cases.config_a()
    bad["layers"][0]["type"] = "lstm"
    del bad["layers"][1]["mixer"]["kv_rank"]
    bad["loop"]["stop"] = 9
    bad["width"] = 95
    with pytest.raises(ConfigError) as e:
        ReravikConfig.from_dict(bad)
    text = str(e.value)
    for piece in ("layers[0]", "kv_rank", "loop", "width"):
        assert piece in text


def test_plain_token_shift_and_recurrence_identities():
    torch.manual_seed(0)
    h = torch.randn(7, 6, dtype=torch.float64)
    assert torch.equal(plain.token_shift(h, torch.zeros(6, dtype=torch.float64)), h)
    shifted = plain.token_shift(h, torch.ones(6, dtype=torch.float64))
    assert torch.allclose(shifted[1:], h[:-1]) and torch.equal(shifted[0], torch.zeros(6, dtype=torch.float64))
    # z = 1 everywhere (huge bias): the state is the candidate of the current token; z = 0: it stays zero
    w = {"z": torch.zeros(5, 6), "z.b": torch.full((5,), 60.0), "x": torch.randn(5, 6), "x.b": torch.zeros(5),
         "g": torch.randn(5, 6), "o": torch.eye(5)}
    w = {"m." + k: v.double() for k, v in w.items()}
    u = h @ w["m.x"].T
    g = h @ w["m.g"].T
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    assert torch.allclose(plain.min_gru(h, w, "m."), cand * g * torch.sigmoid(g))
    w["m.z.b"] = torch.full((5,), -60.0, dtype=torch.float64)
    assert plain.min_gru(h, w, "m.").abs().max() < 1e-20


def test_plain_window_visibility():
    v = plain.visible(6, 3)
    assert v[5].tolist() == [False, False, False, True, True, True]
    assert v[1].tolist() == [True, True, False, False, False, False]
    assert plain.visible(4, None)[3].all() and plain.visible(4, 1).sum() == 4


def test_plain_attention_reads_only_its_window():
    """A change of a token outside every later query's window leaves those queries' outputs as they were."""
    cfg = cases.config_c()
    w = {k: v.double() for k, v in cases.random_weights(cfg, 3).items()}
    h = torch.randn(9, cfg["width"], dtype=torch.float64)
    mixer = copy.deepcopy(cfg["layers"][1]["mixer"])            # window 2
    base = plain.latent_attention(h, w, "l1.mix.", mixer, 1e-6)
    h2 = h.clone()
    h2[3] += 1.0
    moved = plain.latent_attention(h2, w, "l1.mix.", mixer, 1e-6)
    assert torch.allclose(moved[5:], base[5:]) and not torch.allclose(moved[4], base[4])
