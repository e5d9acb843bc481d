"""Mufevik without a GPU: configuration, tensor names, lanes and state, identities of the plain mechanisms."""
from __future__ import annotations

import pytest
import torch

from tests import mufevik_cases as cases
from tests.plain import mufevik_plain as plain


@pytest.mark.parametrize("name", sorted(cases.CONFIGS))
def test_config_round_trip_and_declared_tensors(name, tmp_path):
    from cpmcu_b200.models.model import Model
    from cpmcu_b200.registry import architecture, load_config

    cfg = cases.CONFIGS[name]()
    folder = cases.write_folder(cfg, cases.random_weights(cfg, 1), str(tmp_path / name))
    arch, typed = load_config(folder)                        # the decay's rank comes from the checkpoint's shapes
    assert arch is architecture("Mufevik")
    again = arch.config_class.from_dict(typed.to_dict())
    assert again == typed
    model = Model(arch.model_spec(typed), None)
    specs = model.weight_specs()
    shapes = cases.tensor_shapes(cfg)
    assert set(specs) == set(shapes)
    assert all(tuple(specs[k].shape) == tuple(shapes[k]) for k in shapes)
    assert model.spec.streams == cfg.get("streams", 0)
    needs = model.cache_needs()
    for layer, n in zip(cfg["layers"], needs):
        m = layer["mixer"]
        if layer["type"] == "delta":
            assert n.kv_heads == 0 and n.state["matrix_state"][0] == (m["heads"], m["dim"], m["vdim"])
            assert n.state["conv_inputs"][0] == (max(m["conv"] - 1, 1), 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"])
        else:
            l, r = m["left"], m["right"]
            assert (n.kv_heads, n.head_dim, n.value_dim or n.head_dim) == (l["kv_heads"], l["dim"], l["vdim"])
            assert n.state["matrix_state"][0] == (r["heads"], r["dim"], r["vdim"])


def test_config_errors_are_collected():
    from cpmcu_b200.config.base import ConfigError
    from cpmcu_b200.config.mufevik import MufevikConfig

    bad = cases.config_a()
    bad["layers"][0]["mixer"]["left"]["kv_heads"] = 3
    bad["layers"][1]["mlp"]["router"]["top"] = 7
    del bad["norm"]
    with pytest.raises(ConfigError) as e:
        MufevikConfig.from_dict(bad)
    assert "kv_heads" in str(e.value) and "top" in str(e.value) and "norm" in str(e.value)


def test_plain_recurrence_in_pieces_and_delta_rule_overwrites():
    g = torch.Generator().manual_seed(3)
    T, H, d, dv = 9, 2, 5, 4
    q, k, v = (torch.randn(T, H, n, generator=g, dtype=torch.float64) for n in (d, d, dv))
    decay = torch.rand(T, H, d, generator=g, dtype=torch.float64)
    beta = torch.rand(T, H, generator=g, dtype=torch.float64)
    whole, _ = plain.matrix_recurrence(q, k, v, decay, beta)
    first, S = plain.matrix_recurrence(q[:4], k[:4], v[:4], decay[:4], beta[:4])
    rest, _ = plain.matrix_recurrence(q[4:], k[4:], v[4:], decay[4:], beta[4:], S)
    assert torch.allclose(torch.cat([first, rest]), whole, atol=1e-12)
    # beta = 1, no decay, a unit key written twice: the second value replaces the first
    key = torch.zeros(2, 1, d, dtype=torch.float64)
    key[:, 0, 2] = 1.0
    vals = torch.randn(2, 1, dv, generator=g, dtype=torch.float64)
    o, _ = plain.matrix_recurrence(key, key, vals, torch.ones(2, 1, 1, dtype=torch.float64), torch.ones(2, 1, dtype=torch.float64))
    assert torch.allclose(o[1, 0], vals[1, 0], atol=1e-12)


def test_plain_routing_keeps_whole_groups_and_uses_plain_scores():
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}
    z = torch.tensor([[0.0, 0.1, 3.0, 0.2, 2.9, 2.8]], dtype=torch.float64)
    corr = torch.tensor([-5.0, -5.0, -5.0, -5.0, -5.1, -5.2], dtype=torch.float64)      # every choice score is negative
    s, choice = plain.route_scores(z, corr, r)
    chosen = choice.topk(2, dim=-1).indices[0].tolist()
    assert sorted(chosen) == [2, 3]                          # the best expert's group, although 4 and 5 score higher than 3
    assert torch.isinf(choice[0, [0, 1, 4, 5]]).all()
    assert abs(float(s.sum()) - 1.0) < 1e-12


def test_plain_hyper_connections_with_identity_weights_are_a_plain_residual():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(4, 3, 8, generator=g, dtype=torch.float64)
    y = torch.randn(4, 8, generator=g, dtype=torch.float64)
    w = {"in": torch.tensor([1.0, 0.0, 0.0], dtype=torch.float64), "mix": torch.eye(3, dtype=torch.float64),
         "out": torch.tensor([1.0, 0.0, 0.0], dtype=torch.float64)}
    assert torch.equal(plain.hyper_read(x, w, ""), x[:, 0])
    new = plain.hyper_write(x, y, w, "")
    assert torch.allclose(new[:, 0], x[:, 0] + y) and torch.equal(new[:, 1:], x[:, 1:])
