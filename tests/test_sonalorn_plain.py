"""The Sonalorn design without a GPU: its configuration, its plan (tensor names,
the order of layer runs, which runs share tensors) and hand computations that pin
the plain implementation's reading of each mechanism."""
import math

import pytest
import torch

from plain import sonalorn as plain

DELTA = dict(heads=4, kv_heads=2, dim=8, vdim=6, conv=3)
ATTN = dict(heads=4, kv_heads=2, dim=8, vdim=12, scale=0.4, q_temp={"coef": 0.5, "every": 4})
MOE = {"kind": "moe", "expert": {"ff": 10, "limit": 0.75},
       "router": {"experts": 5, "identity": 1, "top": 2, "groups": {"count": 3, "keep": 2}}}
CFG = dict(architecture="Sonalorn", vocab=50, width=24, max_positions=64, norm={"eps": 1e-5},
           layers=[{"type": "delta", "mixer": DELTA, "mlp": {"kind": "dense", "ff": 40}},
                   {"type": "attention", "mixer": ATTN, "mlp": MOE},
                   {"type": "delta", "mixer": DELTA, "mlp": None},
                   {"type": "attention", "mixer": ATTN, "mlp": MOE, "weights_of": 1}])


def test_configuration_reads_and_refuses():
    import grout_b200.architectures  # noqa: F401
    from grout_b200.config import ConfigError, resolve_architecture
    arch = resolve_architecture(CFG)
    cfg = arch.config_cls.from_dict(CFG)
    assert arch.name == "Sonalorn" and cfg.weights_layer(3) == 1 and cfg.weights_layer(2) == 2
    bad = dict(CFG, layers=[dict(CFG["layers"][0], type="conv")])
    with pytest.raises(ConfigError, match="type"):
        arch.config_cls.from_dict(bad)
    bad = dict(CFG, layers=CFG["layers"][:3] + [dict(CFG["layers"][3], weights_of=3)])
    with pytest.raises(ConfigError, match="weights_of"):
        arch.config_cls.from_dict(bad)
    moe = dict(MOE, router=dict(MOE["router"], groups={"count": 4, "keep": 1}))
    bad = dict(CFG, layers=[dict(CFG["layers"][1], mlp=moe)])
    with pytest.raises(ConfigError, match="equal groups"):
        arch.config_cls.from_dict(bad)
    with pytest.raises(ConfigError, match="max_positions"):
        arch.config_cls.from_dict({k: v for k, v in CFG.items() if k != "max_positions"})


def test_plan_names_tensors_and_orders_layer_runs():
    import grout_b200.architectures  # noqa: F401
    from grout_b200.config import resolve_architecture
    from grout_b200.engine.model import expected_tensors
    arch = resolve_architecture(CFG)
    plan = arch.plan(arch.config_cls.from_dict(CFG))
    assert [e.layer for e in plan.schedule] == [0, 1, 2, 1]          # the fourth run uses layer 1's tensors
    assert all(e.cache_of is None for e in plan.schedule)            # on a cache of its own
    exp = expected_tensors(plan)
    assert exp["l0.mix.q.conv"].shape == (16, 3) and exp["l0.mix.v"].shape == (24, 24)
    assert exp["l1.mix.o"].shape == (24, 48) and exp["l1.mix.v"].shape == (24, 24)
    assert exp["l1.mlp.router"].shape == (6, 24) and exp["l1.mlp.e4.down"].shape == (24, 10)
    assert exp["pos"].shape == (64, 24) and exp["embed.norm"].shape == (24,)
    assert "l2.norm2" not in exp and "l2.ls2" not in exp and "l2.ls1" in exp
    assert not any(n.startswith("l3.") for n in exp)


def test_delta_rule_by_hand():
    """Two tokens, dk = 2, dv = 1: S after the first write is beta k v; the second
    token decays it, corrects it towards its own value and reads with the write in."""
    q = torch.tensor([[1.0, 0.0], [0.0, 1.0]])
    k = torch.tensor([[1.0, 0.0], [0.6, 0.8]])
    v = torch.tensor([[2.0], [1.0]])
    beta, g = torch.tensor([0.5, 0.25]), torch.tensor([0.9, 0.5])
    o, S = plain.delta_rule(q, k, v, beta, g)
    assert o[0].item() == pytest.approx(1.0)                         # S = [[1], [0]]
    s1 = torch.tensor([0.5, 0.0])                                    # decayed
    u = 0.25 * (1.0 - 0.6 * 0.5)
    want = s1 + torch.tensor([0.6, 0.8]) * u
    assert torch.allclose(S[:, 0], want.double())
    assert o[1].item() == pytest.approx(float(want[1]))


def test_short_convolution_starts_from_zeros():
    x = torch.tensor([[1.0], [2.0], [4.0]])
    w = torch.tensor([[100.0, 10.0, 1.0]])                           # the last tap is the current token's
    assert plain.short_conv(x, w)[:, 0].tolist() == [1.0, 12.0, 124.0]


def test_query_temperature_and_sink():
    t = plain.query_temperature([0, 2, 3, 6, 7, 11], 0.5, 4)
    want = [1.0, 1.0, 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(3), 1 + 0.5 * math.log(4)]
    assert torch.allclose(t, torch.tensor(want, dtype=torch.float64))
    q = torch.zeros(1, 2, dtype=torch.float64)
    out = plain.sink_attention(q, torch.ones(1, 2, dtype=torch.float64), torch.tensor([[3.0]], dtype=torch.float64), 1.0)
    assert out.item() == pytest.approx(1.5)                          # exp(0) / (1 + exp(0)) of the value


def test_choice_by_groups_with_corrected_scores():
    """Six outputs in three pairs; the correction lifts the last pair's score above
    the first pair's, whose own scores are larger; weights stay uncorrected."""
    h = torch.eye(6, dtype=torch.float64)[:1] * 0 + 1.0
    router = torch.zeros(6, 6, dtype=torch.float64)
    router[:, 0] = torch.tensor([2.0, 0.1, 1.5, 1.4, 0.0, 0.2])
    hh = torch.zeros(1, 6, dtype=torch.float64)
    hh[0, 0] = 1.0
    corr = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 0.6], dtype=torch.float64)
    r = {"top": 2, "groups": {"count": 3, "keep": 2}}
    chosen, w = plain.route(hh, router, corr, r)
    s = torch.softmax(router[:, 0], 0)
    assert chosen[0].tolist() == [5, 0]                              # groups 0 and 2 stay; 2 and 3 cannot be chosen
    assert torch.allclose(w[0], s[[5, 0]])
    corr[:] = -1.0                                                   # all choice scores negative: still chosen by order
    chosen, _ = plain.route(hh, router, corr, {"top": 2, "groups": {"count": 3, "keep": 1}})
    assert chosen[0].tolist() == [0, 1]
