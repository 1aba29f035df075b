"""The plain Suvazen implementation against hand computation, and the design's
configuration and plan (no GPU)."""
import math

import pytest
import torch

from plain import suvazen as plain

MIXER = dict(heads=6, kv_heads=3, dim=16, vdim=16, scale=0.2, softcap=9.0, mask={"size": 5},
             rot={"dims": 8, "base": 5000.0,
                  "scaling": {"factor": 3.0, "low": 1.0, "high": 5.0, "original": 40}})
CONFIG = dict(architecture="Suvazen", vocab=50, width=24, norm={"eps": 1e-5}, residual_mult=0.6,
              logit_scale=0.8, logit_softcap=11.0, loop={"start": 1, "stop": 3, "times": 2},
              layers=[dict(type="attention", mixer=MIXER, mlp={"kind": "dense", "ff": 40}),
                      dict(type="attention", mixer=dict(MIXER, heads=3, mask=None, softcap=None),
                           mlp=None),
                      dict(type="attention", mixer=dict(MIXER, dim=8, vdim=8, rot=None),
                           mlp={"kind": "dense", "ff": 16}),
                      dict(type="attention", mixer=MIXER, mlp={"kind": "dense", "ff": 32})])


def test_layer_norm_by_hand():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]])
    w = torch.tensor([1.0, 2.0, 0.5, 1.0])
    b = torch.tensor([0.0, 1.0, -1.0, 0.5])
    mean, var = 3.0, (4.0 + 1.0 + 0.0 + 9.0) / 4.0
    want = [(v - mean) / math.sqrt(var + 0.1) * wi + bi
            for v, wi, bi in zip([1.0, 2.0, 3.0, 6.0], w.tolist(), b.tolist())]
    got = plain.layer_norm(x, w, b, 0.1)[0].tolist()
    assert got == pytest.approx(want, rel=1e-12)


def test_frequency_bands():
    """One frequency in each band: kept, divided, and mixed between the two."""
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}
    f = plain.scaled_frequencies(8, 10000.0, sc).tolist()
    raw = [10000.0 ** (-2.0 * i / 8) for i in range(4)]
    waves = [2 * math.pi / r for r in raw]
    assert waves[0] < 64 / 4 < waves[1] < 64 / 1 < waves[2]      # bands: kept, mixed, divided
    assert f[0] == pytest.approx(raw[0], rel=1e-14)
    s = (64 / waves[1] - 1.0) / (4.0 - 1.0)
    assert f[1] == pytest.approx((1 - s) * raw[1] / 4 + s * raw[1], rel=1e-14)
    assert f[2] == pytest.approx(raw[2] / 4, rel=1e-14) and f[3] == pytest.approx(raw[3] / 4, rel=1e-14)
    assert plain.scaled_frequencies(8, 10000.0, None).tolist() == pytest.approx(raw, rel=1e-14)


def test_rotation_pairs_and_untouched_rest():
    x = torch.arange(1.0, 9.0, dtype=torch.float64).reshape(1, 1, 8)
    f = torch.tensor([0.5, 0.25], dtype=torch.float64)       # rotates 4 of the 8 elements
    y = plain.rotate(x, [3], f)[0, 0].tolist()
    for i, fi in enumerate([0.5, 0.25]):
        a = 3 * fi
        u, v = float(x[0, 0, i]), float(x[0, 0, i + 2])
        assert y[i] == pytest.approx(u * math.cos(a) - v * math.sin(a), rel=1e-13)
        assert y[i + 2] == pytest.approx(v * math.cos(a) + u * math.sin(a), rel=1e-13)
    assert y[4:] == [5.0, 6.0, 7.0, 8.0]


def test_sink_window_cap_by_hand():
    """Two heads on one kv head, three tokens, a window of two, scores capped."""
    q = torch.tensor([[[1.0, 0.0], [0.0, 2.0]]] * 3, dtype=torch.float64)
    k = torch.tensor([[[1.0, 1.0]], [[2.0, -1.0]], [[-1.0, 3.0]]], dtype=torch.float64)
    v = torch.tensor([[[1.0, 0.0]], [[0.0, 1.0]], [[2.0, 2.0]]], dtype=torch.float64)
    sink = torch.tensor([0.3, -0.7], dtype=torch.float64)
    out = plain.sink_softmax_attention(q, k, v, scale=0.5, cap=2.0, window=2, sink=sink)
    cap = lambda s: 2.0 * math.tanh(s / 2.0)                 # noqa: E731
    # head 1 at the last token sees keys 1 and 2 only
    s1, s2 = cap(0.5 * (2.0 * -1.0)), cap(0.5 * (2.0 * 3.0))
    e1, e2, es = math.exp(s1), math.exp(s2), math.exp(-0.7)
    want = [(e1 * 0.0 + e2 * 2.0) / (e1 + e2 + es), (e1 * 1.0 + e2 * 2.0) / (e1 + e2 + es)]
    assert out[2, 1].tolist() == pytest.approx(want, rel=1e-12)
    # head 0 at the first token sees itself and the sink
    s0 = cap(0.5 * 1.0)
    assert out[0, 0].tolist() == pytest.approx(
        [math.exp(s0) / (math.exp(s0) + math.exp(0.3)), 0.0], rel=1e-12)
    # without a window the last token also sees key 0
    full = plain.sink_softmax_attention(q, k, v, scale=0.5, cap=2.0, window=None, sink=sink)
    assert not torch.allclose(full[2], out[2]) and torch.allclose(full[:2], out[:2])


def test_relu_squared():
    h = torch.tensor([[1.0, -2.0]])
    up = torch.tensor([[1.0, 0.0], [0.0, 1.0], [2.0, 1.0]])     # -> [1, -2, 0]
    down = torch.tensor([[1.0, 1.0, 1.0], [3.0, 0.0, 0.0]])
    assert plain.relu_squared_ff(h, up, down).tolist() == [[1.0, 3.0]]


def test_layer_runs():
    assert plain.layer_runs(CONFIG) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert plain.layer_runs(dict(CONFIG, loop=None)) == [(i, None) for i in range(4)]


# ------------------------------------------------------------------ configuration and plan
def _cfg(raw):
    import grout_b200.architectures  # noqa: F401  (registers the designs)
    from grout_b200.config import resolve_architecture
    arch = resolve_architecture(raw)
    return arch, arch.config_cls.from_dict(raw)


def test_config_is_found_by_its_architecture_key_and_read_layer_by_layer():
    arch, cfg = _cfg(CONFIG)
    assert arch.name == "Suvazen" and cfg.passes() == 2
    assert cfg.layer_runs() == plain.layer_runs(CONFIG)
    plan = arch.plan(cfg)
    plan.validate()
    assert [(e.layer, e.add) for e in plan.schedule] == [
        (0, None), (1, ("loop.step", 0)), (2, None), (1, ("loop.step", 1)), (2, None), (3, None)]
    m0, m1, m2 = (plan.layers[i].block.args["mixer"].args for i in range(3))
    assert (m0["n_heads"], m0["n_kv_heads"], m0["head_dim"], m0["window"], m0["softcap"]) == (6, 3, 16, 5, 9.0)
    assert m1["n_heads"] == 3 and m1["window"] is None and m1["softcap"] is None
    assert m2["position"].kind == "none" and m0["position"].args["rot_dim"] == 8
    assert "feedforward" not in plan.layers[1].block.args


def test_expected_tensors_follow_the_layers():
    from grout_b200.engine.model import expected_tensors
    arch, cfg = _cfg(CONFIG)
    exp = expected_tensors(arch.plan(cfg))
    assert exp["l0.mix.q"].shape == (96, 24) and exp["l0.mix.k"].shape == (48, 24)
    assert exp["l1.mix.q"].shape == (48, 24) and exp["l2.mix.o"].shape == (24, 48)
    assert exp["l0.mix.sink"].shape == (6,) and exp["loop.step"].shape == (2, 24)
    assert exp["l2.mlp.up"].shape == (16, 24) and exp["l0.norm2b.b"].shape == (24,)
    assert "l1.mlp.up" not in exp and exp["l1.norm2"].optional      # a layer without feed-forward
    assert not any(n.endswith(".v") for n in exp)
    required = {n for n, s in exp.items() if not s.optional}
    assert {"embed", "head", "final.norm", "final.norm.b"} <= required


@pytest.mark.parametrize("change,word", [
    (dict(vocab=0), "vocab"),
    (dict(norm={}), "norm.eps"),
    (dict(loop={"start": 2, "stop": 9, "times": 2}), "loop"),
    (dict(loop={"start": 0, "stop": 1, "times": 0}), "times"),
    (dict(layers=[dict(type="recurrent", mixer=MIXER, mlp=None)]), "type"),
    (dict(layers=[dict(type="attention", mixer=dict(MIXER, heads=5), mlp=None)]), "share"),
    (dict(layers=[dict(type="attention", mixer=dict(MIXER, vdim=8), mlp=None)]), "vdim"),
    (dict(layers=[dict(type="attention", mixer=dict(MIXER, rot={"dims": 18, "base": 1e4}), mlp=None)]), "rot.dims"),
    (dict(layers=[dict(type="attention", mixer=MIXER, mlp={"kind": "routed", "ff": 8})]), "kind"),
    (dict(layers=[dict(type="attention", mixer=dict(MIXER, mask={"size": 0}), mlp=None)]), "mask"),
])
def test_config_problems_are_named(change, word):
    from grout_b200.config import ConfigError
    raw = dict(CONFIG, **change)
    if "layers" in change:
        raw["loop"] = None
    with pytest.raises(ConfigError) as e:
        _cfg(raw)
    assert word in str(e.value)


def test_absent_constants_mean_absent_terms():
    raw = dict(CONFIG)
    for k in ("loop", "logit_scale", "logit_softcap", "residual_mult"):
        raw.pop(k)
    arch, cfg = _cfg(raw)
    plan = arch.plan(cfg)
    assert plan.stream_vectors == () and all(e.add is None for e in plan.schedule)
    assert plan.head.args["scale"] is None and plan.head.args["softcap"] is None
    assert plan.layers[0].block.args["mult"] == 1.0


def test_random_weights_make_a_loadable_folder(tmp_path):
    from grout_b200.weights import Checkpoint, write_random_model
    d = write_random_model(CONFIG, 5, str(tmp_path / "m"))
    ck = Checkpoint(d)
    assert ck.entry("loop.step").shape == (2, 24) and ck.entry("l3.mix.sink").shape == (6,)
    # the plain implementation runs on them
    w = {n: ck.tensor(n) for n in ck.names()}
    out = plain.logits(w, CONFIG, [1, 2, 3, 4, 5, 6, 7])
    assert out.shape == (7, 50) and bool(torch.isfinite(out).all())
    assert float(out.abs().max()) <= 11.0
