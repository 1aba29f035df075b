"""Suvazen models of awkward sizes through the engine against the plain
implementation: widths and head sizes that no fast kernel takes, groups of three
and of one and of many, windows of one token and of exactly a page, a vocabulary
that is no multiple of anything, every optional constant absent, a loop over all
layers and a loop of one pass.  Each runs whole, decoded, in portions and in an
unequal batch, in both precisions."""
import json
import os

import pytest
import torch

from conftest import random_tokens
from helpers import run_batch, run_chunks, run_tail_decoded, run_whole
from plain import suvazen as plain
from test_suvazen_engine_gpu import _sharpen, assert_close

pytestmark = pytest.mark.gpu


def _mix(heads, kv, dim, scale, **kw):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, scale=scale)
    m.update(kw)
    return m


def _lay(mixer, ff):
    return dict(type="attention", mixer=mixer, mlp=None if ff is None else {"kind": "dense", "ff": ff})


ODD = {
    # a width of 100 (no 16-byte rows for the tensor-core products), heads of 24 in groups of three,
    # a rotation of six elements, a window of one token in one layer and of a whole page in another
    "w100": dict(architecture="Suvazen", vocab=77, width=100, norm={"eps": 1e-4}, residual_mult=0.9,
                 logit_softcap=5.0,
                 layers=[_lay(_mix(6, 2, 24, 0.2, softcap=3.0, mask={"size": 1}, rot={"dims": 6, "base": 100.0}), 52),
                         _lay(_mix(3, 3, 24, 0.2, mask={"size": 64},
                                   rot={"dims": 24, "base": 9000.0,
                                        "scaling": {"factor": 16.0, "low": 0.5, "high": 3.0, "original": 16}}), 36),
                         _lay(_mix(1, 1, 40, 0.15, softcap=2.0, mask={"size": 65}), None)]),
    # nothing optional: no cap, no window, no rotation, no loop, no factor, no logit constants
    "bare": dict(architecture="Suvazen", vocab=130, width=48, norm={"eps": 1e-5},
                 layers=[_lay(_mix(2, 1, 32, 0.17), 64), _lay(_mix(4, 4, 16, 0.25), 24)]),
    # groups of 32 query heads on one kv head (beyond the decode kernels' groups), heads of 96
    # (tensor-core attention, no 16-byte-piece rotation), the loop over every layer, three passes
    "wide_groups": dict(architecture="Suvazen", vocab=201, width=64, norm={"eps": 1e-6}, residual_mult=0.4,
                        logit_scale=3.0, loop={"start": 0, "stop": 2, "times": 3},
                        layers=[_lay(_mix(32, 1, 16, 0.25, softcap=5.0, mask={"size": 33},
                                          rot={"dims": 16, "base": 500.0}), 40),
                                _lay(_mix(2, 2, 96, 0.1, softcap=9.0, mask={"size": 100},
                                          rot={"dims": 48, "base": 20000.0}), 72)]),
    # a loop of a single pass at the end (its vector is still added), heads of 256, a long window
    "one_pass": dict(architecture="Suvazen", vocab=99, width=72, norm={"eps": 1e-5}, residual_mult=1.0,
                     logit_scale=1.0, logit_softcap=50.0, loop={"start": 1, "stop": 2, "times": 1},
                     layers=[_lay(_mix(2, 1, 64, 0.125, softcap=4.0, mask={"size": 300},
                                       rot={"dims": 64, "base": 1e6}), 100),
                             _lay(_mix(1, 1, 256, 0.06, softcap=6.0, mask={"size": 7},
                                       rot={"dims": 128, "base": 1e4}), 40)]),
}


@pytest.fixture(scope="module")
def odd_models(tmp_path_factory):
    import grout_b200.architectures  # noqa: F401
    from grout_b200.config import resolve_architecture
    from grout_b200.engine.model import expected_tensors
    from grout_b200.weights import random_tensors, write_safetensors
    base = tmp_path_factory.mktemp("suvazen_odd")
    out = {}
    for k, (name, cfg) in enumerate(ODD.items()):
        arch = resolve_architecture(cfg)
        exp = {n: s for n, s in expected_tensors(arch.plan(arch.config_cls.from_dict(cfg))).items()
               if not s.optional}
        w = _sharpen(random_tensors(exp, 40 + k))
        folder = str(base / name)
        os.makedirs(folder)
        with open(os.path.join(folder, "config.json"), "w") as fh:
            json.dump(cfg, fh)
        write_safetensors(os.path.join(folder, "model.safetensors"), list(w.items()))
        out[name] = (folder, cfg, w)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ODD))
def test_odd_sizes_in_every_cut(odd_models, name, dtype):
    from grout_b200.engine import Engine
    folder, cfg, w = odd_models[name]
    eng = Engine.load(folder, dtype=dtype, max_tokens=2048, max_batch=6, max_seq_len=512)
    V = cfg["vocab"]
    a, b, c = (random_tokens(n, V, 900 + n) for n in (140, 67, 9))
    want = {n: plain.logits(w, cfg, t) for n, t in (("a", a), ("b", b), ("c", c))}
    assert_close(run_whole(eng, a), want["a"], dtype, f"{name} whole")
    assert_close(run_tail_decoded(eng, a, tail=72), want["a"], dtype, f"{name} tail decoded")
    assert_close(run_chunks(eng, a, [2, 62, 1, 64, 2, 9]), want["a"], dtype, f"{name} portions")
    got = run_batch(eng, [a, b, c], [130, 40, 1])
    for g, n in zip(got, "abc"):
        assert_close(g, want[n], dtype, f"{name} batch, request {n}")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and eng.cache.tokens_held() == 0
    eng.check()


def test_a_checkpoint_with_the_norms_of_an_absent_feed_forward_loads(odd_models, tmp_path):
    """A writer that made norm2 / norm2b for a layer without feed-forward: the tensors are
    read by nothing and the model is the same."""
    from grout_b200.engine import Engine
    from grout_b200.weights import write_safetensors
    folder, cfg, w = odd_models["w100"]
    extra = dict(w)
    for n in ("l2.norm2", "l2.norm2.b", "l2.norm2b", "l2.norm2b.b"):
        extra[n] = torch.ones(cfg["width"], dtype=torch.bfloat16)
    d = str(tmp_path / "m")
    os.makedirs(d)
    with open(os.path.join(d, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    write_safetensors(os.path.join(d, "model.safetensors"), list(extra.items()))
    eng = Engine.load(d, dtype="float32", max_tokens=256, max_batch=2)
    toks = random_tokens(30, cfg["vocab"], 950)
    assert_close(run_whole(eng, toks), plain.logits(w, cfg, toks), "float32", "extra norms")
