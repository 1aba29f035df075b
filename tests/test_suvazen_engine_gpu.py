"""The Suvazen design through the engine against the plain implementation, in every
way of cutting the work, on three small models whose sizes and constants differ in
every respect (and from layer to layer).  The random weights are reshaped so that
faults show: query and key projections are scaled up until scores reach the bend
of the cap and attention is far from uniform, and the sinks are large enough to
take a real share of every denominator."""
import json
import os

import pytest
import torch

from conftest import random_tokens
from helpers import run_batch, run_chunks, run_schedule, run_tail_decoded, run_whole
from helpers import assert_close as assert_close_elementwise
from plain import suvazen as plain

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


ROW_BAR = 0.05


def assert_close(got, want, dtype, what=""):
    """32-bit: element by element at the library's 32-bit bar.  bfloat16: the
    sharpened models turn the rounding of a query or key into a visible change of a
    few attention weights, so single logits move by a tenth of the logits' spread
    while rows as a whole stay close; the bar is on rows, as a share of that spread:
    the root mean square over the vocabulary of a row's differences (their mean taken
    off, which no choice of token sees) against the root mean square of the logits."""
    if dtype == "float32":
        return assert_close_elementwise(got, want, dtype, what)
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    d = got - want
    d = d - d.mean(dim=-1, keepdim=True)
    spread = float((want - want.mean(dim=-1, keepdim=True)).pow(2).mean().sqrt())
    rows = d.pow(2).mean(dim=-1).sqrt() / spread
    worst = int(rows.argmax())
    assert float(rows.max()) <= ROW_BAR, (f"{what}: row {worst} differs by {float(rows.max()):.3f} of the "
                                          f"logits' spread; median row {float(rows.median()):.4f}")


def _mixer(**kw):
    m = dict(heads=4, kv_heads=2, dim=16, vdim=16, scale=0.3, softcap=4.0, mask={"size": 24},
             rot={"dims": 8, "base": 10000.0,
                  "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32}})
    m.update(kw)
    return {k: v for k, v in m.items() if v is not None}


def _layer(mlp, **kw):
    return dict(type="attention", mixer=_mixer(**kw), mlp=None if mlp is None else {"kind": "dense", "ff": mlp})


SUV = {
    # small heads whose rotation takes the plain q/k kernel; a loop in the middle
    "P": dict(architecture="Suvazen", vocab=211, width=64, norm={"eps": 1e-5}, residual_mult=0.5,
              logit_scale=0.7, logit_softcap=9.0, loop={"start": 1, "stop": 2, "times": 2},
              layers=[_layer(96), _layer(80), _layer(96)]),
    # every layer different; heads of 64 (the tensor-memory kernels), a window that crosses
    # a page, a layer without feed-forward, one without rotation, one without window or cap;
    # no loop, no residual factor, no logit constants
    "Q": dict(architecture="Suvazen", vocab=300, width=128, norm={"eps": 3e-6},
              layers=[_layer(160, heads=2, kv_heads=1, dim=64, vdim=64, scale=0.125, softcap=6.0,
                             mask={"size": 70}, rot={"dims": 32, "base": 50000.0}),
                      _layer(None, heads=6, kv_heads=3, dim=32, vdim=32, scale=0.2, softcap=None, mask=None,
                             rot={"dims": 32, "base": 300.0,
                                  "scaling": {"factor": 2.0, "low": 2.0, "high": 6.0, "original": 24}}),
                      _layer(200, heads=4, kv_heads=4, dim=64, vdim=64, scale=0.1, softcap=3.0,
                             mask={"size": 40}, rot=None)]),
    # heads of 128 in groups of two; the loop starts at the first layer and runs three times
    "R": dict(architecture="Suvazen", vocab=160, width=96, norm={"eps": 1e-6}, residual_mult=1.3,
              logit_scale=2.0, logit_softcap=30.0, loop={"start": 0, "stop": 2, "times": 3},
              layers=[_layer(128, heads=2, kv_heads=1, dim=128, vdim=128, scale=0.09, softcap=8.0,
                             mask={"size": 130},
                             rot={"dims": 64, "base": 1000.0,
                                  "scaling": {"factor": 2.5, "low": 2.0, "high": 8.0, "original": 64}})
                      for _ in range(3)]),
}
SEEDS = {"P": 11, "Q": 13, "R": 17}
LENGTHS = {"P": [1, 5, 70, 150], "Q": [2, 64, 129, 300], "R": [3, 131, 270]}


def _sharpen(tensors):
    """Scores that spread, sinks that count."""
    g = torch.Generator().manual_seed(1)
    out = {}
    for name, t in tensors:
        if name.endswith(".mix.q") or name.endswith(".mix.k"):
            t = (t.float() * 10.0).to(t.dtype)
        elif name.endswith(".mix.sink"):
            t = (1.5 + 1.5 * torch.randn(t.shape, generator=g)).to(t.dtype)
        elif name == "embed":
            t = (t.float() * 20.0).to(t.dtype)
        elif name == "loop.step":
            t = (t.float() * 4.0).to(t.dtype)
        out[name] = t
    return out


@pytest.fixture(scope="module")
def suv_models(tmp_path_factory):
    """name -> (folder, config dict, {tensor name: CPU tensor})."""
    import grout_b200.architectures  # noqa: F401
    from grout_b200.config import resolve_architecture
    from grout_b200.engine.model import expected_tensors
    from grout_b200.weights import random_tensors, write_safetensors
    base = tmp_path_factory.mktemp("suvazen")
    out = {}
    for name, cfg in SUV.items():
        arch = resolve_architecture(cfg)
        exp = expected_tensors(arch.plan(arch.config_cls.from_dict(cfg)))
        exp = {n: s for n, s in exp.items() if not s.optional}
        w = _sharpen(random_tensors(exp, SEEDS[name]))
        folder = str(base / name)
        os.makedirs(folder)
        with open(os.path.join(folder, "config.json"), "w") as fh:
            json.dump(cfg, fh)
        write_safetensors(os.path.join(folder, "model.safetensors"), list(w.items()))
        out[name] = (folder, cfg, w)
    return out


@pytest.fixture(scope="module")
def engines(suv_models):
    from grout_b200.engine import Engine
    made = {}

    def get(name, dtype, **kw):
        key = (name, dtype, tuple(sorted(kw.items())))
        if key not in made:
            made[key] = Engine.load(suv_models[name][0], dtype=dtype, max_tokens=4096, max_batch=8,
                                    max_seq_len=512, **kw)
        return made[key]
    return get


@pytest.fixture(scope="module")
def oracle(suv_models):
    memo = {}

    def get(name, tokens):
        key = (name, tuple(tokens))
        if key not in memo:
            _d, cfg, w = suv_models[name]
            memo[key] = plain.logits(w, cfg, list(tokens))
        return memo[key]
    return get


def test_the_sharpened_weights_do_what_they_are_for(suv_models):
    """Scores reach the cap's bend, attention is far from uniform, and a sink takes
    a real share: a model on which a lost cap, sink, rotation or window shows."""
    _d, cfg, w = suv_models["P"]
    toks = random_tokens(60, cfg["vocab"], 1)
    full = plain.logits(w, cfg, toks)

    def changed(**kw):
        c = json.loads(json.dumps(cfg))
        for layer in c["layers"]:
            layer["mixer"].update(kw)
            for k, v in kw.items():
                if v is None:
                    layer["mixer"].pop(k)
        return float((plain.logits(w, c, toks) - full).abs().max())

    assert changed(softcap=None) > 0.05
    assert changed(mask={"size": 23}) > 0.05 and changed(mask={"size": 25}) > 0.05
    assert changed(rot=None) > 0.05
    no_sink = {k: (v - 40.0 if k.endswith(".sink") else v) for k, v in w.items()}
    assert float((plain.logits(no_sink, cfg, toks) - full).abs().max()) > 0.05
    no_loop = dict(cfg, loop=None)
    assert float((plain.logits(w, no_loop, toks) - full).abs().max()) > 0.05


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(SUV))
def test_each_request_alone_and_whole(engines, oracle, name, dtype):
    eng = engines(name, dtype)
    for i, n in enumerate(LENGTHS[name]):
        toks = random_tokens(n, SUV[name]["vocab"], 100 + i)
        assert_close(run_whole(eng, toks), oracle(name, toks), dtype, f"{name} whole, {n} tokens")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and eng.cache.tokens_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(SUV))
def test_prefill_against_token_by_token(engines, oracle, name, dtype):
    """The tail decoded one token at a time, long enough for every window to pass
    over decoded tokens only; and a whole request decoded from its first token."""
    eng = engines(name, dtype)
    window = max((l["mixer"].get("mask") or {"size": 0})["size"] for l in SUV[name]["layers"])
    n = LENGTHS[name][-1]
    toks = random_tokens(n, SUV[name]["vocab"], 200)
    want = oracle(name, toks)
    assert_close(run_tail_decoded(eng, toks, tail=min(n - 1, window + 10)), want, dtype, f"{name} tail")
    short = toks[:90]
    got = run_tail_decoded(eng, short, tail=89)
    assert_close(got, oracle(name, short), dtype, f"{name} decoded from the first token")
    if dtype == "float32":
        assert (got - run_whole(eng, short)).abs().max().item() < 2e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(SUV))
def test_a_prompt_fed_in_portions(engines, oracle, name, dtype):
    """Portions of two tokens; portions that end one short of a page, on it and
    beyond it; portions around each window's size."""
    eng = engines(name, dtype)
    for i, chunks in enumerate([[2] * 12 + [1, 3], [63, 1, 64, 2], [60, 10, 70], [23, 2, 24, 25, 41, 2, 39, 40, 2]]):
        toks = random_tokens(sum(chunks), SUV[name]["vocab"], 700 + i)
        got = run_chunks(eng, toks, chunks)
        assert_close(got, oracle(name, toks), dtype, f"{name} portions {chunks}")
        if dtype == "float32":
            assert (got - run_whole(eng, toks)).abs().max().item() < 2e-5, chunks
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(SUV))
def test_unequal_batches_one_after_another(engines, oracle, name, dtype):
    """Three batches in a row on one engine: slots and pages of an earlier batch are
    used again by a later one (also the pages that a window gave back), and within
    a batch the shorter requests end earlier."""
    eng = engines(name, dtype)
    V = SUV[name]["vocab"]
    plans = [[(5, 3), (11, 9), (17, 1)],
             [(1, 20), (7, 2), (30, 11), (64, 5), (130, 33), (200, 80)],
             [(65, 4), (2, 4), (128, 70)]]
    for b, plan in enumerate(plans):
        reqs = [random_tokens(p + d, V, 300 + 10 * b + i) for i, (p, d) in enumerate(plan)]
        got = run_batch(eng, reqs, [p for p, _ in plan])
        for i, r in enumerate(reqs):
            assert_close(got[i], oracle(name, r), dtype, f"{name} batch {b} request {i}")
            if dtype == "float32":
                assert (got[i] - run_whole(eng, r)).abs().max().item() < 2e-5, (b, i)
        eng.cache.check()
        assert eng.cache.slots.n_held == 0 and eng.cache.tokens_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_first_tokens_and_long_decoding(engines, oracle, name, dtype):
    """A prompt of one token and 200 decoded ones: the first positions of a
    sequence (a window that is not full yet, a sink beside a single key) and a long
    run of single steps across page boundaries while windows give pages back."""
    eng = engines(name, dtype)
    toks = random_tokens(201, SUV[name]["vocab"], 400)
    assert_close(run_tail_decoded(eng, toks, tail=200), oracle(name, toks), dtype, "long decoding")
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(SUV))
def test_steps_that_mix_one_and_many_tokens(engines, oracle, name, dtype):
    eng = engines(name, dtype)
    lengths = [20 + 5 + 1 + 3 + 1, 9 + 1 + 1 + 1 + 1 + 1, 70 + 1 + 2]
    schedule = [{0: 20, 1: 9}, {0: 5, 1: 1}, {0: 1, 1: 1, 2: 70}, {0: 3, 1: 1, 2: 1},
                {0: 1, 1: 1, 2: 2}, {1: 1}]
    reqs = [random_tokens(n, SUV[name]["vocab"], 720 + i) for i, n in enumerate(lengths)]
    got = run_schedule(eng, reqs, schedule)
    for i, r in enumerate(reqs):
        assert_close(got[i], oracle(name, r), dtype, f"{name} mixed steps, request {i}")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_captured_steps_against_steps_launched_one_by_one(engines, oracle, dtype):
    """Bit-equal in 32-bit; both within the plain implementation's bar in bfloat16."""
    reqs = [random_tokens(n, SUV["Q"]["vocab"], 740 + i) for i, n in enumerate((90, 33, 140))]
    outs = {}
    for use in (True, False):
        eng = engines("Q", dtype, use_graphs=use)
        outs[use] = run_batch(eng, reqs, [60, 30, 100])
    for i, r in enumerate(reqs):
        assert_close(outs[True][i], oracle("Q", r), dtype, f"captured, request {i}")
        assert_close(outs[False][i], oracle("Q", r), dtype, f"launched, request {i}")
        if dtype == "float32":
            assert torch.equal(outs[True][i], outs[False][i])


def test_the_product_kernels_of_choice(suv_models, oracle):
    """Every way of running the products (pair, single-SM tcgen05, library for a
    prompt; tcgen05 or mma.sync for a decode step) gives the same model."""
    from grout_b200.engine import Engine
    from grout_b200.parts import ProductChoice
    toks = random_tokens(200, SUV["Q"]["vocab"], 760)
    for choice in (ProductChoice("tc", "pair"), ProductChoice("tc", "tc"), ProductChoice("skinny", "library")):
        eng = Engine.load(suv_models["Q"][0], dtype="bfloat16", max_tokens=1024, max_batch=2,
                          max_seq_len=512, products=choice)
        assert_close(run_tail_decoded(eng, toks, tail=20), oracle("Q", toks), "bfloat16", str(choice))


@pytest.mark.parametrize("name", sorted(SUV))
def test_greedy_generation_through_the_engine(suv_models, name):
    """Engine.generate (its scheduler, cache and device sampler) against the plain
    loop, in 32-bit, where the argmax is the same token."""
    from grout_b200.engine import Engine
    folder, cfg, w = suv_models[name]
    eng = Engine.load(folder, dtype="float32", max_tokens=2048, max_batch=3)
    prompts = [random_tokens(n, cfg["vocab"], 800 + i) for i, n in enumerate((1, 7, 30, 64, 5))]
    want = [plain.greedy_generate(w, cfg, p, 12) for p in prompts]
    outs = eng.generate(prompts, 12, ignore_eos=True)          # five requests on three slots
    assert [o.token_ids for o in outs] == want
    stop = want[1][3]
    outs = eng.generate(prompts, 12, stop_ids=[stop])
    assert [o.token_ids for o in outs] == [plain.greedy_generate(w, cfg, p, 12, stop_ids=(stop,))
                                           for p in prompts]
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and eng.cache.tokens_held() == 0


def test_generation_in_bfloat16_and_the_command_line(suv_models, tmp_path):
    """bfloat16 generation runs through captured steps with the tensor-core
    attention; its tokens are the plain loop's wherever the plain logits leave no
    doubt.  And the command line serves the design as it serves the others."""
    import subprocess
    import sys
    from conftest import ROOT
    from grout_b200.engine import Engine
    folder, cfg, w = suv_models["Q"]
    eng = Engine.load(folder, dtype="bfloat16", max_tokens=2048, max_batch=4)
    prompt = random_tokens(70, cfg["vocab"], 820)
    got = eng.generate([prompt], 10, ignore_eos=True)[0].token_ids
    seq = list(prompt)
    for tok in got:
        row = plain.logits(w, cfg, seq, rows=[len(seq) - 1])[0]
        top2 = torch.topk(row, 2).values
        if float(top2[0] - top2[1]) > 0.1:
            assert tok == int(torch.argmax(row)), len(seq)
        seq.append(tok)
    out = tmp_path / "out.json"
    ids = ",".join(str(t) for t in prompt[:9])
    r = subprocess.run([sys.executable, "-m", "grout_b200", "--model", folder, "--prompt-ids", ids,
                        "--max-new-tokens", "6", "--ignore-eos", "--fp32", "--device-argmax",
                        "--output-json", str(out), "--quiet"], cwd=ROOT, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.load(open(out))["token_ids"] == plain.greedy_generate(w, cfg, prompt[:9], 6)


def test_trace_replay_serves_the_design(suv_models, tmp_path):
    """bin/trace_run on a Suvazen folder: a prompt, then single tokens, two requests."""
    import subprocess
    import sys
    import numpy as np
    from conftest import ROOT
    folder, cfg, w = suv_models["P"]
    a, b = random_tokens(40, cfg["vocab"], 840), random_tokens(9, cfg["vocab"], 841)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:37], "want": [0, 36]},
                                     {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[37]], "want": []},
                                     {"id": "b", "tokens": [b[8]], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[38]], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": [a[39]], "want": [0]}], "end": ["a"]}]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                        "--dtype", "float32", "--out", str(tmp_path), "--max-tokens", "128"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    la, lb = plain.logits(w, cfg, a), plain.logits(w, cfg, b)
    want = {0: torch.stack([la[0], la[36], lb[7]]), 1: lb[8:9], 2: la[38:39], 3: la[39:40]}
    for i, wnt in want.items():
        got = torch.from_numpy(np.fromfile(tmp_path / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
        assert_close(got, wnt, "float32", f"step {i}")
