"""Each mechanism that the Sonalorn design brought, alone, against the plain
implementation's function for it: the stream's sum through an output norm and a
per-channel scale, the embedding with learned positions, the gated delta rule
(state carried over steps, slots used again, planted far keys), the routed
feed-forward (choice by groups with corrected scores, pass-through experts,
clamps), attention with values of another size, a query temperature and a sink of
logit zero."""
import math

import pytest
import torch

from plain import sonalorn as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: dict(atol=3e-5, rtol=3e-4), torch.bfloat16: dict(atol=0.03, rtol=0.03)}


def close(got, want, dtype, what=""):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    err = (got - want).abs()
    bound = TOL[dtype]["atol"] + TOL[dtype]["rtol"] * want.abs()
    assert bool((err <= bound).all()), f"{what}: max err {err.max().item():.3g} at {int(err.argmax())}"


def rnd(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


class Step:
    """The fields of a step that the kernels read, for sequences given as (slot, start, n)."""

    def __init__(self, seqs):
        from grout_b200.engine.batch import make_context
        self.ctx = make_context([(s, st, [0] * n) for s, st, n in seqs], None, DEV)


# ------------------------------------------------------------------ the stream's sum
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N", [24, 320, 1000, 5120])
def test_stream_sum_through_norm_and_scale(dtype, N):
    from grout_b200.kernels import ops
    T = 7
    res, d = rnd(T, N, seed=1, scale=3.0), rnd(T, N, seed=2, scale=0.2).to(dtype)
    pw, sc, w = 1 + rnd(N, seed=3, scale=0.2), rnd(N, seed=4), 1 + rnd(N, seed=5, scale=0.2)
    c = plain.rms_norm(d, pw, 1e-5) * sc.double()
    want_res = res.double() + c
    g = lambda t: t.to(DEV)
    r, y = ops.add_postnorm(g(res).clone(), g(d), dtype=dtype, post_weight=g(pw), post_eps=1e-5, scale=g(sc))
    close(r, want_res, torch.float32, "stream")
    close(y, want_res, dtype, "the stream as the next sublayer reads it")
    rows = torch.tensor([5, 0, 5], dtype=torch.int32)
    r2, y2 = ops.add_postnorm(g(res).clone(), g(d), dtype=dtype, post_weight=g(pw), post_eps=1e-5,
                              scale=g(sc), weight=g(w), eps=1e-6, rows=g(rows))
    close(r2, want_res[rows.long()], torch.float32, "gathered rows")
    close(y2, plain.rms_norm(want_res[rows.long()], w, 1e-6), dtype, "final norm of gathered rows")
    parts = torch.stack([d.float() * 0.25, d.float() * 0.5, d.float() * 0.25]).contiguous()
    r3, _ = ops.add_postnorm(g(res).clone(), g(parts), dtype=dtype, post_weight=g(pw), post_eps=1e-5, scale=g(sc))
    close(r3, want_res, torch.float32, "partial sums")
    r4, y4 = ops.add_postnorm(g(res).clone(), None, dtype=dtype)
    assert torch.equal(r4.cpu(), res) and torch.equal(y4.cpu(), res.to(dtype))
    r5, _ = ops.add_postnorm(None, g(d), dtype=dtype)                 # nothing but the delta
    close(r5, d.double(), torch.float32, "delta alone")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_with_positions(dtype):
    from grout_b200.kernels import ops
    V, P, H = 37, 50, 72
    table, pos, w = rnd(V, H, seed=1).to(dtype), rnd(P, H, seed=2).to(dtype), 1 + rnd(H, seed=3, scale=0.1)
    ids = torch.tensor([3, 36, 0, 3], dtype=torch.int32)
    tp = torch.tensor([0, 49, 7, 8], dtype=torch.int32)
    got = ops.embed_pos_norm(table.to(DEV), pos.to(DEV), ids.to(DEV), tp.to(DEV), w.to(DEV), 1e-5)
    x = table.double()[ids.long()] + pos.double()[tp.long()]
    close(got, plain.rms_norm(x, w, 1e-5), torch.float32)            # 32-bit whatever the tables' type


def test_gelu_tanh_gate():
    from grout_b200.kernels import ops
    gu = rnd(5, 2 * 24, seed=1, scale=2.0)
    got = ops.gelu_tanh_mul(gu.to(DEV), 0)
    close(got, plain.gelu_tanh(gu[:, :24].double()) * gu[:, 24:].double(), torch.float32)


@pytest.mark.parametrize("rows", [3, 64, 300])
def test_gelu_tanh_gate_as_the_products_epilogue(rows):
    """The gated feed-forward part in bfloat16: a decode step's product and a prompt's
    apply the gate's activation before they store (gate and up rows interleaved in eights);
    all product choices give the plain result."""
    from grout_b200.parts import BuildContext, PartSpec, ProductChoice, build_part
    W, F = 64, 96
    w = {"gate": rnd(F, W, seed=1, scale=0.3).bfloat16(), "up": rnd(F, W, seed=2, scale=0.3).bfloat16(),
         "down": rnd(W, F, seed=3, scale=0.2).bfloat16()}
    x = rnd(rows, W, seed=4).bfloat16()
    want = plain.dense_ff(x, {"m." + k: v for k, v in w.items()}, "m.")
    for choice in (ProductChoice("tc", "auto"), ProductChoice("tc", "pair"), ProductChoice("skinny", "library")):
        part = build_part("feedforward", PartSpec("gated_mlp", dict(
            hidden=W, intermediate=F, activation="gelu_tanh", names={"gate": "gate", "up": "up", "down": "down"})),
            BuildContext(torch.bfloat16, torch.device(DEV), choice))
        part.load({k: v.to(DEV) for k, v in w.items()})
        assert part.interleave == 8
        got = part.forward(x.to(DEV), None)
        got = (got.sum(0) if got.dim() == 3 else got).double().cpu()
        # the unfused path rounds gate and up before the activation: a bar on the whole
        assert float((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt()) < 0.02, (rows, choice)


# ------------------------------------------------------------------ the gated delta rule
def _delta_weights(H, G, dk, dv, taps, W, seed, slow=True):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, sc=1.0: torch.randn(*s, generator=g) * sc
    w = {"q": r(G * dk, W, sc=0.3), "k": r(G * dk, W, sc=0.3), "v": r(H * dv, W, sc=0.3),
         "g": r(H * dv, W, sc=0.3), "b": r(H, W, sc=0.3), "a": r(H, W, sc=0.3),
         "q.conv": r(G * dk, taps, sc=0.6), "k.conv": r(G * dk, taps, sc=0.6), "v.conv": r(H * dv, taps, sc=0.6),
         # decays from "forgets at once" to "keeps for hundreds of tokens"
         "A_log": torch.linspace(-6.0 if slow else -1.0, 0.5, H), "dt_bias": r(H, sc=0.5),
         "norm": 1 + r(dv, sc=0.2), "o": r(W, H * dv, sc=0.2)}
    return w


def _delta_run(w, m, xs, cuts, dtype, state=None, slot=0, n_slots=3):
    """Feeds rows xs [T, W] through the kernels in steps of the given sizes."""
    from grout_b200.kernels import ops
    H, G, dk, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    g = lambda t: t.float().to(DEV).contiguous()
    wp = torch.cat([w[k] for k in ("q", "k", "v", "g", "b", "a")], 0).double()
    conv = g(torch.cat([w["q.conv"], w["k.conv"], w["v.conv"]], 0))
    if state is None:
        state = torch.zeros(n_slots + 1, ops.delta_state_floats(H, G, dk, dv, taps), device=DEV)
    outs, start = [], 0
    for n in cuts:
        step = Step([(slot, start, n)]).ctx
        proj = g(xs[start:start + n].double() @ wp.T)
        y = ops.delta_forward(proj, state, conv, g(w["A_log"]), g(w["dt_bias"]), g(w["norm"]), H=H, G=G,
                              dk=dk, dv=dv, taps=taps, unit_eps=1e-6, norm_eps=1e-5,
                              token_seq=step.token_seq, cu_q=step.cu_q, slots=step.slots, dtype=dtype)
        outs.append(y.float().cpu())
        start += n
    return torch.cat(outs), state


def _delta_plain(w, m, xs):
    W = dict({"m." + k: v for k, v in w.items()})
    W["m.o"] = torch.eye(m["heads"] * m["vdim"])          # the read-out before the o projection
    return plain.delta_mixer(xs, W, "m.", m, 1e-5)


DELTA_SHAPES = [dict(heads=4, kv_heads=2, dim=16, vdim=8, conv=3),
                dict(heads=3, kv_heads=3, dim=40, vdim=20, conv=4),     # sizes that fill no lane group
                dict(heads=2, kv_heads=1, dim=64, vdim=48, conv=2),
                dict(heads=2, kv_heads=2, dim=128, vdim=16, conv=1),    # no convolution to speak of
                dict(heads=2, kv_heads=1, dim=30, vdim=10, conv=5)]     # sizes that are no multiple of four


@pytest.mark.parametrize("m", DELTA_SHAPES)
def test_delta_rule_whole_in_portions_and_token_by_token(m):
    W, T = 24, 150
    w = _delta_weights(m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], W, seed=3)
    xs = rnd(T, W, seed=4)
    want = _delta_plain(w, m, xs)
    whole, _ = _delta_run(w, m, xs, [T], torch.float32)
    close(whole, want, torch.float32, "whole")
    for cuts in ([2] * 75, [1] * T, [1, 2, 3, 100, 44], [149, 1]):
        got, _ = _delta_run(w, m, xs, cuts, torch.float32)
        # the same recurrence however the rows are cut (rows are walked in groups that
        # start where a step starts, so the rounding differs)
        assert float((got - whole).abs().max()) < 1e-5, cuts
    half, _ = _delta_run(w, m, xs, [T], torch.bfloat16)
    close(half, want, torch.bfloat16, "bfloat16 output")


def test_delta_rule_batches_slots_used_again_and_padding():
    from grout_b200.kernels import ops
    m = DELTA_SHAPES[0]
    H, G, dk, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    W = 24
    w = _delta_weights(H, G, dk, dv, taps, W, seed=5)
    xa, xb = rnd(40, W, seed=6), rnd(9, W, seed=7)
    alone_a, _ = _delta_run(w, m, xa, [40], torch.float32)
    alone_b, _ = _delta_run(w, m, xb, [9], torch.float32)
    g = lambda t: t.float().to(DEV).contiguous()
    wp = torch.cat([w[k] for k in ("q", "k", "v", "g", "b", "a")], 0).double()
    conv = g(torch.cat([w["q.conv"], w["k.conv"], w["v.conv"]], 0))
    state = torch.zeros(4, ops.delta_state_floats(H, G, dk, dv, taps), device=DEV)
    state[1].fill_(7.0)                                               # a slot that someone left dirty ...
    state[1].zero_()                                                  # ... is zeroed when it is opened
    args = dict(H=H, G=G, dk=dk, dv=dv, taps=taps, unit_eps=1e-6, norm_eps=1e-5, dtype=torch.float32)
    run = lambda step, rows: ops.delta_forward(g(rows.double() @ wp.T), state, conv, g(w["A_log"]), g(w["dt_bias"]),
                                               g(w["norm"]), token_seq=step.token_seq, cu_q=step.cu_q,
                                               slots=step.slots, **args).cpu()
    # a in slot 2 and b in slot 1 start together with a padding sequence between them
    s1 = Step([(2, 0, 30), (-1, 0, 3), (1, 0, 8)]).ctx
    y = run(s1, torch.cat([xa[:30], rnd(3, W, seed=8), xb[:8]]))
    same = lambda p, q: float((p - q).abs().max()) < 1e-5
    assert same(y[:30], alone_a[:30]) and same(y[33:], alone_b[:8])
    assert float(state[3].abs().max()) == 0.0                         # padding rows store nothing
    s2 = Step([(1, 8, 1), (2, 30, 1)]).ctx                            # then decoded together, other order
    y = run(s2, torch.cat([xb[8:9], xa[30:31]]))
    assert same(y[0], alone_b[8]) and same(y[1], alone_a[30])
    state[1].zero_()                                                  # b ends; its slot serves a new request
    s3 = Step([(2, 31, 9), (1, 0, 9)]).ctx
    y = run(s3, torch.cat([xa[31:], xb]))
    assert same(y[:9], alone_a[31:]) and same(y[9:], alone_b)


def test_delta_rule_reads_a_far_key():
    """One head keeps what it wrote 400 tokens ago (slow decay): the planted value
    comes back when its key is asked for, and does not with a fast decay."""
    m = dict(heads=1, kv_heads=1, dim=16, vdim=8, conv=1)
    W = 32
    w = _delta_weights(1, 1, 16, 8, 1, W, seed=9)
    for k in ("q.conv", "k.conv", "v.conv"):
        w[k] = torch.ones_like(w[k])
    w["q"], w["k"] = torch.eye(16, W) * 4, torch.eye(16, W) * 4
    w["v"] = torch.zeros(8, W)
    w["v"][:, 16:24] = torch.eye(8) * 4
    w["b"] = torch.full((1, W), 0.0)
    w["b"][0, 31] = 8.0                                               # beta near one where channel 31 is set
    w["a"], w["dt_bias"] = torch.zeros(1, W), torch.zeros(1)
    xs = torch.zeros(402, W)
    xs[:, 3] = 0.3                                                    # every token asks for "key 3" a little
    xs[0, 5], xs[0, 16:24], xs[0, 31] = 5.0, torch.arange(1.0, 9.0), 1.0   # the planted pair: key 5 -> value
    xs[401, 5] = 5.0                                                  # the last token asks for key 5
    for a_log, keeps in ((-9.0, True), (0.0, False)):
        w["A_log"] = torch.tensor([a_log])
        got, _ = _delta_run(w, m, xs, [300, 101, 1], torch.float32)
        close(got, _delta_plain(w, m, xs), torch.float32, f"A_log {a_log}")
        w2 = dict(w)
        x2 = xs.clone()
        x2[0, 16:24] = 0.0
        other, _ = _delta_run(w2, m, x2, [402], torch.float32)
        moved = float((got[401] - other[401]).abs().max())
        assert (moved > 0.1) == keeps, (a_log, moved)


# ------------------------------------------------------------------ routed experts
def _moe_weights(E, ident, F, W, seed, router_scale=3.0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, sc=1.0: torch.randn(*s, generator=g) * sc
    w = {"router": r(E + ident, W, sc=router_scale / math.sqrt(W)), "correction": r(E + ident, sc=0.15) - 0.1}
    for j in range(E):
        w[f"e{j}.gate"], w[f"e{j}.up"] = r(F, W, sc=2.0 / math.sqrt(W)), r(F, W, sc=2.0 / math.sqrt(W))
        w[f"e{j}.down"] = r(W, F, sc=1.0 / math.sqrt(F))
    return w


def _moe_run(w, mlp, x, dtype):
    from grout_b200.kernels import ops
    r = mlp["router"]
    E = r["experts"]
    st = lambda what: torch.stack([w[f"e{j}.{what}"] for j in range(E)]).to(dtype).to(DEV).contiguous()
    g = r.get("groups") or {"count": 1, "keep": 1}
    return ops.moe_forward(x.to(dtype).to(DEV), w["router"].float().to(DEV), w["correction"].float().to(DEV),
                           st("gate"), st("up"), st("down"), top=r["top"], n_identity=r.get("identity", 0),
                           n_groups=g["count"], keep_groups=g["keep"], limit=mlp["expert"]["limit"],
                           slope=1.702, want_choice=True)


MOES = [{"kind": "moe", "expert": {"ff": 24, "limit": 0.8},
         "router": {"experts": 6, "identity": 2, "top": 3, "groups": {"count": 4, "keep": 2}}},
        {"kind": "moe", "expert": {"ff": 50, "limit": 2.5},
         "router": {"experts": 9, "identity": 0, "top": 1, "groups": {"count": 3, "keep": 1}}},
        {"kind": "moe", "expert": {"ff": 17, "limit": 0.3},
         "router": {"experts": 5, "identity": 1, "top": 4}},                       # no groups
        {"kind": "moe", "expert": {"ff": 64, "limit": 1.0},
         "router": {"experts": 30, "identity": 2, "top": 2, "groups": {"count": 8, "keep": 3}}}]


@pytest.mark.parametrize("mlp", MOES)
def test_routed_experts_choice_and_output(mlp):
    W, T = 40, 70
    r = mlp["router"]
    w = _moe_weights(r["experts"], r.get("identity", 0), mlp["expert"]["ff"], W, seed=11)
    x = rnd(T, W, seed=12)
    out, ids, wts = _moe_run(w, mlp, x, torch.float32)
    chosen, weights = plain.route(x, w["router"], w["correction"], r)
    assert torch.equal(ids.cpu().long(), chosen)
    close(wts, weights, torch.float32, "weights are the uncorrected scores")
    want = plain.routed_ff(x, {"m." + k: v for k, v in w.items()}, "m.", mlp)
    close(out.sum(0), want, torch.float32, "output")
    # what the test is for: corrected scores below zero, clamps that bite, pass-through experts chosen
    c = torch.softmax(x.double() @ w["router"].double().T, -1) + w["correction"].double()
    if r["top"] >= 3:
        assert bool((c.gather(1, chosen) < 0).any())
    if r.get("identity", 0) * 8 >= w["router"].shape[0]:
        assert bool((chosen >= r["experts"]).any())
    # a token's result does not depend on the rows around it
    alone, _, _ = _moe_run(w, mlp, x[17:18], torch.float32)
    assert torch.equal(alone[:, 0], out[:, 17])
    xb = x.to(torch.bfloat16)
    outb, idsb, _ = _moe_run(w, mlp, xb, torch.bfloat16)
    wb = {k: (v if k in ("router", "correction") else v.to(torch.bfloat16)) for k, v in w.items()}
    same = (idsb.cpu().long() == plain.route(xb, w["router"], w["correction"], r)[0]).all(dim=1)
    wantb = plain.routed_ff(xb, {"m." + k: v for k, v in wb.items()}, "m.", mlp)
    close(outb.sum(0)[same], wantb[same], torch.bfloat16, "bfloat16 output")
    assert int(same.sum()) >= T - 2


# ------------------------------------------------------------------ attention
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(4, 2, 16, 16), (4, 2, 16, 40), (6, 3, 48, 16), (2, 1, 96, 96)])
def test_attention_value_size_temperature_and_sink(dtype, shape):
    """Through the mixer part: q/k norms, the query factor, the sink of logit zero,
    values narrower and wider than the keys; a prompt and its continuation."""
    from grout_b200.cache import CacheLayout, SequenceCache
    from grout_b200.parts import BuildContext, PartSpec, build_part
    H, G, dk, dv = shape
    W, T, eps = 32, 100, 1e-5
    m = dict(heads=H, kv_heads=G, dim=dk, vdim=dv, scale=1.7 / math.sqrt(dk), q_temp={"coef": 0.8, "every": 7})
    g = torch.Generator().manual_seed(21)
    r = lambda *s, sc=1.0: torch.randn(*s, generator=g) * sc
    w = {"q": r(H * dk, W), "k": r(G * dk, W), "v": r(G * dv, W), "o": r(W, H * dv, sc=0.2),
         "q.norm": 1 + r(dk, sc=0.3), "k.norm": 1 + r(dk, sc=0.3)}
    w = {k: v.to(dtype) for k, v in w.items()}
    x = r(T, W).to(dtype)
    want = plain.attention_mixer(x, {"m." + k: v for k, v in w.items()}, "m.", m, eps)
    ctx = BuildContext(dtype, torch.device(DEV))
    part = build_part("mixer", PartSpec("gqa_attention", dict(
        hidden=W, n_heads=H, n_kv_heads=G, head_dim=dk, v_head_dim=dv, position=PartSpec("none", {}),
        qk_norm_eps=eps, scale=m["scale"], sink_logit=0.0, q_temp=(0.8, 7),
        names={"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"})), ctx)
    part.load({k: v.to(DEV) for k, v in w.items()})
    cache = SequenceCache(CacheLayout.from_specs([part.cache_spec()]), max_tokens=512, max_slots=2,
                          max_seq_len=256, dtype=dtype, device=DEV)
    slot = cache.open()
    outs, start = [], 0
    for n in (63, 2, 34, 1):
        cache.reserve(slot, n)
        cache.flush()
        step = Step([(slot, start, n)]).ctx
        outs.append(part.forward(x[start:start + n].to(DEV), step, cache.view(0)))
        outs[-1] = (outs[-1].sum(0) if outs[-1].dim() == 3 else outs[-1]).float().cpu()
        cache.advance(slot, n)
        start += n
    got = torch.cat(outs)
    if dtype == torch.float32:
        close(got, want, dtype)
    else:
        d = (got.double() - want)
        assert float(d.pow(2).mean().sqrt() / want.pow(2).mean().sqrt()) < 0.03
    # the sink and the temperature are there: the plain result without them differs
    m2 = dict(m, q_temp=None)
    assert float((plain.attention_mixer(x, {"m." + k: v for k, v in w.items()}, "m.", m2, eps) - want).abs().max()) > 0.05


def test_attention_finds_a_far_key_beside_the_sink():
    """One key far back is made to stand out for the last query: with the sink's
    share known, the output is that key's value times exp(s) / (1 + sum exp)."""
    dk = dv = 16
    T = 700
    k = rnd(T, dk, seed=31, scale=0.05).double()
    v = rnd(T, dv, seed=32).double()
    q = torch.zeros(T, dk, dtype=torch.float64)
    k[3] = 0
    k[3, 2] = 4.0
    q[T - 1, 2] = 2.0
    out = plain.sink_attention(q, k, v, 1.0)[T - 1]
    e = torch.exp(q[T - 1] @ k.T)
    assert torch.allclose(out, (e[:, None] * v).sum(0) / (1 + e.sum()))
    assert float(e[3] / (1 + e.sum())) > 0.7
    from grout_b200.kernels import ops
    from grout_b200.cache import CacheLayout, KVSpec, SequenceCache
    for dtype in (torch.float32, torch.bfloat16):
        cache = SequenceCache(CacheLayout.from_specs([KVSpec(1, dk, None)]), max_tokens=1024, max_slots=1,
                              max_seq_len=1024, dtype=dtype, device=DEV)
        slot = cache.open()
        cache.reserve(slot, T)
        cache.flush()
        step = Step([(slot, 0, T)]).ctx
        view = cache.view(0)
        qkv = torch.cat([q, k, v], dim=1).to(dtype).to(DEV).contiguous()
        qq, _ = ops.qk_prepare(qkv, 1, 1, dk, token_seq=step.token_seq, token_pos=step.token_pos,
                               slots=step.slots, block_table=view.block_table, k_pages=view.k_pages,
                               v_pages=view.v_pages, page=view.page)
        sinks = torch.zeros(1, device=DEV)
        got = ops.attention(qq, view.k_pages, view.v_pages, view.block_table, step=step, page=view.page,
                            scale=1.0, sinks=sinks)[T - 1, 0].float().cpu()
        close(got, out, dtype, "prompt")
        # the same query alone, as a decode step over the cached keys
        step1 = Step([(slot, T - 1, 1)]).ctx
        got1 = ops.attention(qq[T - 1:].contiguous(), view.k_pages, view.v_pages, view.block_table,
                             step=step1, page=view.page, scale=1.0, sinks=sinks)[0, 0].float().cpu()
        close(got1, out, dtype, "decoded")
