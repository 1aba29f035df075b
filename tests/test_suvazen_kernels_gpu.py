"""The mechanisms that the Suvazen design brought, each alone against the plain
implementation: the fused add + layer norm of sandwich layers, q/k preparation
with values taken from the unrotated keys and a partial rotation, every attention
kernel with a score cap and sinks, the squared relu in the products' epilogues,
and the scaled, capped logits."""
import math

import pytest
import torch

from plain import suvazen as plain
from test_kernels_gpu import DEV, DT, FAST_TOL, Paged, _clear_axis, _eps, _plant_window_edge, _rand, _restore

pytestmark = pytest.mark.gpu


def _ops():
    from grout_b200.kernels import ops
    return ops


# ------------------------------------------------------------------ add + layer norm
@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("rows", [9, 100])      # few rows of a wide model share a row among blocks
@pytest.mark.parametrize("N", [200, 203, 2560, 5000, 12000])
def test_add_layernorm_every_form(dtype, N, rows):
    dt = DT[dtype]
    res = _rand((rows, N), torch.float32, 3, 2.0)
    delta = _rand((rows, N), dt, 4) + 0.3                         # a mean that is not zero
    w, b = 1 + 0.1 * _rand((N,), torch.float32, 5), 0.2 * _rand((N,), torch.float32, 6)
    pw, pb = 1 + 0.2 * _rand((N,), torch.float32, 7), 0.3 * _rand((N,), torch.float32, 8)
    off = _rand((N,), torch.float32, 9)
    eps, peps, mult = 1e-5, 3e-4, 0.7
    tol = dict(atol=6 * _eps(dt), rtol=3 * _eps(dt))
    g = lambda t: None if t is None else t.to(DEV)                # noqa: E731
    ops = _ops()

    # the whole sandwich step, in place
    want_res = res.double() + mult * plain.layer_norm(delta.double(), pw, pb, peps) + off.double()
    want_y = plain.layer_norm(want_res, w, b, eps)
    r = res.clone().to(DEV)
    res_out, y = ops.add_layernorm(r, g(delta), g(w), g(b), eps, dtype=dt, mult=mult, offset=g(off),
                                   post_weight=g(pw), post_bias=g(pb), post_eps=peps)
    assert res_out.data_ptr() == r.data_ptr()
    assert torch.allclose(res_out.cpu().double(), want_res, atol=2e-5, rtol=1e-5)
    assert torch.allclose(y.cpu().double(), want_y, **tol)

    # gathered rows (what the final norm does), no offset
    idx = torch.tensor([8, 0, 3], dtype=torch.int32)
    want_res = res.double() + mult * plain.layer_norm(delta.double(), pw, pb, peps)
    res2, y2 = ops.add_layernorm(g(res), g(delta), g(w), g(b), eps, dtype=dt, rows=g(idx), mult=mult,
                                 post_weight=g(pw), post_bias=g(pb), post_eps=peps)
    assert torch.allclose(res2.cpu().double(), want_res[idx.long()], atol=2e-5, rtol=1e-5)
    assert torch.allclose(y2.cpu().double(), plain.layer_norm(want_res, w, b, eps)[idx.long()], **tol)

    # first-layer form: no stream yet, the delta is the embedding, plus an offset
    res3, y3 = ops.add_layernorm(None, g(delta), g(w), g(b), eps, dtype=dt, offset=g(off))
    want3 = delta.double() + off.double()
    assert torch.allclose(res3.cpu().double(), want3, atol=1e-6, rtol=1e-6)
    assert torch.allclose(y3.cpu().double(), plain.layer_norm(want3, w, b, eps), **tol)

    # the plain norm, and the sum without a norm
    _r, y4 = ops.add_layernorm(None, g(delta), g(w), g(b), eps, dtype=dt, write_res=False)
    assert _r is None and torch.allclose(y4.cpu().double(), plain.layer_norm(delta.double(), w, b, eps), **tol)
    res5, y5 = ops.add_layernorm(g(res), g(delta), None, None, eps, dtype=dt, rows=g(idx), mult=mult)
    assert y5 is None
    assert torch.allclose(res5.cpu().double(), (res.double() + mult * delta.double())[idx.long()],
                          atol=1e-5, rtol=1e-6)

    # a norm that leaves the mean in and has no bias
    _r, y6 = ops.add_layernorm(None, g(delta), g(w), None, eps, False, dtype=dt, write_res=False)
    x = delta.double()
    want6 = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.double()
    assert torch.allclose(y6.cpu().double(), want6, **tol)


@pytest.mark.parametrize("N", [200, 2560])
def test_add_layernorm_takes_partial_sums(N):
    """A split-K product leaves its sum to the norm: the parts are added in order
    and then treated as the delta."""
    ops = _ops()
    parts = _rand((5, 7, N), torch.float32, 11)
    res = _rand((7, N), torch.float32, 12)
    w, b = 1 + 0.1 * _rand((N,), torch.float32, 13), 0.1 * _rand((N,), torch.float32, 14)
    pw, pb = 1 + 0.1 * _rand((N,), torch.float32, 15), 0.1 * _rand((N,), torch.float32, 16)
    d = parts.double().sum(0)
    want_res = res.double() + 0.5 * plain.layer_norm(d, pw, pb, 1e-5)
    got_res, y = ops.add_layernorm(res.to(DEV), parts.to(DEV), w.to(DEV), b.to(DEV), 1e-6,
                                   dtype=torch.bfloat16, mult=0.5, post_weight=pw.to(DEV),
                                   post_bias=pb.to(DEV), post_eps=1e-5)
    assert torch.allclose(got_res.cpu().double(), want_res, atol=2e-5, rtol=1e-5)
    assert torch.allclose(y.cpu().double(), plain.layer_norm(want_res, w, b, 1e-6), atol=0.03, rtol=0.01)


def test_add_layernorm_row_independent():
    """In 32-bit a row's result is the same in a step of one row and of many."""
    ops = _ops()
    N = 2560
    res, delta = _rand((40, N), torch.float32, 17), _rand((40, N), torch.float32, 18)
    w, b = _rand((N,), torch.float32, 19), _rand((N,), torch.float32, 20)
    kw = dict(dtype=torch.float32, mult=0.7, post_weight=w.to(DEV), post_bias=b.to(DEV), post_eps=1e-5)
    _r, many = ops.add_layernorm(res.to(DEV), delta.to(DEV), w.to(DEV), b.to(DEV), 1e-5, **kw)
    _r, one = ops.add_layernorm(res[17:18].to(DEV), delta[17:18].to(DEV), w.to(DEV), b.to(DEV), 1e-5, **kw)
    assert torch.equal(many[17:18], one)


# ------------------------------------------------------------------ q/k preparation
@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("T", [3, 200])
@pytest.mark.parametrize("nq,nkv,D,rot", [(6, 2, 48, 16), (4, 4, 64, 32), (8, 1, 128, 128),
                                          (3, 3, 16, 8), (4, 2, 32, 32), (2, 1, 256, 64), (5, 5, 64, 0)])
def test_qk_prepare_values_are_unrotated_keys(dtype, T, nq, nkv, D, rot):
    """The projection holds q and k only; the keys are stored rotated (their first
    ``rot`` elements) and the values are the keys before the rotation."""
    ops = _ops()
    dt = DT[dtype]
    qk = _rand((T, (nq + nkv) * D), dt, 21)
    lens = [T + 70]                                   # one sequence that already holds 70 tokens
    pc = Paged(lens, nkv, D, dt, 22, fill=0.0)
    pos = torch.arange(70, 70 + T, dtype=torch.int32)
    freqs = plain.scaled_frequencies(rot, 7000.0, None) if rot else None
    inv = freqs.float().to(DEV) if rot else None
    kp, vp = pc.k_pages.to(DEV), pc.v_pages.to(DEV)
    q, kv = ops.qk_prepare(qk.to(DEV), nq, nkv, D, inv_freq=inv, rot_dim=rot,
                           token_seq=torch.zeros(T, dtype=torch.int32, device=DEV),
                           token_pos=pos.to(DEV), slots=torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV),
                           block_table=pc.table.to(DEV), k_pages=kp, v_pages=vp, page=64,
                           want_kv_out=True, values_are_keys=True)
    x = qk.double().reshape(T, nq + nkv, D)
    want_q, want_k, want_v = x[:, :nq], x[:, nq:], x[:, nq:]
    if rot:
        # the table is rounded to 32-bit once, and so is the angle
        ang = (pos.float()[:, None] * freqs.float()[None, :]).double()
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        h = rot // 2

        def turn(t):
            a, b, rest = t[..., :h], t[..., h:rot], t[..., rot:]
            return torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)
        want_q, want_k = turn(want_q), turn(want_k)
    tol = dict(atol=3 * _eps(dt), rtol=2 * _eps(dt))
    assert torch.allclose(q.cpu().double(), want_q, **tol)
    assert torch.allclose(kv.cpu().double()[:, :nkv], want_k, **tol)
    assert torch.allclose(kv.cpu().double()[:, nkv:], want_v, **tol)
    kp, vp, table = kp.cpu(), vp.cpu(), pc.table
    for t in (0, T // 2, T - 1):
        p = 70 + t
        pg = int(table[pc.slot_of[0], p // 64])
        assert torch.allclose(kp[pg, :, p % 64].double(), want_k[t], **tol), t
        assert torch.allclose(vp[pg, :, p % 64].double(), want_v[t], **tol), t
    # the rotation agrees with the plain one (same pairing, same untouched rest)
    if rot:
        ref = plain.rotate(x[:, :nq], pos.tolist(), freqs)
        assert torch.allclose(q.cpu().double(), ref, atol=2e-2 if dt == torch.bfloat16 else 2e-3, rtol=1e-2)


@pytest.mark.parametrize("nq,nkv,D,rot", [(4, 4, 64, 32), (8, 1, 128, 64), (6, 2, 48, 16)])
def test_qk_prepare_values_are_keys_from_partial_sums(nq, nkv, D, rot):
    ops = _ops()
    T = 5
    parts = _rand((3, T, (nq + nkv) * D), torch.float32, 23)
    whole = parts.sum(0).to(torch.bfloat16)
    args = dict(inv_freq=plain.scaled_frequencies(rot, 1e4, None).float().to(DEV), rot_dim=rot,
                token_seq=torch.zeros(T, dtype=torch.int32, device=DEV),
                token_pos=torch.arange(9, 9 + T, dtype=torch.int32, device=DEV),
                slots=torch.tensor([-1], dtype=torch.int32, device=DEV), want_kv_out=True,
                values_are_keys=True)
    q1, kv1 = ops.qk_prepare(parts.to(DEV), nq, nkv, D, **args)
    q2, kv2 = ops.qk_prepare(whole.to(DEV), nq, nkv, D, **args)
    assert torch.allclose(q1.float(), q2.float(), atol=0.03, rtol=0.02)
    assert torch.allclose(kv1.float(), kv2.float(), atol=0.03, rtol=0.02)


# ------------------------------------------------------------------ attention with a cap and sinks
def _oracle(q, k, v, pos, scale, window, cap, sinks):
    """q [nq, D] at absolute position pos over keys k, v [n, nkv, D]."""
    nq, D = q.shape
    nkv = k.shape[1]
    out = torch.empty(nq, D, dtype=torch.float64)
    lo = 0 if window is None else max(0, pos - window + 1)
    for h in range(nq):
        kh, vh = k[lo:pos + 1, h // (nq // nkv)].double(), v[lo:pos + 1, h // (nq // nkv)].double()
        s = plain.capped((kh @ q[h].double()) * scale, cap)
        top = s.max()
        if sinks is not None:
            top = torch.maximum(top, sinks[h].double())
        e = torch.exp(s - top)
        den = e.sum() + (torch.exp(sinks[h].double() - top) if sinks is not None else 0.0)
        out[h] = (e / den) @ vh
    return out


def _sinks(nq, seed):
    """Sinks that matter: one head's sink dwarfs its keys, one is far below them."""
    s = 2.0 * _rand((nq,), torch.float32, seed)
    s[0] = 9.0
    if nq > 1:
        s[1] = -30.0
    return s


CAPS = [(None, False), (7.0, True), (7.0, False), (None, True)]


@pytest.mark.parametrize("cap,with_sinks", CAPS)
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("nq,nkv,D", [(6, 2, 48), (8, 1, 128)])
def test_attn_generic_cap_and_sinks(dtype, nq, nkv, D, window, cap, with_sinks):
    dt = DT[dtype]
    lens = [1, 130, 200, 64]
    pc = Paged(lens, nkv, D, dt, 7)
    places = [(0, 0), (1, 129), (2, 199), (3, 63), (2, 0), (2, 63), (2, 64), (2, 127), (2, 128)]
    q = _rand((len(places), nq, D), dt, 8, 3.0)       # scores well into the cap's bend
    scale = 1.0 / math.sqrt(D)
    sinks = _sinks(nq, 9) if with_sinks else None
    got = _ops().attn_generic(
        q.to(DEV), pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV),
        token_seq=torch.tensor([s for s, _ in places], dtype=torch.int32, device=DEV),
        token_pos=torch.tensor([p for _, p in places], dtype=torch.int32, device=DEV),
        slots=torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV), page=64, scale=scale,
        window=window, softcap=cap, sinks=None if sinks is None else sinks.to(DEV)).cpu()
    for r, (s, p) in enumerate(places):
        want = _oracle(q[r], pc.k[s], pc.v[s], p, scale, window, cap, sinks)
        # (scores of ten or so: their own 32-bit rounding is a relative 5e-7 of a weight)
        k_eps = 6 if dt == torch.bfloat16 else 24
        assert torch.allclose(got[r].double(), want, atol=k_eps * _eps(dt), rtol=k_eps * _eps(dt)), (r, s, p)
    if with_sinks:
        # the first token sees itself and the sink: head 0's output is almost nothing
        assert float(got[0, 0].float().abs().max()) < 0.02 * float(pc.v[0][0, 0].float().abs().max())


def _prefill_case(nkv, D, seed, fill):
    plan = [(0, 1), (0, 130), (37, 100), (64, 64), (0, 300), (5, 63), (100, 200)]
    lens = [s + n for s, n in plan]
    pc = Paged(lens, nkv, D, torch.bfloat16, seed, fill=fill)
    cu = [0]
    for _s, n in plan:
        cu.append(cu[-1] + n)
    return plan, lens, pc, cu


@pytest.mark.parametrize("cap,with_sinks", CAPS[1:])
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("kernel,nq,nkv,D", [("mma", 6, 2, 48), ("mma", 16, 4, 64), ("tc-128", 6, 2, 64),
                                            ("tc-256", 6, 2, 64), ("tc-256", 8, 1, 128), ("tc-128", 4, 4, 128)])
def test_prompt_attention_cap_and_sinks(kernel, nq, nkv, D, window, cap, with_sinks):
    ops = _ops()
    plan, lens, pc, cu = _prefill_case(nkv, D, 46, 300.0 if kernel != "mma" else float("nan"))
    q = _rand((cu[-1], nq, D), torch.bfloat16, 47, 3.0)
    scale = 1.0 / math.sqrt(D)
    sinks = _sinks(nq, 48) if with_sinks else None
    common = dict(cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV),
                  slots=torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV),
                  kv_len=torch.tensor(lens, dtype=torch.int32, device=DEV),
                  q_lens=tuple(n for _, n in plan), page=64, scale=scale, window=window, softcap=cap,
                  sinks=None if sinks is None else sinks.to(DEV))
    args = (q.to(DEV), pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV))
    if kernel == "mma":
        got = ops.attn_prefill_bf16(*args, **common).cpu()
    else:
        got = ops.attn_prefill_tc(*args, rows_per_block=int(kernel[3:]), **common).cpu()
        ops.check_kernel_errors()
    assert not torch.isnan(got.float()).any()
    for s, (start, n) in enumerate(plan):
        for i in sorted(set([0, min(n - 1, 1), n // 2, n - 1, min(n - 1, 63), min(n - 1, 64), min(n - 1, 127), min(n - 1, 128)])):
            want = _oracle(q[cu[s] + i], pc.k[s], pc.v[s], start + i, scale, window, cap, sinks)
            assert torch.allclose(got[cu[s] + i].double(), want, **FAST_TOL), (s, i)
    s, (start, n) = 2, plan[2]
    for i in range(n):
        want = _oracle(q[cu[s] + i], pc.k[s], pc.v[s], start + i, scale, window, cap, sinks)
        assert torch.allclose(got[cu[s] + i].double(), want, **FAST_TOL), (s, i)


@pytest.mark.parametrize("cap,with_sinks", CAPS[1:])
@pytest.mark.parametrize("n_splits", [1, 3, 11, None])
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("kernel,nq,nkv,D", [("mma", 6, 2, 48), ("mma", 32, 8, 128), ("mma", 16, 1, 32),
                                            ("tma", 8, 1, 128), ("tma", 6, 2, 64), ("tma", 16, 1, 64)])
def test_decode_attention_cap_and_sinks(kernel, nq, nkv, D, window, n_splits, cap, with_sinks):
    ops = _ops()
    lens = [1, 130, 200, 64, 33, 65, 700]
    pc = Paged(lens, nkv, D, torch.bfloat16, 42)
    B = len(lens) + 1                               # one padding row at the end
    q = _rand((B, nq, D), torch.bfloat16, 43, 3.0)
    scale = 1.0 / math.sqrt(D)
    sinks = _sinks(nq, 44) if with_sinks else None
    run = ops.attn_decode_tma if kernel == "tma" else ops.attn_decode_bf16
    got = run(q.to(DEV), pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV),
              slots=torch.tensor(pc.slot_of + [-1], dtype=torch.int32, device=DEV),
              kv_len=torch.tensor(lens + [7], dtype=torch.int32, device=DEV), page=64, scale=scale,
              max_kv_len=1024, window=window, n_splits=n_splits, softcap=cap,
              sinks=None if sinks is None else sinks.to(DEV)).cpu()
    ops.check_kernel_errors()
    assert not torch.isnan(got.float()).any()
    for s, n in enumerate(lens):
        want = _oracle(q[s], pc.k[s], pc.v[s], n - 1, scale, window, cap, sinks)
        assert torch.allclose(got[s].double(), want, **FAST_TOL), (s, n)
    assert bool((got[B - 1] == 0).all())            # the padding row


@pytest.mark.parametrize("kernel", ["generic", "decode-1", "decode-3", "tma-decode-1", "tma-decode-3", "mma",
                                    "tc-128", "tc-256"])
def test_the_window_edge_under_a_cap_with_sinks(kernel):
    """Keys planted just inside and just outside the window, as for the plain
    kernels' own test, but seen through a cap (which squeezes the two planted
    scores together without changing their order) and beside sinks."""
    ops = _ops()
    nq, nkv, D, W, cap = 6, 3, 64, 70, 50.0
    dt = torch.bfloat16
    scale = 1.0 / math.sqrt(D)
    sinks = _sinks(nq, 70).clamp(max=3.0)
    if "decode" in kernel or kernel == "generic":
        lens = [W + 64, W + 81, 3 * 64 + 5, W + 1]
        pc = Paged(lens, nkv, D, dt, 60)
        q = _rand((len(lens), nq, D), dt, 61)
        planted = []
        for s, n in enumerate(lens):
            _clear_axis(pc, s)
            _plant_window_edge(q, s, pc, s, n - 1, W)
            _restore(pc, s)
            planted.append((s, s, n - 1))
        args = (q.to(DEV), pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV))
        slots = torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV)
        if kernel == "generic":
            got = ops.attn_generic(*args, token_seq=torch.arange(len(lens), dtype=torch.int32, device=DEV),
                                   token_pos=torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV),
                                   slots=slots, page=64, scale=scale, window=W, softcap=cap,
                                   sinks=sinks.to(DEV)).cpu()
        else:
            run = ops.attn_decode_tma if kernel.startswith("tma") else ops.attn_decode_bf16
            got = run(*args, slots=slots, kv_len=torch.tensor(lens, dtype=torch.int32, device=DEV),
                      page=64, scale=scale, max_kv_len=512, window=W, n_splits=int(kernel[-1]),
                      softcap=cap, sinks=sinks.to(DEV)).cpu()
    else:
        plan = [(0, 260), (50, 200)]
        spots = {0: [63 + W, 210], 1: [63 + W, 249]}
        lens = [a + n for a, n in plan]
        pc = Paged(lens, nkv, D, dt, 62, fill=300.0)
        cu = [0, plan[0][1], plan[0][1] + plan[1][1]]
        q = _rand((cu[-1], nq, D), dt, 63)
        planted = []
        for s, (held, n) in enumerate(plan):
            _clear_axis(pc, s)
            for pos in spots[s]:
                _plant_window_edge(q, cu[s] + pos - held, pc, s, pos, W)
                planted.append((cu[s] + pos - held, s, pos))
            _restore(pc, s)
        common = dict(cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV),
                      slots=torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV),
                      kv_len=torch.tensor(lens, dtype=torch.int32, device=DEV),
                      q_lens=tuple(n for _, n in plan), page=64, scale=scale, window=W, softcap=cap,
                      sinks=sinks.to(DEV))
        args = (q.to(DEV), pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV))
        if kernel == "mma":
            got = ops.attn_prefill_bf16(*args, **common).cpu()
        else:
            got = ops.attn_prefill_tc(*args, rows_per_block=int(kernel[3:]), **common).cpu()
    ops.check_kernel_errors()
    g = nq // nkv
    for row, s, pos in planted:
        for h in range(nq):
            inner = pc.v[s][pos - W + 1, h // g].double()
            assert torch.allclose(got[row, h].double(), inner, atol=1e-2, rtol=1e-2), (kernel, row, s, pos, h)


def test_a_sink_that_dwarfs_a_far_key():
    """Hundreds of keys, one of which stands out, and a sink as large as its score:
    the output is half that key's value.  A sink that is left out, counted twice
    (once per split) or scaled shows at once."""
    ops = _ops()
    nq, nkv, D = 4, 2, 64
    lens = [900]
    pc = Paged(lens, nkv, D, torch.bfloat16, 80)
    q = torch.zeros((1, nq, D), dtype=torch.bfloat16)
    q[0, :, 0] = 16.0
    pc.k[0][:, :, 0] = 0
    pc.k[0][17, :, 0] = 16.0
    _restore(pc, 0)
    scale, cap = 0.25, 16.0
    top = cap * math.tanh(16.0 * 16.0 * scale / cap)
    sinks = torch.tensor([top, top, -50.0, top + math.log(3.0)])
    want_share = [0.5, 0.5, 1.0, 0.25]
    args = (q.to(DEV), pc.k_pages.to(DEV), pc.v_pages.to(DEV), pc.table.to(DEV))
    slots = torch.tensor(pc.slot_of, dtype=torch.int32, device=DEV)
    kv_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    outs = {}
    for name, run in (("decode", ops.attn_decode_bf16), ("tma", ops.attn_decode_tma)):
        for ns in (1, 4, 13):
            outs[f"{name}-{ns}"] = run(*args, slots=slots, kv_len=kv_len, page=64, scale=scale,
                                       max_kv_len=1024, n_splits=ns, softcap=cap, sinks=sinks.to(DEV)).cpu()
    outs["generic"] = ops.attn_generic(*args, token_seq=torch.zeros(1, dtype=torch.int32, device=DEV),
                                       token_pos=torch.tensor([899], dtype=torch.int32, device=DEV),
                                       slots=slots, page=64, scale=scale, softcap=cap, sinks=sinks.to(DEV)).cpu()
    ops.check_kernel_errors()
    for name, got in outs.items():
        for h in range(nq):
            want = want_share[h] * pc.v[0][17, h // 2].double()
            assert torch.allclose(got[0, h].double(), want, atol=2e-2, rtol=2e-2), (name, h)


# ------------------------------------------------------------------ squared relu, capped logits
@pytest.mark.parametrize("dtype", list(DT))
def test_relu_squared_and_scale_softcap(dtype):
    ops = _ops()
    dt = DT[dtype]
    x = _rand((37, 203), dt, 90, 3.0)
    got = ops.relu_squared(x.to(DEV)).cpu().double()
    want = torch.clamp(x.double(), min=0) ** 2
    assert torch.allclose(got, want, atol=0, rtol=2 * _eps(dt))
    z = _rand((11, 333), torch.float32, 91, 20.0)
    got = ops.scale_softcap_(z.clone().to(DEV), 0.6, 9.0).cpu().double()
    assert torch.allclose(got, plain.capped(z.double() * 0.6, 9.0), atol=1e-5, rtol=1e-5)
    got = ops.scale_softcap_(z.clone().to(DEV), 0.6, None).cpu().double()
    assert torch.allclose(got, z.double() * 0.6, atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("M", [1, 8, 33, 64])
@pytest.mark.parametrize("N,K", [(200, 264), (2560, 96), (320, 4096)])
def test_decode_product_squares_the_relu(M, N, K):
    ops = _ops()
    x, w = _rand((M, K), torch.bfloat16, 92), _rand((N, K), torch.bfloat16, 93, 0.05)
    got = ops.gemm_tc_bf16(x.to(DEV), w.to(DEV), torch.bfloat16, swap=True, relu_squared=True).cpu().double()
    ops.check_kernel_errors()
    want = plain.relu_squared_ff(x.double(), w, torch.eye(N, dtype=torch.float64))
    assert torch.allclose(got, want, atol=2e-3 * float(want.abs().max()), rtol=2e-2)


@pytest.mark.parametrize("kernel", ["pair", "tc"])
@pytest.mark.parametrize("M,N,K", [(300, 520, 264), (129, 2048, 512), (1000, 96, 96)])
def test_prompt_products_square_the_relu(kernel, M, N, K):
    ops = _ops()
    x, w = _rand((M, K), torch.bfloat16, 94), _rand((N, K), torch.bfloat16, 95, 0.05)
    if kernel == "pair":
        got = ops.gemm_tc2_bf16(x.to(DEV), w.to(DEV), torch.bfloat16, relu_squared=True)
    else:
        got = ops.gemm_tc_bf16(x.to(DEV), w.to(DEV), torch.bfloat16, swap=False, relu_squared=True)
    ops.check_kernel_errors()
    want = plain.relu_squared_ff(x.double(), w, torch.eye(N, dtype=torch.float64))
    assert torch.allclose(got.cpu().double(), want, atol=2e-3 * float(want.abs().max()), rtol=2e-2)


# ------------------------------------------------------------------ contributions through any norm
@pytest.mark.parametrize("dtype", list(DT))
def test_a_contribution_through_norms_with_and_without_a_kernel_for_it(dtype):
    """A sublayer's output on its way into the stream (its own norm, a factor, an
    offset): ``LayerNorm`` takes it whole, ``RMSNorm`` and a mixed pair resolve it
    step by step; all agree with the plain arithmetic."""
    from grout_b200.parts import BuildContext, Contribution, PartSpec, build_part
    dt = DT[dtype]
    ctx = BuildContext(dt, torch.device(DEV))
    N, T = 256, 5
    ln_a = build_part("norm", PartSpec("layernorm", dict(dim=N, eps=1e-5)), ctx)
    ln_b = build_part("norm", PartSpec("layernorm", dict(dim=N, eps=2e-5)), ctx)
    rms = build_part("norm", PartSpec("rmsnorm", dict(dim=N, eps=1e-6)), ctx)
    wa, ba = 1 + 0.1 * _rand((N,), torch.float32, 1), 0.1 * _rand((N,), torch.float32, 2)
    wb, bb = 1 + 0.1 * _rand((N,), torch.float32, 3), 0.1 * _rand((N,), torch.float32, 4)
    wr = 1 + 0.1 * _rand((N,), torch.float32, 5)
    ln_a.load({"weight": wa.to(DEV), "bias": ba.to(DEV)})
    ln_b.load({"weight": wb.to(DEV), "bias": bb.to(DEV)})
    rms.load({"weight": wr.to(dt).to(DEV)})
    wr = wr.to(dt)
    res, delta = _rand((T, N), torch.float32, 6), _rand((T, N), dt, 7)
    off = _rand((N,), torch.float32, 8)
    tol = dict(atol=8 * _eps(dt), rtol=4 * _eps(dt))

    def rms_plain(x):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6) * wr.double()

    # layer norm behind, layer norm in front: one kernel
    want = res.double() + 0.6 * plain.layer_norm(delta.double(), wb, bb, 2e-5) + off.double()
    r, y = ln_a.add_norm(res.clone().to(DEV), Contribution(delta.to(DEV), ln_b, 0.6, off.to(DEV)))
    assert torch.allclose(r.cpu().double(), want, atol=1e-5, rtol=1e-5)
    assert torch.allclose(y.cpu().double(), plain.layer_norm(want, wa, ba, 1e-5), **tol)
    # layer norm behind, RMS norm in front: resolved, then the RMS norm's kernel
    r, y = rms.add_norm(res.clone().to(DEV), Contribution(delta.to(DEV), ln_b, 0.6, off.to(DEV)))
    assert torch.allclose(r.cpu().double(), want, atol=4 * _eps(dt), rtol=4 * _eps(dt))
    assert torch.allclose(y.cpu().double(), rms_plain(want), atol=16 * _eps(dt), rtol=8 * _eps(dt))
    # RMS norm behind, layer norm in front
    want = res.double() + 0.6 * rms_plain(delta.double())
    r, y = ln_a.add_norm(res.clone().to(DEV), Contribution(delta.to(DEV), rms, 0.6))
    assert torch.allclose(r.cpu().double(), want, atol=4 * _eps(dt), rtol=4 * _eps(dt))
    assert torch.allclose(y.cpu().double(), plain.layer_norm(want, wa, ba, 1e-5), atol=16 * _eps(dt), rtol=8 * _eps(dt))
    # no norm behind, only an offset (what a pass's vector is in front of a model's first layer)
    r, y = ln_a.add_norm(None, Contribution(delta.to(DEV), None, 1.0, off.to(DEV)))
    want = delta.double() + off.double()
    assert torch.allclose(r.cpu().double(), want, atol=1e-6, rtol=1e-6)
    assert torch.allclose(y.cpu().double(), plain.layer_norm(want, wa, ba, 1e-5), **tol)
