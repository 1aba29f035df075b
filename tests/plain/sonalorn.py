"""Plain Sonalorn decoder: whole sequences, no cache, one function per mechanism.

Sonalorn is a decoder whose layers normalise a sublayer's *output* only: the
mixer and the feed-forward read the residual stream x as it is, and

    x <- x + s1 * N1(mixer(x));    x <- x + s2 * N2(ff(x))        (second line only with an ff)

with RMS norms N and learned per-channel scales s ("layer scale").  The stream
starts as N(embed[token] + pos[p]).  A layer's mixer is either a gated delta
rule (a matrix-valued recurrent state per head, short causal convolutions in
front of it) or causal attention without rotation whose queries grow with the
logarithm of the position and whose softmax has one more term, exp(0), in the
denominator.  A feed-forward is dense (gelu-tanh gate) or a mixture of small
experts with clamped activations, chosen through corrected scores restricted to
the best groups of experts; the last few router outputs stand for experts that
hand their input on unchanged.  A layer may run another layer's weights on a
state of its own.

All arithmetic is float64 on the CPU.  Inputs are a dict ``name -> tensor`` with
the checkpoint's tensor names and the raw ``config.json`` dict.  Nothing here is
shared with the product package.
"""
from __future__ import annotations

import math

import torch

DT = torch.float64


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w (w may be None)."""
    x = x.to(DT)
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + float(eps))
    return y if w is None else y * w.to(DT)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def embed(tokens, table, pos_table, norm_w, eps, first_pos=0):
    """N(table[token] + pos_table[p]), p counted from ``first_pos``."""
    p = torch.arange(first_pos, first_pos + len(tokens))
    x = table.to(DT)[torch.as_tensor(tokens)] + pos_table.to(DT)[p]
    return rms_norm(x, norm_w, eps)


def short_conv(x, taps_w):
    """x [T, C], taps_w [C, taps]; y[t, c] = sum_j taps_w[c, taps-1-j] x[t-j, c],
    zeros in front of the sequence."""
    T, C = x.shape
    taps = taps_w.shape[1]
    w = taps_w.to(DT)
    y = torch.zeros(T, C, dtype=DT)
    for j in range(taps):
        if j < T:
            y[j:] += w[:, taps - 1 - j] * x[:T - j]
    return y


def delta_rule(q, k, v, beta, decay):
    """One head.  q, k [T, dk]; v [T, dv]; beta, decay [T].  S starts at zero;
    per token S <- decay S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    q, k, v, beta, decay = (x.to(DT) for x in (q, k, v, beta, decay))
    T, dk = k.shape
    S = torch.zeros(dk, v.shape[1], dtype=DT)
    out = []
    for t in range(T):
        S = decay[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out.append(S.T @ q[t])
    return torch.stack(out), S


def delta_mixer(h, W, prefix, m, eps):
    """The gated-delta mixer on rows h [T, width]; m = the layer's mixer sizes."""
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    h = h.to(DT)
    g = lambda n: W[prefix + n].to(DT)
    T = h.shape[0]
    q = silu(short_conv(h @ g("q").T, g("q.conv"))).view(T, G, dk)
    k = silu(short_conv(h @ g("k").T, g("k.conv"))).view(T, G, dk)
    v = silu(short_conv(h @ g("v").T, g("v.conv"))).view(T, H, dv)
    unit = lambda x: x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)
    q = unit(q) * dk ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ g("b").T)                                        # [T, H]
    decay = torch.exp(-torch.exp(g("A_log")) *
                      torch.nn.functional.softplus(h @ g("a").T + g("dt_bias")))   # [T, H]
    gate = silu(h @ g("g").T).view(T, H, dv)
    outs = []
    for i in range(H):
        kv = i // (H // G)
        o, _S = delta_rule(q[:, kv], k[:, kv], v[:, i], beta[:, i], decay[:, i])
        outs.append(rms_norm(o, g("norm"), eps) * gate[:, i])
    return torch.cat(outs, dim=-1) @ g("o").T


def query_temperature(positions, coef, every):
    """1 + coef ln(floor((p + 1) / every) + 1) for every position."""
    p = torch.as_tensor(positions, dtype=torch.int64)
    return 1.0 + float(coef) * torch.log((torch.div(p + 1, int(every), rounding_mode="floor") + 1).to(DT))


def sink_attention(q, k, v, scale):
    """One head, causal; the denominator holds one more term exp(0) = 1."""
    q, k, v = q.to(DT), k.to(DT), v.to(DT)
    s = (q @ k.T) * float(scale)
    T = q.shape[0]
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, -math.inf)
    mx = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - mx)
    p = e / (torch.exp(-mx) + e.sum(dim=-1, keepdim=True))
    return p @ v


def attention_mixer(h, W, prefix, m, eps, first_pos=0):
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    h = h.to(DT)
    g = lambda n: W[prefix + n].to(DT)
    T = h.shape[0]
    q = rms_norm((h @ g("q").T).view(T, H, dk), g("q.norm"), eps)
    k = rms_norm((h @ g("k").T).view(T, G, dk), g("k.norm"), eps)
    v = (h @ g("v").T).view(T, G, dv)
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(range(first_pos, first_pos + T), qt["coef"], qt["every"])[:, None, None]
    outs = [sink_attention(q[:, i], k[:, i // (H // G)], v[:, i // (H // G)], m["scale"])
            for i in range(H)]
    return torch.cat(outs, dim=-1) @ g("o").T


def dense_ff(h, W, prefix):
    h = h.to(DT)
    g = lambda n: W[prefix + n].to(DT)
    return (gelu_tanh(h @ g("gate").T) * (h @ g("up").T)) @ g("down").T


def route(h, router_w, correction, r):
    """Returns (chosen [T, top] expert indices, weights [T, top]).  Scores are the
    softmax over all router outputs; the choice uses scores + correction, only
    inside the ``keep`` groups whose best corrected score is largest; the weights
    are the uncorrected scores of the chosen."""
    n_all = router_w.shape[0]
    s = torch.softmax(h.to(DT) @ router_w.to(DT).T, dim=-1)
    c = s + correction.to(DT)
    groups = r.get("groups")
    if groups:
        per = n_all // groups["count"]
        best = c.view(-1, groups["count"], per).max(dim=-1).values
        kept = best.topk(groups["keep"], dim=-1).indices
        allow = torch.zeros(c.shape[0], groups["count"], dtype=torch.bool)
        allow.scatter_(1, kept, True)
        c = c.masked_fill(~allow.repeat_interleave(per, dim=1), -math.inf)
    chosen = c.topk(r["top"], dim=-1).indices
    return chosen, s.gather(1, chosen)


def expert(h, W, prefix, limit):
    g = lambda n: W[prefix + n].to(DT)
    a = torch.clamp(h @ g("gate").T, max=float(limit))
    u = torch.clamp(h @ g("up").T, min=-float(limit), max=float(limit))
    return (a * torch.sigmoid(1.702 * a) * (u + 1.0)) @ g("down").T


def routed_ff(h, W, prefix, mlp):
    r = mlp["router"]
    h = h.to(DT)
    chosen, weights = route(h, W[prefix + "router"], W[prefix + "correction"], r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weights[t]):
            if e >= r["experts"]:            # an expert that hands its input on
                out[t] += w * h[t]
            else:
                out[t] += w * expert(h[t:t + 1], W, f"{prefix}e{e}.", mlp["expert"]["limit"])[0]
    return out


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] (and the stream after every layer run) of one sequence."""
    eps = cfg["norm"]["eps"]
    x = embed(tokens, W["embed"], W["pos"], W["embed.norm"], eps)
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        m = layer["mixer"]
        if layer["type"] == "delta":
            y = delta_mixer(x, W, p + "mix.", m, eps)
        elif layer["type"] == "attention":
            y = attention_mixer(x, W, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + W[p + "ls1"].to(DT) * rms_norm(y, W[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(x, W, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(x, W, p + "mlp.", mlp)
            x = x + W[p + "ls2"].to(DT) * rms_norm(y, W[p + "norm2"], eps)
        after.append(x.clone())
    logits = rms_norm(x, W["final.norm"], eps) @ W["head"].to(DT).T
    return (logits, torch.stack(after)) if return_layers else logits


def logits(W, cfg, tokens, rows=None):
    """Logits [T, vocab] of one sequence (or of the given rows)."""
    out = forward(cfg, W, list(tokens))
    return out if rows is None else out[list(rows)]


def greedy_generate(W, cfg, prompt, n_new, stop_ids=()):
    """The plain loop: the whole sequence again for every new token."""
    seq, out = list(prompt), []
    for _ in range(n_new):
        tok = int(torch.argmax(forward(cfg, W, seq)[-1]))
        if tok in stop_ids:
            break
        out.append(tok)
        seq.append(tok)
    return out
