"""Plain Suvazen decoder: whole sequences, no cache, one function per mechanism.

Suvazen is a decoder whose layers are "sandwiched": every sublayer has a layer
norm (weight and bias) in front of it and another behind it, and its normalised
output enters the residual stream times a constant.  Its attention has grouped
heads whose values are the keys as projected (before the rotation), a partial
rotation with Llama-3.1-style scaling of the frequencies, scores that are capped
by a tanh, a sliding window and one learned "sink" logit per head that takes
part in the softmax's denominator only.  The feed-forward is up, relu squared,
down.  A run of layers may be passed through several times, each pass with its
own keys and a learned vector added to the stream in front of it.

All arithmetic is float64 on the CPU.  Inputs are a dict ``name -> tensor`` with
the checkpoint's tensor names and the raw ``config.json`` dict.  Nothing here is
shared with the product package.
"""
from __future__ import annotations

import math

import torch

DT = torch.float64


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b, var = mean of squared deviations."""
    x = x.to(DT)
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    var = (d * d).mean(dim=-1, keepdim=True)
    return d / torch.sqrt(var + float(eps)) * w.to(DT) + b.to(DT)


def scaled_frequencies(n_rot: int, base: float, scaling=None):
    """f_i = base^(-2i / n_rot), i < n_rot / 2.  With ``scaling`` (factor, low,
    high, original): a frequency whose wavelength 2 pi / f is shorter than
    original / high stays; one whose wavelength is longer than original / low is
    divided by factor; between the two the weights (1 - s) and s mix f / factor
    and f, s = (original / wavelength - low) / (high - low)."""
    out = []
    for i in range(n_rot // 2):
        f = float(base) ** (-2.0 * i / n_rot)
        if scaling:
            fac, lo, hi, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave < orig / hi:
                pass
            elif wave > orig / lo:
                f = f / fac
            else:
                s = (orig / wave - lo) / (hi - lo)
                f = (1.0 - s) * f / fac + s * f
        out.append(f)
    return torch.tensor(out, dtype=DT)


def rotate(x, positions, freqs):
    """x [T, heads, D]; the first 2 * len(freqs) elements of every head are
    rotated, element i together with element i + len(freqs), by the angle
    position * freqs[i]; the rest is left as it is."""
    n = freqs.shape[0]
    if n == 0:
        return x
    ang = torch.as_tensor(positions, dtype=DT)[:, None] * freqs[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b, rest = x[..., :n], x[..., n:2 * n], x[..., 2 * n:]
    return torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)


def capped(s, cap):
    """cap * tanh(s / cap); no cap when ``cap`` is None."""
    return s if cap is None else float(cap) * torch.tanh(s / float(cap))


def sink_softmax_attention(q, k, v, *, scale, cap=None, window=None, sink=None):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] of one sequence from position 0.
    Query head h reads kv head h // (H / G).  Scores q.k * scale, capped; key j is
    seen by query i when 0 <= i - j < window (all j <= i without a window); the
    softmax's denominator holds exp(sink[h]) besides the seen keys' terms."""
    T, H, _D = q.shape
    G = k.shape[1]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < int(window))
    out = torch.empty(T, H, v.shape[-1], dtype=DT)
    for h in range(H):
        g = h // (H // G)
        s = capped((q[:, h] @ k[:, g].T) * float(scale), cap)
        s = s.masked_fill(~seen, float("-inf"))
        top = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            top = torch.maximum(top, sink[h].to(DT).reshape(1, 1))
        e = torch.exp(s - top)
        den = e.sum(dim=-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h].to(DT) - top)
        out[:, h] = (e / den) @ v[:, g]
    return out


def attention_mixer(h, w, prefix, m, positions):
    """The whole mixer: q and k projections, v = k before the rotation, the
    rotation of q and k, attention, output projection.  ``m`` is the layer's
    ``mixer`` object of config.json."""
    T = h.shape[0]
    H, G, D = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    h = h.to(DT)
    q = (h @ w[prefix + "q"].to(DT).T).reshape(T, H, D)
    k = (h @ w[prefix + "k"].to(DT).T).reshape(T, G, D)
    v = k
    rot = m.get("rot")
    if rot:
        f = scaled_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
        q, k = rotate(q, positions, f), rotate(k, positions, f)
    mask = m.get("mask")
    o = sink_softmax_attention(q, k, v, scale=m["scale"], cap=m.get("softcap"),
                               window=mask["size"] if mask else None,
                               sink=w.get(prefix + "sink"))
    return o.reshape(T, -1) @ w[prefix + "o"].to(DT).T


def relu_squared_ff(h, w_up, w_down):
    """W_down (max(W_up h, 0))^2."""
    u = torch.clamp(h.to(DT) @ w_up.to(DT).T, min=0.0)
    return (u * u) @ w_down.to(DT).T


def _ln(x, w, name, eps):
    return layer_norm(x, w[name], w[name + ".b"], eps)


def sandwich_layer(x, w, i, cfg, positions):
    """x += m * norm1b(mixer(norm1(x))); x += m * norm2b(ff(norm2(x)))."""
    L = cfg["layers"][i]
    p, eps, mult = f"l{i}.", cfg["norm"]["eps"], float(cfg.get("residual_mult", 1.0))
    if L["type"] != "attention":
        raise ValueError(f"no plain mixer of type {L['type']!r}")
    a = attention_mixer(_ln(x, w, p + "norm1", eps), w, p + "mix.", L["mixer"], positions)
    x = x + mult * _ln(a, w, p + "norm1b", eps)
    if L.get("mlp"):
        if L["mlp"]["kind"] != "dense":
            raise ValueError(f"no plain feed-forward of kind {L['mlp']['kind']!r}")
        f = relu_squared_ff(_ln(x, w, p + "norm2", eps), w[p + "mlp.up"], w[p + "mlp.down"])
        x = x + mult * _ln(f, w, p + "norm2b", eps)
    return x


def layer_runs(cfg):
    """The order in which layers run: (layer, pass number or None when it is the
    first layer of no pass).  Layers start..stop-1 are gone through ``times``
    times before the rest follows."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(int(loop["times"])):
        for i in range(loop["start"], loop["stop"]):
            runs.append((i, t if i == loop["start"] else None))
    runs += [(i, None) for i in range(loop["stop"], n)]
    return runs


def hidden_states(w, cfg, tokens, trace=None):
    """Embedding and every layer run of one whole sequence at positions 0..T-1.
    ``trace``: a list that receives the stream after each layer run."""
    x = w["embed"].to(DT)[torch.as_tensor(tokens, dtype=torch.long)]
    positions = list(range(len(tokens)))
    for i, t in layer_runs(cfg):
        if t is not None:
            x = x + w["loop.step"].to(DT)[t]
        x = sandwich_layer(x, w, i, cfg, positions)
        if trace is not None:
            trace.append(x.clone())
    return x


def logits(w, cfg, tokens, rows=None):
    x = hidden_states(w, cfg, tokens)
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long)]
    h = _ln(x, w, "final.norm", cfg["norm"]["eps"])
    z = (h @ w["head"].to(DT).T) * float(cfg.get("logit_scale", 1.0))
    return capped(z, cfg.get("logit_softcap"))


def greedy_generate(w, cfg, prompt, max_new_tokens: int, stop_ids=()):
    """Recomputes the whole prefix for every token; ties go to the lowest index."""
    seq, out = list(prompt), []
    for _ in range(max_new_tokens):
        tok = int(torch.argmax(logits(w, cfg, seq, rows=[len(seq) - 1])[0]))
        if tok in stop_ids:
            break
        out.append(tok)
        seq.append(tok)
    return out
