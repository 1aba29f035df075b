"""The Suvazen decoder as a plan.

Sandwich layers (a layer norm with weight and bias in front of and behind each
sublayer, the normalised output times ``residual_mult``); attention with grouped
heads, values that are the unrotated keys, a partial rotation with band-wise
scaled frequencies, capped scores, a sliding window and one sink logit per head;
an up / relu squared / down feed-forward; a run of layers that is gone through
several times, each pass with keys of its own and a learned vector added to the
stream in front of it; a scaled and capped output head.  This file holds the
checkpoint's tensor names and the order of the parts; every size and constant
comes from the configuration, layer by layer.

Tensor names: ``embed``, ``head``, ``final.norm`` (+ ``.b``), ``loop.step``
[passes, width], and per layer i ``l<i>.norm1`` / ``norm1b`` / ``norm2`` /
``norm2b`` (+ ``.b``), ``l<i>.mix.{q,k,o,sink}``, ``l<i>.mlp.{up,down}``.
"""
from __future__ import annotations

from ..config import SuvazenConfig, register_architecture
from ..parts.base import PartSpec
from ..parts.plan import LayerPlan, ModelPlan, ScheduleEntry

LOOP_VECTORS = "loop.step"
NO_POSITION_LIMIT = 1 << 30       # the design states no longest sequence


def _norm(width: int, eps: float) -> PartSpec:
    return PartSpec("layernorm", dict(dim=width, eps=eps, weight_name="", bias_name=".b"))


def _attention(width: int, m: dict) -> PartSpec:
    rot = m.get("rot")
    if rot:
        position = PartSpec("rotary_half_split", dict(
            head_dim=m["dim"], theta=float(rot["base"]), rot_dim=int(rot["dims"]),
            scaling=rot.get("scaling"), exact_table=True))
    else:
        position = PartSpec("none", {})
    mask = m.get("mask")
    return PartSpec("gqa_attention", dict(
        hidden=width, n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"],
        position=position, window=int(mask["size"]) if mask else None, scale=float(m["scale"]),
        softcap=m.get("softcap"), sinks=True, values_are_keys=True,
        names={"q": "q", "k": "k", "o": "o", "sink": "sink"}))


def suvazen_plan(cfg: SuvazenConfig) -> ModelPlan:
    W, eps = cfg.width, float(cfg.norm["eps"])
    layers, unread = [], []
    for i, layer in enumerate(cfg.layers):
        args = dict(norm1=_norm(W, eps), mixer=_attention(W, layer["mixer"]), norm1b=_norm(W, eps),
                    mult=float(cfg.residual_mult))
        mlp = layer.get("mlp")
        if mlp is not None:
            args.update(norm2=_norm(W, eps), norm2b=_norm(W, eps),
                        feedforward=PartSpec("relu2_mlp", dict(
                            hidden=W, intermediate=int(mlp["ff"]),
                            names={"up": "up", "down": "down"})))
        else:       # a writer may still have made the norms of the absent sublayer
            unread += [(f"l{i}.{n}{b}", (W,)) for n in ("norm2", "norm2b") for b in ("", ".b")]
        layers.append(LayerPlan(PartSpec("sandwich", args), f"l{i}.", {
            "norm1": "norm1", "norm1b": "norm1b", "norm2": "norm2", "norm2b": "norm2b",
            "mixer": "mix.", "feedforward": "mlp."}))
    # every run of a layer owns its keys: a layer that is passed through three
    # times appears three times in the schedule
    schedule = tuple(ScheduleEntry(i, add=None if t is None else (LOOP_VECTORS, t))
                     for i, t in cfg.layer_runs())
    return ModelPlan(
        embedding=PartSpec("token", dict(vocab=cfg.vocab, hidden=W, name="embed")),
        embedding_prefix="",
        layers=tuple(layers),
        schedule=schedule,
        final_norm=_norm(W, eps),
        final_norm_prefix="final.norm",
        head=PartSpec("linear", dict(vocab=cfg.vocab, hidden=W, tied=False, name="head",
                                     scale=cfg.logit_scale, softcap=cfg.logit_softcap)),
        head_prefix="",
        vocab_size=cfg.vocab,
        max_position=NO_POSITION_LIMIT,
        stop_tokens=cfg.eos_token_ids(),
        stream_vectors=((LOOP_VECTORS, (cfg.passes(), W)),) if cfg.passes() else (),
        unread_tensors=tuple(unread) + (
            ((LOOP_VECTORS, (int(cfg.loop["times"]), W)),) if cfg.loop and not cfg.passes() else ()),
    )


register_architecture("Suvazen", SuvazenConfig, suvazen_plan, model_types=("suvazen",))
