"""The Sonalorn decoder as a plan.

Layers that normalise a sublayer's output only (the sublayers read the stream
as it is; the normalised output enters it times a learned per-channel scale); a
stream that starts as the norm of token embedding plus learned position vector;
mixers that are either a gated delta rule behind short convolutions or causal
attention without rotation, with normalised queries and keys, a query factor
that grows with the logarithm of the position and a sink of logit zero; dense
(gelu-tanh gate) or routed feed-forwards, the latter with clamped experts,
corrected scores, a choice restricted to the best groups and router outputs
that stand for "hand the input on".  A layer may run another layer's tensors on
a state of its own.  This file holds the checkpoint's tensor names and the order
of the parts; every size and constant comes from the configuration.

Tensor names: ``embed``, ``pos``, ``embed.norm``, ``final.norm``, ``head`` and
per layer i ``l<i>.norm1`` / ``norm2`` / ``ls1`` / ``ls2``; a delta mixer's
``l<i>.mix.{q,k,v}`` (+ ``.conv``), ``b``, ``a``, ``A_log``, ``dt_bias``, ``g``,
``norm``, ``o``; an attention mixer's ``l<i>.mix.{q,k,v,o}``, ``q.norm``,
``k.norm``; ``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.e<j>.{gate,up,down}``,
``router``, ``correction``.
"""
from __future__ import annotations

from ..config import SonalornConfig, register_architecture
from ..parts.base import PartSpec
from ..parts.plan import LayerPlan, ModelPlan, ScheduleEntry

SINK_LOGIT = 0.0            # the design's softmax has exp(0) in its denominator
UNIT_EPS = 1e-6             # under the root when q and k of the delta rule are made unit vectors
EXPERT_GATE_SLOPE = 1.702   # g * sigmoid(1.702 g) in an expert


def _rms(dim: int, eps: float, name: str) -> PartSpec:
    return PartSpec("rmsnorm", dict(dim=dim, eps=eps, name=name))


def _mixer(kind: str, width: int, m: dict, eps: float) -> PartSpec:
    if kind == "delta":
        return PartSpec("gated_delta", dict(
            hidden=width, n_heads=m["heads"], n_kv_heads=m["kv_heads"], key_dim=m["dim"],
            value_dim=m["vdim"], conv_taps=m["conv"], norm_eps=eps, unit_eps=UNIT_EPS))
    qt = m.get("q_temp")
    return PartSpec("gqa_attention", dict(
        hidden=width, n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"],
        v_head_dim=m["vdim"], position=PartSpec("none", {}), qk_norm_eps=eps,
        scale=float(m["scale"]), sink_logit=SINK_LOGIT,
        q_temp=(float(qt["coef"]), int(qt["every"])) if qt else None,
        names={"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"}))


def _feedforward(width: int, mlp: dict) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", dict(hidden=width, intermediate=int(mlp["ff"]),
                                          activation="gelu_tanh",
                                          names={"gate": "gate", "up": "up", "down": "down"}))
    r, ex = mlp["router"], mlp["expert"]
    g = r.get("groups")
    return PartSpec("routed_experts", dict(
        hidden=width, intermediate=int(ex["ff"]), n_experts=int(r["experts"]),
        n_identity=int(r.get("identity", 0)), top=int(r["top"]),
        n_groups=int(g["count"]) if g else 1, keep_groups=int(g["keep"]) if g else 1,
        limit=float(ex["limit"]), gate_slope=EXPERT_GATE_SLOPE))


def sonalorn_plan(cfg: SonalornConfig) -> ModelPlan:
    W, eps = cfg.width, float(cfg.norm["eps"])
    own = [i for i in range(len(cfg.layers)) if cfg.weights_layer(i) == i]
    index = {layer: n for n, layer in enumerate(own)}
    layers = []
    for i in own:
        layer = cfg.layers[i]
        args = dict(mixer=_mixer(layer["type"], W, layer["mixer"], eps), norm1=_rms(W, eps, ""),
                    scale1="ls1")
        if layer.get("mlp") is not None:
            args.update(feedforward=_feedforward(W, layer["mlp"]), norm2=_rms(W, eps, ""),
                        scale2="ls2")
        layers.append(LayerPlan(PartSpec("postnorm", args), f"l{i}.", {
            "norm1": "norm1", "norm2": "norm2", "mixer": "mix.", "feedforward": "mlp."}))
    # a layer that runs another's tensors is one more run of that layer, with a
    # cache or state of its own
    schedule = tuple(ScheduleEntry(index[cfg.weights_layer(i)]) for i in range(len(cfg.layers)))
    return ModelPlan(
        embedding=PartSpec("token_positional", dict(
            vocab=cfg.vocab, hidden=W, max_positions=cfg.max_positions, eps=eps,
            names={"token": "embed", "position": "pos", "norm": "embed.norm"})),
        embedding_prefix="",
        layers=tuple(layers),
        schedule=schedule,
        final_norm=_rms(W, eps, ""),
        final_norm_prefix="final.norm",
        head=PartSpec("linear", dict(vocab=cfg.vocab, hidden=W, tied=False, name="head")),
        head_prefix="",
        vocab_size=cfg.vocab,
        max_position=cfg.max_positions,
        stop_tokens=cfg.eos_token_ids(),
    )


register_architecture("Sonalorn", SonalornConfig, sonalorn_plan, model_types=("sonalorn",))
