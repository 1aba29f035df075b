"""Configuration of the Sonalorn decoder.

The file names the design under ``architecture`` and describes the model layer
by layer: ``layers`` is a list of objects ``{"type", "mixer", "mlp"}`` (``mlp``
null: the layer has no feed-forward).  A layer with ``weights_of: j`` has no
tensors of its own and runs layer j's (its sizes and constants are layer j's), on
a cache or state of its own.  Nothing
that the arithmetic needs is defaulted: a constant that is absent stands for a
term that is absent (no ``q_temp``: queries are not scaled by position; no
``groups``: every expert can be chosen).

    vocab, width, max_positions   sizes of the two embedding tables and of the stream
    norm.eps                      epsilon of every RMS norm
    layers[i].type                "delta" | "attention"
    layers[i].mixer  (delta)      heads, kv_heads, dim, vdim, conv (taps)
    layers[i].mixer  (attention)  heads, kv_heads, dim, vdim, scale, q_temp.{coef, every}
    layers[i].mlp                 {"kind": "dense", "ff"} or {"kind": "moe",
                                  "expert": {"ff", "limit"}, "router": {"experts", "top",
                                  "identity", "groups": {"count", "keep"}}}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ModelConfig

_MIXER_TYPES = ("delta", "attention")
_MLP_KINDS = ("dense", "moe")


def _number(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def _positive_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool) and v > 0


def _count(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool) and v >= 0


@dataclass(frozen=True)
class SonalornConfig(ModelConfig):
    vocab: int
    width: int
    max_positions: int
    layers: Tuple[dict, ...]
    norm: dict
    architecture: str = "Sonalorn"
    eos_token_id: Optional[int] = None

    def validate(self):
        for key in ("vocab", "width", "max_positions"):
            if not _positive_int(getattr(self, key)):
                yield f"'{key}' must be a positive integer, found {getattr(self, key)!r}"
        if not _number(self.norm.get("eps")) or not self.norm["eps"] > 0:
            yield f"'norm.eps' must be a positive number, found {self.norm.get('eps')!r}"
        if not self.layers:
            yield "'layers' is empty"
        for i, layer in enumerate(self.layers):
            yield from self._layer_problems(i, layer)

    def _layer_problems(self, i, layer):
        where = f"layers[{i}]"
        if not isinstance(layer, dict):
            yield f"{where} is not an object"
            return
        if layer.get("type") not in _MIXER_TYPES:
            yield f"{where}.type={layer.get('type')!r}: this design has {list(_MIXER_TYPES)}"
            return
        src = layer.get("weights_of")
        if src is not None:
            if not _count(src) or src >= len(self.layers) or src == i or \
                    not isinstance(self.layers[src], dict) or "weights_of" in self.layers[src]:
                yield f"{where}.weights_of={src!r} must name another layer that has tensors of its own"
            elif layer["type"] != self.layers[src].get("type"):
                yield f"{where} uses the weights of layer {src}, which is of another type"
            return
        m = layer.get("mixer")
        if not isinstance(m, dict):
            yield f"{where}.mixer is missing"
            return
        for key in ("heads", "kv_heads", "dim", "vdim"):
            if not _positive_int(m.get(key)):
                yield f"{where}.mixer.{key} must be a positive integer, found {m.get(key)!r}"
                return
        if m["heads"] % m["kv_heads"]:
            yield f"{where}.mixer: {m['heads']} heads cannot share {m['kv_heads']} kv heads"
        if layer["type"] == "delta":
            if not _positive_int(m.get("conv")):
                yield f"{where}.mixer.conv (taps) must be a positive integer, found {m.get('conv')!r}"
        else:
            if not _number(m.get("scale")):
                yield f"{where}.mixer.scale must be a number, found {m.get('scale')!r}"
            qt = m.get("q_temp")
            if qt is not None and not (isinstance(qt, dict) and _number(qt.get("coef"))
                                       and _positive_int(qt.get("every"))):
                yield f"{where}.mixer.q_temp needs a number 'coef' and a positive integer 'every', found {qt!r}"
        yield from self._mlp_problems(where, layer.get("mlp"))

    def _mlp_problems(self, where, mlp):
        if mlp is None:
            return
        if not isinstance(mlp, dict) or mlp.get("kind") not in _MLP_KINDS:
            yield f"{where}.mlp.kind={mlp!r}: this design has {list(_MLP_KINDS)}"
            return
        if mlp["kind"] == "dense":
            if not _positive_int(mlp.get("ff")):
                yield f"{where}.mlp.ff must be a positive integer, found {mlp.get('ff')!r}"
            return
        ex, r = mlp.get("expert"), mlp.get("router")
        if not (isinstance(ex, dict) and _positive_int(ex.get("ff")) and _number(ex.get("limit"))
                and ex["limit"] > 0):
            yield f"{where}.mlp.expert needs a positive integer 'ff' and a positive 'limit', found {ex!r}"
        if not (isinstance(r, dict) and _positive_int(r.get("experts")) and _positive_int(r.get("top"))
                and _count(r.get("identity", 0))):
            yield f"{where}.mlp.router needs positive integers 'experts' and 'top', found {r!r}"
            return
        n_all = r["experts"] + r.get("identity", 0)
        if r["top"] > n_all:
            yield f"{where}.mlp.router.top={r['top']} exceeds its {n_all} outputs"
        g = r.get("groups")
        if g is not None:
            if not (isinstance(g, dict) and _positive_int(g.get("count")) and _positive_int(g.get("keep"))
                    and g["keep"] <= g["count"]):
                yield f"{where}.mlp.router.groups needs 'count' >= 'keep' >= 1, found {g!r}"
            elif n_all % g["count"]:
                yield f"{where}.mlp.router: {n_all} outputs do not form {g['count']} equal groups"
            elif r["top"] > g["keep"] * (n_all // g["count"]):
                yield f"{where}.mlp.router: top={r['top']} exceeds the experts of {g['keep']} groups"

    # ---- derived -------------------------------------------------------
    def weights_layer(self, i: int) -> int:
        """The layer whose tensors layer i runs."""
        return int(self.layers[i].get("weights_of", i))

    def eos_token_ids(self) -> Tuple[int, ...]:
        return () if self.eos_token_id is None else (int(self.eos_token_id),)
