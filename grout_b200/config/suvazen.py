"""Configuration of the Suvazen decoder.

The file names the design under ``architecture`` and describes the model layer
by layer: ``layers`` is a list of objects ``{"type", "mixer", "mlp"}``, where
``mixer`` holds the sizes and constants of that layer's mixer and ``mlp`` those
of its feed-forward (null: the layer has none).  Nothing is defaulted that the
arithmetic needs: a constant that is absent stands for a term that is absent
(no ``softcap``: scores are not capped; no ``mask``: every earlier key is seen;
no ``rot``: no rotation; no ``loop``: every layer runs once).

    vocab, width              sizes of the embedding and of the residual stream
    norm.eps                  epsilon of every layer norm
    residual_mult             factor of every sublayer's normalised output
    layers[i].type            "attention"
    layers[i].mixer           heads, kv_heads, dim, vdim, scale, softcap,
                              mask.size, rot.{dims, base, scaling.{factor, low,
                              high, original}}
    layers[i].mlp             {"kind": "dense", "ff": rows of the up projection}
    loop.{start, stop, times} layers start..stop-1 run ``times`` times in a row
    logit_scale, logit_softcap
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ModelConfig

_MIXER_TYPES = ("attention",)
_MLP_KINDS = ("dense",)


def _number(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def _positive_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool) and v > 0


@dataclass(frozen=True)
class SuvazenConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[dict, ...]
    norm: dict
    architecture: str = "Suvazen"
    residual_mult: float = 1.0
    loop: Optional[dict] = None
    logit_scale: Optional[float] = None
    logit_softcap: Optional[float] = None
    eos_token_id: Optional[int] = None

    def validate(self):
        for key in ("vocab", "width"):
            if not _positive_int(getattr(self, key)):
                yield f"'{key}' must be a positive integer, found {getattr(self, key)!r}"
        if not _number(self.norm.get("eps")) or not self.norm["eps"] > 0:
            yield f"'norm.eps' must be a positive number, found {self.norm.get('eps')!r}"
        if not self.layers:
            yield "'layers' is empty"
        for i, layer in enumerate(self.layers):
            yield from self._layer_problems(i, layer)
        yield from self._loop_problems()
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            yield f"'logit_softcap' must be positive, found {self.logit_softcap!r}"

    def _layer_problems(self, i, layer):
        where = f"layers[{i}]"
        if not isinstance(layer, dict):
            yield f"{where} is not an object"
            return
        if layer.get("type") not in _MIXER_TYPES:
            yield f"{where}.type={layer.get('type')!r}: this design has {list(_MIXER_TYPES)}"
            return
        m = layer.get("mixer")
        if not isinstance(m, dict):
            yield f"{where}.mixer is missing"
            return
        for key in ("heads", "kv_heads", "dim"):
            if not _positive_int(m.get(key)):
                yield f"{where}.mixer.{key} must be a positive integer, found {m.get(key)!r}"
                return
        if m["heads"] % m["kv_heads"]:
            yield f"{where}.mixer: {m['heads']} heads cannot share {m['kv_heads']} kv heads"
        if m.get("vdim", m["dim"]) != m["dim"]:
            yield (f"{where}.mixer: vdim={m.get('vdim')!r} differs from dim={m['dim']}, but the "
                   f"values are the keys")
        if not _number(m.get("scale")):
            yield f"{where}.mixer.scale must be a number, found {m.get('scale')!r}"
        if m.get("softcap") is not None and not (_number(m["softcap"]) and m["softcap"] > 0):
            yield f"{where}.mixer.softcap must be positive, found {m['softcap']!r}"
        mask = m.get("mask")
        if mask is not None and not (isinstance(mask, dict) and _positive_int(mask.get("size"))):
            yield f"{where}.mixer.mask.size must be a positive integer, found {mask!r}"
        rot = m.get("rot")
        if rot is not None:
            if not isinstance(rot, dict) or not _positive_int(rot.get("dims")) or rot["dims"] % 2 \
                    or rot["dims"] > m["dim"]:
                yield f"{where}.mixer.rot.dims must be even and at most dim, found {rot!r}"
            elif not (_number(rot.get("base")) and rot["base"] > 0):
                yield f"{where}.mixer.rot.base must be positive, found {rot.get('base')!r}"
            sc = rot.get("scaling") if isinstance(rot, dict) else None
            if sc is not None:
                bad = [k for k in ("factor", "low", "high", "original")
                       if not (isinstance(sc, dict) and _number(sc.get(k)) and sc[k] > 0)]
                if bad:
                    yield f"{where}.mixer.rot.scaling needs positive {bad}"
                elif sc["high"] == sc["low"]:
                    yield f"{where}.mixer.rot.scaling: high and low are equal"
        mlp = layer.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind") not in _MLP_KINDS:
                yield f"{where}.mlp.kind={mlp!r}: this design has {list(_MLP_KINDS)}"
            elif not _positive_int(mlp.get("ff")):
                yield f"{where}.mlp.ff must be a positive integer, found {mlp.get('ff')!r}"

    def _loop_problems(self):
        lp = self.loop
        if lp is None:
            return
        if not isinstance(lp, dict) or not all(
                isinstance(lp.get(k), int) and not isinstance(lp.get(k), bool)
                for k in ("start", "stop", "times")):
            yield f"'loop' needs integer start, stop and times, found {lp!r}"
            return
        if not 0 <= lp["start"] <= lp["stop"] <= len(self.layers):
            yield f"'loop' spans layers {lp['start']}..{lp['stop']} of {len(self.layers)}"
        if lp["times"] < 1:
            yield f"'loop.times' must be at least 1, found {lp['times']}"

    # ---- derived -------------------------------------------------------
    def passes(self) -> int:
        """How often the looped layers run (0: there is no loop)."""
        lp = self.loop
        return int(lp["times"]) if lp and lp["stop"] > lp["start"] else 0

    def layer_runs(self):
        """The order of the layer runs: (layer, pass) with ``pass`` the number of
        the pass that this run opens, None for every other run."""
        n = len(self.layers)
        if not self.passes():
            return [(i, None) for i in range(n)]
        a, b = self.loop["start"], self.loop["stop"]
        runs = [(i, None) for i in range(a)]
        for t in range(self.passes()):
            runs += [(i, t if i == a else None) for i in range(a, b)]
        return runs + [(i, None) for i in range(b, n)]

    def eos_token_ids(self) -> Tuple[int, ...]:
        return () if self.eos_token_id is None else (int(self.eos_token_id),)
