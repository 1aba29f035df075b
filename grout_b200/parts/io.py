"""The two ends of the model: token embedding and output head."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import BuildContext, ParamSpec, Part, register_part
from .linear import Linear


class Embedding(Part):
    family = "embedding"

    def forward(self, tokens, step):
        raise NotImplementedError


@register_part("embedding", "token")
class TokenEmbedding(Embedding):
    """x[t] = E[ids[t]], no scaling (src/training.rs:278-282)."""

    def __init__(self, ctx: BuildContext, vocab: int, hidden: int, name: str = "weight"):
        super().__init__(ctx)
        self.vocab, self.hidden, self.name = int(vocab), int(hidden), name
        self.weight = None

    def param_specs(self):
        return {self.name: ParamSpec((self.vocab, self.hidden))}

    def load(self, params):
        self.weight = params[self.name].contiguous()

    def kernel_modules(self):
        return ("embed", "elementwise")

    def captures_prompts(self):
        return True

    def forward(self, tokens, step):
        x = ops.embed(self.weight, tokens)
        return ops.cast(x, self.ctx.dtype) if x.dtype != self.ctx.dtype else x


class Head(Part):
    family = "head"

    def forward(self, h):
        raise NotImplementedError


@register_part("head", "linear")
class LinearHead(Head):
    """logits = h W^T in 32-bit; W is the embedding table when ``tied``
    (src/training.rs:352-362).  With ``scale`` the logits are multiplied by it, and
    with ``softcap`` c they then become c * tanh(logit / c); both in 32-bit.
    ``name``: the weight's local name."""

    def __init__(self, ctx: BuildContext, vocab: int, hidden: int, tied: bool,
                 scale: Optional[float] = None, softcap: Optional[float] = None,
                 name: str = "weight"):
        super().__init__(ctx)
        self.vocab, self.hidden, self.tied = int(vocab), int(hidden), bool(tied)
        self.scale = float(scale) if scale is not None else 1.0
        self.softcap = float(softcap) if softcap else None
        self.name = name
        self.proj: Optional[Linear] = None

    def param_specs(self):
        return {} if self.tied else {self.name: ParamSpec((self.vocab, self.hidden))}

    def load(self, params):
        if not self.tied:
            self.proj = Linear(params[self.name], self.ctx.products)

    def tie(self, table: torch.Tensor) -> None:
        self.proj = Linear(table, self.ctx.products)   # shares the allocation (src/model.rs:1375-1377)

    def kernel_modules(self):
        mods = self.proj.kernel_modules() if self.proj else ()
        return mods + (("elementwise",) if self.scale != 1.0 or self.softcap else ())

    def captures_prompts(self):
        return True

    def forward(self, h):
        logits = self.proj(h, out_dtype=torch.float32)
        if self.scale != 1.0 or self.softcap:
            ops.scale_softcap_(logits, self.scale, self.softcap)
        return logits
