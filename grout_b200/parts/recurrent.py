"""Mixers that carry a state of fixed size from token to token instead of keys
and values.  Their cache need is a ``StateSpec``: one row of 32-bit floats per
sequence and layer, zero when the sequence starts; the rows of a sequence are
walked in order (``step.cu_q``), so the state after a prompt is the same
whether its tokens came in one step, in portions or one by one.
"""
from __future__ import annotations

import torch

from ..cache.spec import StateSpec
from ..kernels import ops
from .base import BuildContext, ParamSpec, register_part
from .linear import Linear
from .mixer import Mixer


@register_part("mixer", "gated_delta")
class GatedDelta(Mixer):
    """The gated delta rule.  With h the mixer's input,

        q = Wq h, k = Wk h  (n_kv_heads x key_dim),  v = Wv h  (n_heads x value_dim)
        each through a causal convolution over time of ``conv_taps`` taps per channel
        (no bias, zeros before the sequence's start; the last tap is the current
        token's), then silu;  q and k made unit vectors per head,
        x / sqrt(sum(x^2) + unit_eps), q also times key_dim^(-1/2)
        beta = sigmoid(Wb h),  g = exp(-exp(A_log) softplus(Wa h + dt_bias))   per head
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q            per head
        y = Wo [ o / sqrt(mean(o^2) + norm_eps) * w * silu(Wg h) ]

    Head i reads q and k of kv head i // (n_heads / n_kv_heads); the norm's weight
    w [value_dim] is shared by the heads.  S [key_dim, value_dim] starts at zero and
    is kept, with the last ``conv_taps - 1`` inputs of the convolutions, per
    sequence.  The six projections are one product, which leaves 32-bit sums; all
    that follows up to y is 32-bit whatever the activation type.  ``names``
    replaces local tensor names (keys q, k, v, q_conv, k_conv, v_conv, b, a, A_log,
    dt_bias, g, norm, o)."""

    NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv",
             "v_conv": "v.conv", "b": "b", "a": "a", "A_log": "A_log", "dt_bias": "dt_bias",
             "g": "g", "norm": "norm", "o": "o"}

    def __init__(self, ctx: BuildContext, hidden: int, n_heads: int, n_kv_heads: int, key_dim: int,
                 value_dim: int, conv_taps: int, norm_eps: float, unit_eps: float = 1e-6,
                 names=None):
        super().__init__(ctx)
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads cannot share {n_kv_heads} kv heads")
        if conv_taps < 1:
            raise ValueError("a convolution has at least one tap")
        self.hidden, self.H, self.G = int(hidden), int(n_heads), int(n_kv_heads)
        self.dk, self.dv, self.taps = int(key_dim), int(value_dim), int(conv_taps)
        self.norm_eps, self.unit_eps = float(norm_eps), float(unit_eps)
        self.names = dict(self.NAMES, **(names or {}))
        self.proj = self.o = None
        self.conv_w = self.a_log = self.dt_bias = self.norm_w = None

    def param_specs(self):
        W, H, G, dk, dv, nm = self.hidden, self.H, self.G, self.dk, self.dv, self.names
        return {nm["q"]: ParamSpec((G * dk, W)), nm["k"]: ParamSpec((G * dk, W)),
                nm["v"]: ParamSpec((H * dv, W)), nm["g"]: ParamSpec((H * dv, W)),
                nm["b"]: ParamSpec((H, W)), nm["a"]: ParamSpec((H, W)),
                nm["q_conv"]: ParamSpec((G * dk, self.taps), "vector"),
                nm["k_conv"]: ParamSpec((G * dk, self.taps), "vector"),
                nm["v_conv"]: ParamSpec((H * dv, self.taps), "vector"),
                nm["A_log"]: ParamSpec((H,), "offset"), nm["dt_bias"]: ParamSpec((H,), "offset"),
                nm["norm"]: ParamSpec((dv,), "vector"), nm["o"]: ParamSpec((W, H * dv))}

    def load(self, params):
        nm = self.names
        ws = [params[nm[k]] for k in ("q", "k", "v", "g", "b", "a")]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("the projections of one mixer must be stored in one dtype to be fused")
        self.proj = Linear(torch.cat(ws, dim=0), self.ctx.products)
        self.o = Linear(params[nm["o"]], self.ctx.products)
        # what enters the recurrence is 32-bit whatever the checkpoint stores
        f32 = lambda t: t.float().contiguous()
        self.conv_w = f32(torch.cat([params[nm[k]] for k in ("q_conv", "k_conv", "v_conv")], dim=0))
        self.a_log, self.dt_bias = f32(params[nm["A_log"]]), f32(params[nm["dt_bias"]])
        self.norm_w = f32(params[nm["norm"]])

    def kernel_modules(self):
        return ("delta",) + self.proj.kernel_modules() + self.o.kernel_modules()

    def cache_spec(self):
        return StateSpec((ops.delta_state_floats(self.H, self.G, self.dk, self.dv, self.taps),),
                         torch.float32)

    def captures_prompts(self):
        return True

    def forward(self, x, step, cache):
        if cache is None or tuple(cache.spec.shape) != tuple(self.cache_spec().shape):
            raise ValueError(f"the gated delta rule was given the cache "
                             f"{None if cache is None else cache.spec}")
        proj = self.proj(x, out_dtype=torch.float32)
        y = ops.delta_forward(proj, cache.state, self.conv_w, self.a_log, self.dt_bias,
                              self.norm_w, H=self.H, G=self.G, dk=self.dk, dv=self.dv,
                              taps=self.taps, unit_eps=self.unit_eps, norm_eps=self.norm_eps,
                              token_seq=step.token_seq, cu_q=step.cu_q, slots=step.slots,
                              dtype=self.ctx.dtype, max_rows=step.max_q_len)
        return self.o(y, partial_ok=True)
