"""A gated linear recurrence behind a short causal convolution: the recurrent
block of Griffin (De et al., "Griffin: Mixing Gated Linear Recurrences with
Local Attention for Efficient Language Models").

Two branches of ``width`` numbers from the mixer's input h:
  g = gelu_tanh(W_y h + b_y)
  u = conv(W_x h + b_x)         per channel, ``taps`` long, causal
and, with u cut into ``blocks`` equal parts u_b and square matrices R_b, I_b:
  r = sigmoid(R_b u_b + b_r),  i = sigmoid(I_b u_b + b_i)
  a = exp(-decay * r * softplus(lam))
  S_t = a S_(t-1) + sqrt(1 - a^2) (i u_t),   S = 0 before the first token
  out = W_o (S g)
Between steps a request keeps S and the convolution's last ``taps`` - 1
inputs in its state slot, in 32-bit; everything after the first product is
32-bit until S g is rounded for the output product.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache.manager import StateNeed
from ..weights.loader import TensorSpec
from .base import Mixer
from .registry import register_mixer


class GatedRecurrence(Mixer):
    """params: ``hidden_size``, ``width``, ``blocks``, ``taps``, ``decay``
    (the constant in a's exponent, default 8), ``base`` (what the tensor
    names start with after the prefix, default "mix."; the tensors are y,
    y.b, x, x.b, conv, conv.b, ra, ra.b, ri, ri.b, lam, o)."""

    @classmethod
    def _base(cls, p, prefix):
        return prefix + (p.get("base") if p.get("base") is not None else "mix.")

    @classmethod
    def tensor_specs(cls, p, prefix):
        W, C, B, K = p["hidden_size"], p["width"], p["blocks"], p["taps"]
        bs = C // B
        b = cls._base(p, prefix)
        return {b + "y": TensorSpec((C, W)), b + "y.b": TensorSpec((C,)), b + "x": TensorSpec((C, W)),
                b + "x.b": TensorSpec((C,)), b + "conv": TensorSpec((C, K)), b + "conv.b": TensorSpec((C,)),
                b + "ra": TensorSpec((B, bs, bs)), b + "ra.b": TensorSpec((B, bs)),
                b + "ri": TensorSpec((B, bs, bs)), b + "ri.b": TensorSpec((B, bs)),
                b + "lam": TensorSpec((C,)), b + "o": TensorSpec((W, C))}

    @classmethod
    def cache_need(cls, p):
        return StateNeed((int(p["taps"]), int(p["width"])), "float32")

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        self.C, self.B, self.K = int(p["width"]), int(p["blocks"]), int(p["taps"])
        if self.C % self.B:
            raise ValueError(f"width {self.C} does not split into {self.B} equal blocks")
        self.bs = self.C // self.B
        self.decay = float(p.get("decay") if p.get("decay") is not None else 8.0)
        b = self._base(p, prefix)
        f32 = lambda n: tensors.get(b + n, torch.float32).contiguous()
        self.w_yx = torch.cat([tensors.get(b + "y", env.dtype), tensors.get(b + "x", env.dtype)], dim=0).contiguous()
        tensors.drop(b + "y", b + "x")
        self.yb, self.xb, self.taps, self.cb, self.lam = f32("y.b"), f32("x.b"), f32("conv"), f32("conv.b"), f32("lam")
        self.rb, self.ib = f32("ra.b").view(-1), f32("ri.b").view(-1)
        # both gates' matrices side by side, laid out for u_b @ [R_b^T | I_b^T]: [blocks, bs, 2 bs], 32-bit
        self.w_gates = torch.cat([f32("ra"), f32("ri")], dim=1).transpose(1, 2).contiguous()
        tensors.drop(b + "ra", b + "ri")
        self.w_in = self.w_yx
        self.w_o = tensors.get(b + "o", env.dtype)
        self.out_features = self.C

    def mix(self, x, batch, cache, writes=True, out=None, out_scale: float = 1.0, proj=None):
        """S g [T, width] times ``out_scale``, before the output product (into ``out`` if given).  The state
        advances by the step's tokens.  ``proj``: x times ``w_in``, if the caller has it already (as columns
        of a wider product)."""
        C, B, bs = self.C, self.B, self.bs
        if proj is None:
            proj = ops.linear(x, self.w_yx)                                    # [T, 2 C] = gate branch | input branch
        u = ops.recurrent_conv(proj, C, self.xb, self.taps, self.cb, cache.state, batch)
        gates = torch.bmm(u.view(-1, B, bs).transpose(0, 1), self.w_gates)     # [B, T, 2 bs] in true 32-bit
        return ops.recurrent_scan(proj, 0, C, self.yb, self.xb, u, gates, self.rb, self.ib, self.lam, self.decay,
                                  cache.state, batch, out, out_scale)

    def forward(self, x, batch, cache, writes=True):
        w_o = self.w_o if self.w_o.is_contiguous() else self.w_o.contiguous()     # a share of a stacked matrix
        return ops.linear(self.mix(x, batch, cache, writes), w_o)


register_mixer("gated_recurrence", GatedRecurrence)
