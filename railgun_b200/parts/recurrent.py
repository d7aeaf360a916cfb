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
32-bit until S g is rounded for the output product.  The gates' products
R_b u_b, I_b u_b are a batched library product: in 32-bit mode a true 32-bit
one; in bfloat16 mode, where the matrices are bfloat16 numbers anyway, u is
split into two bfloat16 numbers (u = hi + lo to 2^-17) and [hi | lo] is
multiplied with the matrix stacked twice on the tensor cores, accumulated in
32-bit, which is as good as the 32-bit product at a sixth of its time.
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

    # from this many rows of a step on (bfloat16) the gates' products run on the tensor cores: every step, since the
    # product from two bfloat16 halves is the faster one at 8 rows too (2.95 against 6.0 us) and prompts and
    # single tokens then share one arithmetic
    HALVES_MIN_ROWS = 1

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
        # in bfloat16, portions run the gates' products on the tensor cores with u as two bfloat16 numbers (hi + lo,
        # exact to 2^-17) against the matrices (which ARE bfloat16) twice, accumulated in 32-bit
        self.w_gates_halves = None
        if env.dtype == torch.bfloat16:
            w16 = self.w_gates.to(torch.bfloat16)
            if torch.equal(w16.float(), self.w_gates):
                self.w_gates_halves = torch.cat([w16, w16], dim=1).contiguous()        # [blocks, 2 bs, 2 bs]
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
        if self.w_gates_halves is not None and proj.shape[0] >= self.HALVES_MIN_ROWS:
            u, halves = ops.recurrent_conv(proj, C, self.xb, self.taps, self.cb, cache.state, batch, halves_blocks=B)
            gates = torch.bmm(halves.view(-1, B, 2 * bs).transpose(0, 1), self.w_gates_halves,
                              out_dtype=torch.float32)                             # [B, T, 2 bs], 32-bit sums
        else:
            u = ops.recurrent_conv(proj, C, self.xb, self.taps, self.cb, cache.state, batch)
            gates = torch.bmm(u.view(-1, B, bs).transpose(0, 1), self.w_gates)     # [B, T, 2 bs] in true 32-bit
        return ops.recurrent_scan(proj, 0, C, self.yb, self.xb, u, gates, self.rb, self.ib, self.lam, self.decay,
                                  cache.state, batch, out, out_scale)

    def forward(self, x, batch, cache, writes=True):
        w_o = self.w_o if self.w_o.is_contiguous() else self.w_o.contiguous()     # a share of a stacked matrix
        return ops.linear(self.mix(x, batch, cache, writes), w_o)


register_mixer("gated_recurrence", GatedRecurrence)
