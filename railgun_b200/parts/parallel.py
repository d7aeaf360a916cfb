"""Mixers side by side: every branch reads the same input, and the result is
the sum of the branches' outputs, each times a constant.

A branch is any mixer that can hand out what goes into its output product
(``mix(x, batch, cache, writes, out, out_scale, proj)`` -> [T, out_features],
``w_o`` [hidden, out_features]) and takes its first product from outside
(``w_in`` [in_features, hidden]; ``proj`` = x w_in^T).  ONE product with the
branches' input matrices stacked feeds them all; they write side by side
into one buffer, already multiplied by their constants in 32-bit before the
one rounding, and ONE product with the output matrices side by side gives
sum_b c_b W_o,b z_b.  What the branches keep between steps is asked for as a
tuple of needs, one per branch.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer
from .registry import MIXERS, register_mixer


class Parallel(Mixer):
    """params: ``branches``: ((PartSpec of a mixer, constant), ...)."""

    @classmethod
    def tensor_specs(cls, p, prefix):
        out = {}
        for spec, _ in p["branches"]:
            out.update(MIXERS.get(spec.kind).tensor_specs(spec.params, prefix))
        return out

    @classmethod
    def cache_need(cls, p):
        return tuple(MIXERS.get(spec.kind).cache_need(spec.params) for spec, _ in p["branches"])

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        self.parts = [MIXERS.get(spec.kind)(spec.params, prefix, env, tensors) for spec, _ in p["branches"]]
        self.scales = [float(c) for _, c in p["branches"]]
        for part in self.parts:
            if not all(hasattr(part, a) for a in ("mix", "w_o", "w_in")):
                raise ValueError(f"{type(part).__name__} cannot be a branch of 'parallel': it has no mix(), w_in and w_o")
        self.w_in = torch.cat([part.w_in for part in self.parts], dim=0).contiguous()
        self.w_o = torch.cat([part.w_o for part in self.parts], dim=1).contiguous()
        self.widths = [int(part.out_features) for part in self.parts]
        self.in_widths = [int(part.w_in.shape[0]) for part in self.parts]
        # the stacked matrices are the ones that are kept: the branches see their share of them
        at = off = 0
        for part, n_in, n in zip(self.parts, self.in_widths, self.widths):
            part.w_in = self.w_in[at:at + n_in]
            part.w_o = self.w_o[:, off:off + n]
            for name in ("w_qkv", "w_yx"):
                if hasattr(part, name):
                    setattr(part, name, part.w_in)
            at += n_in
            off += n
        self.graph_safe = all(getattr(part, "graph_safe", True) for part in self.parts)

    def forward(self, x, batch, cache, writes=True):
        T = x.shape[0]
        proj = ops.linear(x, self.w_in)
        z = torch.empty((T, sum(self.widths)), dtype=self.env.dtype, device=self.w_o.device)
        off = at = 0
        for part, c, n, n_in, view in zip(self.parts, self.scales, self.widths, self.in_widths, cache.parts):
            part.mix(x, batch, view, writes, out=z[:, off:off + n], out_scale=c, proj=proj[:, at:at + n_in])
            off += n
            at += n_in
        return ops.linear(z, self.w_o)


register_mixer("parallel", Parallel)
