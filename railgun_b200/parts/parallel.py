"""Mixers side by side: every branch reads the same input, and the result is
the sum of the branches' outputs, each times a constant.

A branch is any mixer that can hand out what goes into its output product
(``mix(x, batch, cache, writes, out, out_scale)`` -> [T, out_features], and
``w_o`` [hidden, out_features]).  The branches write side by side into one
buffer, already multiplied by their constants in 32-bit before the one
rounding, and ONE product with the output matrices side by side gives
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
            if not hasattr(part, "mix") or not hasattr(part, "w_o"):
                raise ValueError(f"{type(part).__name__} cannot be a branch of 'parallel': it has no mix() and w_o")
        self.w_o = torch.cat([part.w_o for part in self.parts], dim=1).contiguous()
        self.widths = [int(part.out_features) for part in self.parts]
        self.graph_safe = all(getattr(part, "graph_safe", True) for part in self.parts)

    def forward(self, x, batch, cache, writes=True):
        T = x.shape[0]
        z = torch.empty((T, sum(self.widths)), dtype=self.env.dtype, device=self.w_o.device)
        off = 0
        for part, c, n, view in zip(self.parts, self.scales, self.widths, cache.parts):
            part.mix(x, batch, view, writes, out=z[:, off:off + n], out_scale=c)
            off += n
        return ops.linear(z, self.w_o)


register_mixer("parallel", Parallel)
