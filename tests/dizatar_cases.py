"""Small Dizatar configurations for the tests, their model folders and plain logits.

Every case differs from the others in every size; together they cover layers
that are unlike one another, a layer without a feed-forward, a feed-forward
without identity experts or without a shared expert, one choice per token,
all router outputs chosen, one head, a looped span of one layer, of all
layers, run once, and no loop at all.
"""
from __future__ import annotations

import math
import tempfile
from pathlib import Path

import numpy as np


def mixer(heads, dim, rot_dim, vdim, kv_rank, base=10000.0, scale=None):
    return dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank,
                rot=dict(base=base, dims=rot_dim), scale=scale or 1.0 / math.sqrt(dim + rot_dim))


def moe(experts, identity, top, ff, shared):
    return dict(kind="moe", router=dict(experts=experts, identity=identity, top=top), expert=dict(ff=ff),
                shared=dict(ff=shared) if shared else None)


def layer(mix, mlp):
    return dict(type="latent_attention", mixer=mix, mlp=mlp)


# P: three unlike layers (odd head counts, sizes that are no multiple of 16, the middle one without a
#    feed-forward, the last one with one choice and neither identity nor shared expert), the first two looped
#    three times; a residual multiplier above 1.
CASE_P = dict(
    architecture="Dizatar", width=48, vocab=211, norm=dict(eps=1e-5), residual_mult=1.3, logit_softcap=8.0,
    loop=dict(start=0, stop=2, times=3),
    layers=[layer(mixer(3, 16, 8, 24, 40, base=100.0), moe(5, 2, 2, 24, 16)),
            layer(mixer(2, 8, 16, 8, 24, base=1000.0, scale=0.3), None),
            layer(mixer(4, 32, 4, 16, 16, base=50.0), moe(3, 0, 1, 40, None))])
# Q: sizes in multiples of 16 (the tensor-core kernels), a looped span of one layer, four choices of nine.
CASE_Q = dict(
    architecture="Dizatar", width=128, vocab=320, norm=dict(eps=1e-6), residual_mult=0.5, logit_softcap=30.0,
    loop=dict(start=1, stop=2, times=2),
    layers=[layer(mixer(4, 32, 16, 32, 64), moe(8, 1, 4, 64, 96)) for _ in range(3)])
# S: one head, one choice, every size equal, the span of all layers run once.
CASE_S = dict(
    architecture="Dizatar", width=32, vocab=64, norm=dict(eps=1e-3), residual_mult=1.0, logit_softcap=3.0,
    loop=dict(start=0, stop=2, times=1),
    layers=[layer(mixer(1, 16, 16, 16, 16, base=10.0), moe(2, 1, 1, 16, 16)),
            layer(mixer(1, 16, 16, 16, 16, base=10.0), moe(1, 2, 3, 16, None))])
# N: no loop; a wide latent against narrow heads, 16 heads.
CASE_N = dict(
    architecture="Dizatar", width=64, vocab=100, norm=dict(eps=1e-6), residual_mult=0.8, logit_softcap=50.0,
    layers=[layer(mixer(16, 16, 32, 16, 128, base=500000.0), moe(4, 4, 3, 32, 48)),
            layer(mixer(16, 16, 32, 16, 128, base=500000.0), None)])

# M: six heads of 48 + 32 over a latent of 80 with values of 40 (every size a different multiple of 8), one
#    layer looped twice and one behind it; all eight router outputs chosen (no ties: bfloat16 is held to the
#    tight bound everywhere, here for prompts in the expanded form).
CASE_M = dict(
    architecture="Dizatar", width=72, vocab=150, norm=dict(eps=1e-5), residual_mult=0.9, logit_softcap=20.0,
    loop=dict(start=0, stop=1, times=2),
    layers=[layer(mixer(6, 48, 32, 40, 80, base=3000.0), moe(6, 2, 8, 40, 24)),
            layer(mixer(6, 48, 32, 40, 80, base=3000.0), None)])

# A: heads of 40 + 16 (no multiple of 16, so prompts stay in the compressed form) over a latent of 64 + 16 that
#    the tensor-core kernel takes; every router output is chosen in both layers, so no choice is ever near a tie
#    and bfloat16 is held to the tight bound at every position.
CASE_A = dict(
    architecture="Dizatar", width=56, vocab=90, norm=dict(eps=1e-6), residual_mult=1.1, logit_softcap=12.0,
    loop=dict(start=1, stop=2, times=3),
    layers=[layer(mixer(4, 40, 16, 24, 64, base=700.0), moe(3, 2, 5, 24, 40)),
            layer(mixer(4, 40, 16, 24, 64, base=700.0), moe(2, 1, 3, 32, None))])

CASES = {"P": (CASE_P, 3, 8), "Q": (CASE_Q, 5, 16), "S": (CASE_S, 7, 4), "N": (CASE_N, 9, 32),
         "M": (CASE_M, 11, 16), "A": (CASE_A, 13, 8)}                                          # config, seed, page

_made: dict = {}
_plain: dict = {}


def model_dir(name: str, std: float = 0.1) -> Path:
    key = (name, std)
    if key not in _made:
        from railgun_b200.config.dizatar import DizatarConfig
        from railgun_b200.weights.random_init import write_random_model
        cfg, seed, _ = CASES[name]
        d = Path(tempfile.mkdtemp(prefix=f"rg_dizatar_{name}_"))
        write_random_model(DizatarConfig.from_dict(cfg), seed, d, std=std)
        _made[key] = d
    return _made[key]


def plain_model(name: str):
    if name not in _plain:
        from plain_dizatar import PlainDizatar
        _plain[name] = PlainDizatar(model_dir(name))
    return _plain[name]


def prompts(vocab: int, lengths, seed: int):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=n).tolist() for n in lengths]
