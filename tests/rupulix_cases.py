"""Small Rupulix configurations for the tests, their model folders and plain logits.

The cases differ from one another in every size.  Together they cover: both
kinds of layer in different orders, a layer without a feed-forward, two,
three and four copies of the residual stream, one copy, and none (the plain
pre-norm block); a looped span of one layer, of several, of all, run once, and
no loop; windows of 1, a few, and none; one head, one key/value head per
head, several heads per key/value head; rotation of part of a head; values
larger and smaller than keys; a recurrence as wide as the model, narrower and
wider; blocks of one channel and one block; convolutions of one to five taps.

Weights are random but not all alike: decays near 1 (so that the recurrence
remembers), sinks and mixing matrices far from neutral, hyper-connection
coefficients that are no identity.
"""
from __future__ import annotations

import json
import math
import tempfile
from pathlib import Path

import numpy as np


def latent(heads, dim, rot_dim, vdim, kv_rank, base=10000.0, window=0, scale=None):
    d = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, rot=dict(base=base, dims=rot_dim),
             scale=scale or 1.0 / math.sqrt(dim + rot_dim))
    if window:
        d["mask"] = dict(size=window)
    return dict(type="latent_attention", mixer=d)


def parallel(heads, kv_heads, dim, vdim, rot_dims, width, blocks, conv, base=10000.0, left_scale=0.7, right_scale=0.4,
             scale=None):
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, rot=dict(base=base, dims=rot_dims),
                scale=scale or 1.0 / math.sqrt(dim))
    return dict(type="parallel", mixer=dict(left=left, right=dict(width=width, blocks=blocks, conv=conv),
                                            left_scale=left_scale, right_scale=right_scale))


def layer(mix, ff):
    return dict(mix, mlp=dict(kind="dense", ff=ff) if ff else None)


# H: two copies; a windowed latent layer, two unlike parallel layers (part of the head rotated; values smaller and
#    larger than keys; recurrences narrower than and as wide as the model), the middle layer without feed-forward;
#    the first two layers looped three times.
CASE_H = dict(
    architecture="Rupulix", width=64, vocab=200, norm=dict(eps=1e-5), streams=2, logit_scale=0.7,
    loop=dict(start=0, stop=2, times=3),
    layers=[layer(latent(3, 16, 8, 24, 40, base=100.0, window=9), 96),
            layer(parallel(4, 2, 16, 8, 8, 48, 3, 3, base=1000.0), None),
            layer(parallel(2, 1, 24, 32, 24, 64, 1, 2, base=50.0, left_scale=1.2, right_scale=0.9), 40)])
# J: no copies (plain residual additions), no loop; every head its own key/value head; blocks of one channel and
#    a convolution of one tap; a latent layer with one head and no window; logits scaled up.
CASE_J = dict(
    architecture="Rupulix", width=96, vocab=130, norm=dict(eps=1e-6), logit_scale=2.0,
    layers=[layer(parallel(6, 6, 16, 16, 16, 96, 96, 1, base=500.0), 64),
            layer(latent(1, 32, 16, 16, 16, base=10.0), 128),
            layer(parallel(3, 1, 8, 40, 4, 120, 5, 5, left_scale=0.3, right_scale=1.5), None)])
# K: one copy with hyper-connection coefficients; a window of one (a token sees only itself) and a window longer than
#    any prompt; the span of all layers run once.
CASE_K = dict(
    architecture="Rupulix", width=32, vocab=64, norm=dict(eps=1e-3), streams=1, logit_scale=1.0,
    loop=dict(start=0, stop=3, times=1),
    layers=[layer(latent(2, 8, 8, 8, 8, base=10.0, window=1), 32),
            layer(parallel(1, 1, 16, 16, 16, 32, 2, 2), 16),
            layer(latent(4, 8, 4, 16, 24, window=1000), None)])
# L: four copies; sizes in multiples of 16 with prompts of several hundred tokens; a looped span of two layers.
CASE_L = dict(
    architecture="Rupulix", width=128, vocab=320, norm=dict(eps=1e-6), streams=4, logit_scale=0.25,
    loop=dict(start=1, stop=3, times=2),
    layers=[layer(parallel(4, 2, 32, 64, 32, 128, 2, 5, base=50000.0), 192),
            layer(latent(4, 32, 16, 32, 64, base=100000.0, window=50), 192),
            layer(parallel(8, 2, 16, 16, 8, 64, 4, 3, base=300.0), 256),
            layer(latent(2, 64, 32, 64, 96, window=130), 64)])
# T: three copies; a looped span of one layer; heads of sizes that are no multiple of 8.
CASE_T = dict(
    architecture="Rupulix", width=40, vocab=90, norm=dict(eps=1e-5), streams=3, logit_scale=1.5,
    loop=dict(start=1, stop=2, times=4),
    layers=[layer(latent(5, 12, 6, 10, 20, base=70.0, window=17), 56),
            layer(parallel(6, 3, 12, 20, 6, 40, 4, 4, base=70.0), 24)])

CASES = {"H": (CASE_H, 3, 8), "J": (CASE_J, 5, 16), "K": (CASE_K, 7, 4), "L": (CASE_L, 9, 16),
         "T": (CASE_T, 11, 32)}                                                              # config, seed, page

_made: dict = {}
_plain: dict = {}


def random_tensors(cfg: dict, seed: int, std: float = 0.12) -> dict:
    """name -> float32 array for every tensor of the model, by name."""
    rng = np.random.default_rng(seed)
    W, S = cfg["width"], cfg.get("streams")
    n = lambda *shape, s=std: rng.normal(0.0, s, size=shape)
    near_one = lambda *shape: 1.0 + rng.uniform(-0.3, 0.3, size=shape)
    t = {"embed": n(cfg["vocab"], W, s=0.5), "final.norm": near_one(W)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        t[p + "norm1"] = near_one(W)
        if S:
            for hc in ("hc1", "hc2")[:2 if L["mlp"] else 1]:
                t[p + hc + ".in"] = near_one(S)
                t[p + hc + ".out"] = near_one(S) * rng.choice([-1.0, 1.0], size=S)
                t[p + hc + ".mix"] = np.eye(S) + n(S, S, s=0.25)
        if L["type"] == "latent_attention":
            H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            t.update({p + "mix.q": n(H * (dn + dr), W), p + "mix.dkv": n(R + dr, W), p + "mix.dkv.norm": near_one(R),
                      p + "mix.uk": n(H * dn, R, s=0.3), p + "mix.uv": n(H * dv, R, s=0.3),
                      p + "mix.sink": n(H, s=1.5), p + "mix.o": n(W, H * dv)})
        else:
            a, r = m["left"], m["right"]
            H, G, d, dv, C, B, K = a["heads"], a["kv_heads"], a["dim"], a["vdim"], r["width"], r["blocks"], r["conv"]
            q = p + "mix.left."
            t.update({q + "q": n(H * d, W), q + "k": n(G * d, W), q + "v": n(G * dv, W), q + "q.norm": near_one(d) * 2.0,
                      q + "k.norm": near_one(d) * 2.0, q + "talk": np.eye(H) + n(H, H, s=0.4), q + "o": n(W, H * dv)})
            q = p + "mix.right."
            t.update({q + "y": n(C, W), q + "y.b": n(C, s=0.3), q + "x": n(C, W), q + "x.b": n(C, s=0.3),
                      q + "conv": n(C, K, s=0.6), q + "conv.b": n(C, s=0.2), q + "ra": n(B, C // B, C // B, s=0.4),
                      q + "ra.b": n(B, C // B, s=0.5), q + "ri": n(B, C // B, C // B, s=0.4), q + "ri.b": n(B, C // B, s=0.5),
                      q + "lam": rng.normal(-3.0, 1.5, size=C), q + "o": n(W, C)})
        if L["mlp"]:
            t.update({p + "norm2": near_one(W), p + "mlp.up": n(L["mlp"]["ff"], W), p + "mlp.down": n(W, L["mlp"]["ff"])})
    return {k: np.asarray(v, dtype=np.float32) for k, v in t.items()}


def write_model(cfg: dict, seed: int, out_dir, change=None) -> Path:
    """config.json and model.safetensors (bfloat16) for ``cfg``; ``change(tensors)`` may edit the arrays first."""
    import torch
    from railgun_b200.weights.safetensors_io import write_safetensors
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    tensors = random_tensors(cfg, seed)
    if change is not None:
        change(tensors)
    (out_dir / "config.json").write_text(json.dumps(cfg))
    write_safetensors(out_dir / "model.safetensors",
                      {k: torch.from_numpy(v).to(torch.bfloat16) for k, v in tensors.items()})
    return out_dir


def model_dir(name: str) -> Path:
    if name not in _made:
        cfg, seed, _ = CASES[name]
        _made[name] = write_model(cfg, seed, tempfile.mkdtemp(prefix=f"rg_rupulix_{name}_"))
    return _made[name]


class Plain:
    """The plain statement over a model folder."""

    def __init__(self, folder):
        import plain_rupulix as P
        self.P = P
        self.cfg = json.loads((Path(folder) / "config.json").read_text())
        self.w = P.read_safetensors(Path(folder) / "model.safetensors")

    def forward(self, ids):
        return self.P.forward(self.cfg, self.w, ids)

    def greedy(self, prompt, n):
        ids = list(prompt)
        for _ in range(n):
            ids.append(int(np.argmax(self.forward(ids)[-1])))
        return ids[len(prompt):]


def plain_model(name: str) -> Plain:
    if name not in _plain:
        _plain[name] = Plain(model_dir(name))
    return _plain[name]


def prompts(vocab: int, lengths, seed: int):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=n).tolist() for n in lengths]
