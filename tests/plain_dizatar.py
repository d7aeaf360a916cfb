"""A plain, slow statement of the Dizatar decoder, one function per mechanism.

Everything here is written from the design's equations with dense tensors on
the CPU: no cache, no pages, no batching, whole sequences at once.  It shares
no code with the package; the package's kernels and parts are compared with it.

Notation: x [T, W] the residual stream of one sequence, W the width;
weights are stored [out, in] and applied as ``W @ v``.
"""
from __future__ import annotations

import math

import torch


def rms_unit(v: torch.Tensor, eps: float) -> torch.Tensor:
    """v / sqrt(mean(v^2) + eps) along the last axis."""
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def rms_norm(v: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(v, eps) * weight


def rotate_half_pairs(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Rotate the first ``dims`` features of v [T, ..., n]: feature i is paired with
    feature i + dims/2 and the pair (a, b) at position p becomes
    (a cos t - b sin t, b cos t + a sin t), t = p * base^(-2i/dims); features from
    ``dims`` on pass unchanged."""
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(v.dtype)[:, None] * freq[None, :]                    # [T, half]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], dim=-1)


def latent_attention(h: torch.Tensor, w: dict, p: dict, eps: float, return_weights: bool = False):
    """The mixer: queries per head, one compressed key/value vector per token
    that every head expands with its own matrices, one rotated key part shared
    by all heads, causal softmax, output projection.  ``w``: the mixer's tensors
    by short name; ``p``: its sizes (heads, dim, rot_dim, vdim, kv_rank, scale,
    rot = {dims, base}).  With ``return_weights`` also the attention weights
    [heads, query, key]."""
    T = h.shape[0]
    H, dn, dr, dv, R = p["heads"], p["dim"], p["rot_dim"], p["vdim"], p["kv_rank"]
    pos = torch.arange(T)
    q = (h @ w["q"].T).view(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], q[..., dn:]
    down = h @ w["dkv"].T                                                    # [T, R + dr]
    latent = rms_norm(down[:, :R], w["dkv.norm"], eps)
    k_rot = rotate_half_pairs(down[:, R:], pos, p["rot"]["dims"], p["rot"]["base"])     # [T, dr]
    q_rot = rotate_half_pairs(q_rot, pos, p["rot"]["dims"], p["rot"]["base"])           # [T, H, dr]
    k_plain = (latent @ w["uk"].T).view(T, H, dn)
    value = (latent @ w["uv"].T).view(T, H, dv)
    scores = torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)
    scores = scores * p["scale"]
    hidden = torch.ones(T, T, dtype=torch.bool).triu(1)                      # j > i
    scores = scores.masked_fill(hidden, -math.inf)
    weights = torch.softmax(scores, dim=-1)
    out = torch.einsum("hij,jhd->ihd", weights, value).reshape(T, H * dv)
    return (out @ w["o"].T, weights) if return_weights else out @ w["o"].T


def gated_expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    g = h @ gate.T
    return ((g * torch.sigmoid(g)) * (h @ up.T)) @ down.T


def route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, top: int):
    """Chosen experts [T, top] and their weights: softmax over all router
    outputs; the choice is by score + correction, the weights are the chosen
    scores themselves divided by their sum."""
    scores = torch.softmax(h @ router.T, dim=-1)
    chosen = torch.topk(scores + correction, top, dim=-1).indices
    picked = torch.gather(scores, 1, chosen)
    return chosen, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20)


def route_margin(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, top: int) -> torch.Tensor:
    """How far each token's choice is from a tie [T]: the gap between the last
    chosen and the first unchosen corrected score, relative to the sum of the
    two experts' scores (infinite when every router output is chosen).  A model
    in reduced precision may choose differently where this is small."""
    scores = torch.softmax(h @ router.T, dim=-1)
    if top >= scores.shape[-1]:
        return torch.full((h.shape[0],), math.inf, dtype=h.dtype)
    order = torch.sort(scores + correction, dim=-1, descending=True)
    pair = torch.gather(scores, 1, order.indices[:, top - 1:top + 1])
    return (order.values[:, top - 1] - order.values[:, top]) / pair.sum(dim=-1)


def expert_mixture(h: torch.Tensor, w: dict, p: dict) -> torch.Tensor:
    """Routed experts plus an always-on shared one.  The last ``identity``
    router outputs stand for experts that return their input."""
    n_real, n_id, top = p["router"]["experts"], p["router"]["identity"], p["router"]["top"]
    chosen, weights = route(h, w["router"], w["correction"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weights[t]):
            if e >= n_real:
                assert e < n_real + n_id
                out[t] += g * h[t]
            else:
                out[t] += g * gated_expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if p.get("shared"):
        out = out + gated_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"])
    return out


def softcap(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def layer_order(cfg: dict) -> list:
    """(layer index, pass starts here) in run order: layers before the loop, the
    looped span ``times`` times, the rest."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    order += [(i, False) for i in range(b, n)]
    return order


def forward(cfg: dict, tensors: dict, tokens, dtype=torch.float64, return_layers: bool = False,
            return_margins: bool = False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after
    every layer run, or each position's smallest ``route_margin`` over all
    feed-forwards that ran)."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x0 = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0
    trail = []
    margins = torch.full((x.shape[0],), math.inf, dtype=dtype)
    for i, starts_pass in layer_order(cfg):
        L = cfg["layers"][i]
        pre = f"l{i}."
        if starts_pass:
            x = torch.cat([x, x0], dim=-1) @ t["loop.in"].T
        assert L["type"] == "latent_attention"
        y = latent_attention(rms_norm(x, t[pre + "norm1"], eps), sub(t, pre + "mix."), L["mixer"], eps)
        x = x + m * (rms_norm(y, t[pre + "norm1b"], eps) * t[pre + "ls1"])
        if L.get("mlp"):
            assert L["mlp"]["kind"] == "moe"
            h2 = rms_norm(x, t[pre + "norm2"], eps)
            margins = torch.minimum(margins, route_margin(h2, t[pre + "mlp.router"], t[pre + "mlp.correction"],
                                                          L["mlp"]["router"]["top"]))
            y = expert_mixture(h2, sub(t, pre + "mlp."), L["mlp"])
            x = x + m * (rms_norm(y, t[pre + "norm2b"], eps) * t[pre + "ls2"])
        trail.append(x)
    logits = softcap(rms_norm(x, t["final.norm"], eps) @ t["head"].T, cfg["logit_softcap"])
    if return_margins:
        return logits, margins
    return (logits, torch.stack(trail)) if return_layers else logits


class PlainDizatar:
    """The plain model over a folder with config.json and model.safetensors,
    read with the test suite's own reader; 64-bit arithmetic on the stored
    values."""

    def __init__(self, model_dir):
        import json
        from pathlib import Path

        from plain_llama import read_safetensors
        model_dir = Path(model_dir)
        self.cfg = json.loads((model_dir / "config.json").read_text())
        self.tensors = {k: torch.from_numpy(v) for k, v in read_safetensors(model_dir / "model.safetensors").items()}

    def forward(self, tokens, return_layers: bool = False, return_margins: bool = False):
        out = forward(self.cfg, self.tensors, tokens, torch.float64, return_layers, return_margins)
        return (out[0].numpy(), out[1].numpy()) if return_layers or return_margins else out.numpy()

    def greedy(self, prompt, n: int) -> list:
        toks = list(prompt)
        for _ in range(n):
            toks.append(int(self.forward(toks)[-1].argmax()))
        return toks[len(prompt):]
