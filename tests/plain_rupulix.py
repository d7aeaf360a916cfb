"""Rupulix, stated plainly: dense numpy in 64-bit, one function per mechanism,
whole sequences at once, no cache and no kernels.  Shares nothing with the
package; the tests hold the package's steps to this.

Notation: T tokens, W width, weights are stored [out, in] and applied as
y = x @ w.T.  ``w`` maps tensor names to float64 arrays.
"""
from __future__ import annotations

import json
import struct

import numpy as np


def read_safetensors(path) -> dict:
    """name -> float64 array (integers stay integers)."""
    raw = open(path, "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        buf = raw[8 + n + lo:8 + n + hi]
        if meta["dtype"] == "BF16":
            a = (np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif meta["dtype"] == "F32":
            a = np.frombuffer(buf, dtype="<f4").astype(np.float64)
        elif meta["dtype"] == "I32":
            a = np.frombuffer(buf, dtype="<i4")
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        out[name] = a.reshape(meta["shape"])
    return out


# ---- small pieces ---------------------------------------------------------------------------------
def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def rotary_angles(pos, dims, base):
    """[T, dims/2]: position * base^(-2i/dims)."""
    i = np.arange(dims // 2, dtype=np.float64)
    return np.asarray(pos, dtype=np.float64)[:, None] * (float(base) ** (-2.0 * i / dims))[None, :]


def rotate(x, pos, dims, base, layout):
    """x [T, heads, d]: the first ``dims`` numbers of every head are rotated in
    pairs, (i, i + dims/2) for layout "half" and (2i, 2i+1) for "interleaved";
    (u, v) -> (u cos a - v sin a, v cos a + u sin a).  The rest passes."""
    if dims == 0:
        return x.copy()
    a = rotary_angles(pos, dims, base)
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    out = x.copy()
    if layout == "half":
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = u * c - v * s
        out[..., dims // 2:dims] = v * c + u * s
    elif layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        raise ValueError(layout)
    return out


def visible(T, window):
    """[T, T] mask: query i sees key j when 0 <= i - j (< window, if there is one)."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    m = j <= i
    if window:
        m &= (i - j) < window
    return m


def softmax_rows(scores, mask, sink=None):
    """Softmax over the visible keys of [..., T, T] scores; with ``sink`` [heads]
    the denominator also holds exp(sink) per head (scores are [heads, T, T] then)."""
    s = np.where(mask, scores, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    if sink is not None:
        m = np.maximum(m, sink[:, None, None])
    e = np.exp(s - m)
    den = e.sum(axis=-1, keepdims=True)
    if sink is not None:
        den = den + np.exp(sink[:, None, None] - m)
    return e / den


# ---- mixers ---------------------------------------------------------------------------------------
def latent_attention(h, w, p, m, eps):
    """m: the mixer's configuration (heads, dim, rot_dim, vdim, kv_rank, scale, rot, mask)."""
    T = h.shape[0]
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T)
    q = (h @ w[p + "q"].T).reshape(T, H, dn + dr)
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :R], w[p + "dkv.norm"], eps)
    rot = m["rot"]
    k_rot = rotate(down[:, None, R:], pos, rot["dims"], rot["base"], "interleaved")[:, 0]     # shared by the heads
    q_rot = rotate(q[:, :, dn:], pos, rot["dims"], rot["base"], "interleaved")
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    scores = (np.einsum("ihd,jhd->hij", q[:, :, :dn], k_plain) + np.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    window = (m.get("mask") or {}).get("size", 0)
    sink = w.get(p + "sink")
    pr = softmax_rows(scores, visible(T, window)[None], sink)
    out = np.einsum("hij,jhd->ihd", pr, v).reshape(T, H * dv)
    return out @ w[p + "o"].T


def talking_attention(h, w, p, m, eps):
    """Grouped-query attention with a norm on q and k per head, partial rotation
    ("half" layout) and scores mixed across heads before the softmax."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q = (h @ w[p + "q"].T).reshape(T, H, d)
    k = (h @ w[p + "k"].T).reshape(T, G, d)
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    rot = m["rot"]
    q = rotate(q, pos, rot["dims"], rot["base"], "half")
    k = rotate(k, pos, rot["dims"], rot["base"], "half")
    group = np.arange(H) // (H // G)
    scores = np.einsum("ihd,jhd->hij", q, k[:, group]) * m["scale"]
    scores = np.einsum("hg,gij->hij", w[p + "talk"], scores)
    window = (m.get("mask") or {}).get("size", 0)
    pr = softmax_rows(scores, visible(T, window)[None])
    out = np.einsum("hij,jhd->ihd", pr, v[:, group]).reshape(T, H * dv)
    return out @ w[p + "o"].T


def causal_conv(x, taps, bias):
    """x [T, C], taps [C, K]: y_t = bias + sum_k taps[:, K-1-k] x_(t-k), zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    y = np.tile(bias, (T, 1)).astype(np.float64)
    for k in range(min(K, T)):
        y[k:] += x[:T - k] * taps[:, K - 1 - k]
    return y


def gated_recurrence(h, w, p, m):
    """Two branches of size ``width``: a gate branch gelu(W_y h + b) and a
    convolved branch u; block-diagonal gates r and i from u; state
    S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t with a_t = exp(-8 r_t softplus(lam))."""
    T = h.shape[0]
    C, B = m["width"], m["blocks"]
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    ub = u.reshape(T, B, C // B)
    r = sigmoid(np.einsum("tbi,boi->tbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(T, C)
    g = sigmoid(np.einsum("tbi,boi->tbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(T, C)
    a = np.exp(-8.0 * r * softplus(w[p + "lam"]))
    drive = np.sqrt(1.0 - a * a) * g * u
    S = np.zeros(C)
    out = np.empty((T, C))
    for t in range(T):
        S = a[t] * S + drive[t]
        out[t] = S
    return (out * y) @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    left = talking_attention(h, w, p + "left.", m["left"], eps)
    right = gated_recurrence(h, w, p + "right.", m["right"])
    return m["left_scale"] * left + m["right_scale"] * right


def mixer(h, w, layer_cfg, prefix, eps):
    kind = layer_cfg["type"]
    if kind == "latent_attention":
        return latent_attention(h, w, prefix + "mix.", layer_cfg["mixer"], eps)
    if kind == "parallel":
        return parallel_mixer(h, w, prefix + "mix.", layer_cfg["mixer"], eps)
    raise ValueError(kind)


def feed_forward(h, w, prefix):
    z = np.maximum(h @ w[prefix + "mlp.up"].T, 0.0)
    return (z * z) @ w[prefix + "mlp.down"].T


# ---- the block and the model ----------------------------------------------------------------------
def hyper_step(xs, w, name, norm_w, eps, fn):
    """xs [S, T, W]: u = sum_s in[s] x_s; y = fn(norm(u)); x_t <- sum_s mix[s, t] x_s + out[t] y."""
    u = np.einsum("s,stw->tw", w[name + ".in"], xs)
    y = fn(rms_norm(u, norm_w, eps))
    return np.einsum("st,sjw->tjw", w[name + ".mix"], xs) + w[name + ".out"][:, None, None] * y[None]


def run_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    span = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + span * loop["times"] + list(range(loop["stop"], n))


def forward(cfg, w, ids, keep_layers=False):
    """Logits [T, vocab] of one sequence (and, with ``keep_layers``, the residual
    stream after every layer run, [runs, T, W]; the sum of the streams if there are several)."""
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][np.asarray(ids)]
    S = cfg.get("streams")
    xs = np.stack([x0] * S) if S else x0
    kept = []
    for li in run_order(cfg):
        L = cfg["layers"][li]
        p = f"l{li}."
        subs = [("hc1", "norm1", lambda h, L=L, p=p: mixer(h, w, L, p, eps))]
        if L.get("mlp") is not None:
            subs.append(("hc2", "norm2", lambda h, p=p: feed_forward(h, w, p)))
        for hc, norm, fn in subs:
            if S:
                xs = hyper_step(xs, w, p + hc, w[p + norm], eps, fn)
            else:
                xs = xs + fn(rms_norm(xs, w[p + norm], eps))
        kept.append(xs.sum(axis=0) if S else xs.copy())
    x = xs.sum(axis=0) if S else xs
    logits = rms_norm(x, w["final.norm"], eps) @ w["embed"].T * cfg.get("logit_scale", 1.0)
    return (logits, np.stack(kept)) if keep_layers else logits
