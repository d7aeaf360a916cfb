"""Grouped-query attention whose heads talk before the softmax.

q, k, v = x Wq^T, x Wk^T, x Wv^T; every q and k head is RMS-normed over its
own numbers with one weight vector shared by the heads (one for q, one for
k), then the first ``rot_dims`` numbers of each are rotated in pairs
(i, i + rot_dims/2); the scaled scores of all heads for one (query, key) pair
are mixed by a matrix M [heads, heads], s'_h = sum_g M[h, g] s_g, before each
head's softmax; values may have another size than keys.  One cache row per
token holds all value heads, then all key heads.

In bfloat16, where the sizes fit, the attention runs on the tensor cores in
the form of attention over a latent cache: the mixing is linear in q, so the
step mixes the queries instead of the scores (Q'_h holds, for every key/value
head c, scale * sum over c's heads g of M[h, g] q_g), every head then scores
the same cache rows, and the kernel of ``latent_attention`` does the rest,
each head keeping the values of its own key/value head.  Requests that bring
several tokens run on the flash kernel of ordinary paged attention instead
where all key heads side by side fit its head sizes: their contexts are laid
out as temporary pages in which every key/value head sees all keys and its
own values.  Everything else, and the whole 32-bit path, runs the general
kernel, which mixes the scores themselves.

Sizes and constants are parameters; the norm and the mixing can be left out,
which gives plain grouped-query attention with separate key and value sizes.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache.manager import PagedKVNeed
from ..weights.loader import TensorSpec
from .base import Mixer
from .latent_attention import rotary_frequencies
from .registry import register_mixer


class TalkingAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``
    (query/key numbers per head), ``v_dim``, ``scale``, ``rot_dims``,
    ``rot_base``, ``eps`` (of the q and k norms), ``window`` (0: none),
    ``base`` (what the tensor names start with after the prefix, default
    "mix."; the tensors are q, k, v, o, q.norm, k.norm, talk), ``qk_norm`` and
    ``talk`` (default true: false leaves the mechanism and its tensor out)."""

    @classmethod
    def _base(cls, p, prefix):
        return prefix + (p.get("base") if p.get("base") is not None else "mix.")

    @classmethod
    def tensor_specs(cls, p, prefix):
        W, H, G, d, dv = p["hidden_size"], p["num_heads"], p["num_kv_heads"], p["head_dim"], p["v_dim"]
        b = cls._base(p, prefix)
        out = {b + "q": TensorSpec((H * d, W)), b + "k": TensorSpec((G * d, W)), b + "v": TensorSpec((G * dv, W)),
               b + "o": TensorSpec((W, H * dv))}
        if p.get("qk_norm", True):
            out[b + "q.norm"] = TensorSpec((d,), init="norm")
            out[b + "k.norm"] = TensorSpec((d,), init="norm")
        if p.get("talk", True):
            out[b + "talk"] = TensorSpec((H, H), init="eye")
        return out

    @classmethod
    def cache_need(cls, p):
        G, d, dv = p["num_kv_heads"], p["head_dim"], p["v_dim"]
        return PagedKVNeed(G, d + dv, int(p.get("window") or 0), page_shape=("page", G * (d + dv)))

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        self.H, self.G, self.d, self.dv = p["num_heads"], p["num_kv_heads"], p["head_dim"], p["v_dim"]
        if self.H % self.G:
            raise ValueError(f"{self.H} heads cannot share {self.G} key/value heads")
        self.rot_dims = int(p.get("rot_dims") or 0)
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.d:
            raise ValueError(f"{self.rot_dims} rotated numbers do not fit a head of {self.d}")
        self.window = int(p.get("window") or 0)
        self.scale = float(p["scale"]) if p.get("scale") is not None else float(self.d) ** -0.5
        self.eps = float(p.get("eps") or 0.0)
        b = self._base(p, prefix)
        self.w_qkv = torch.cat([tensors.get(b + n, env.dtype) for n in ("q", "k", "v")], dim=0).contiguous()
        tensors.drop(b + "q", b + "k", b + "v")
        self.w_in = self.w_qkv
        self.w_o = tensors.get(b + "o", env.dtype)
        self.out_features = self.H * self.dv
        norm = p.get("qk_norm", True)
        self.q_norm = tensors.get(b + "q.norm", torch.float32).contiguous() if norm else None
        self.k_norm = tensors.get(b + "k.norm", torch.float32).contiguous() if norm else None
        self.talk = tensors.get(b + "talk", torch.float32).contiguous() if p.get("talk", True) else None
        base = float(p.get("rot_base") or 10000.0)
        self.freq = tensors.shared_part(("rotary_frequencies", self.rot_dims, base),
                                        lambda: rotary_frequencies(self.rot_dims, base).to(env.device))

    def mix(self, x, batch, cache, writes=True, out=None, out_scale: float = 1.0, proj=None):
        """The heads' outputs [T, heads * v_dim] times ``out_scale``, before the output product (into ``out``, a
        view whose rows may be further apart, if given).  ``proj``: x times ``w_in``, if the caller has it
        already (as columns of a wider product)."""
        H, G, d, dv = self.H, self.G, self.d, self.dv
        qkv = proj if proj is not None else ops.linear(x, self.w_qkv)
        T = qkv.shape[0]
        slots = batch.slot_mapping[cache.group] if writes else None
        table = batch.block_table[cache.group]
        R, D = G * dv, G * (d + dv)
        if dv % 2 == 0 and ops.latent_attention_mma_ok(qkv.dtype, H, R, D):
            # the tensor-core forms, both over mixed queries: requests that bring several tokens on the flash kernel
            # of paged attention over temporary pages (where the sizes fit it, there is no window, and the pages of
            # the step's contexts stay within a few times its tokens), single tokens over the rows [values | keys]
            flash = (self.window == 0 and batch.num_prefill_tiles > 0 and ops.talking_flash_ok(qkv.dtype, G, d, dv)
                     and table.shape[0] * table.shape[1] * cache.page_size <= max(8192, 4 * T))
            rows_form = batch.decode_only or batch.num_decode_rows > 0 or not flash
            qa = torch.empty((T, H, D), dtype=qkv.dtype, device=qkv.device) if rows_form else None
            qc = torch.empty((T, H, G * d), dtype=qkv.dtype, device=qkv.device) if flash else None
            ops.talking_prepare(qkv, None, cache.kv, self.q_norm, self.k_norm, self.eps, self.freq, self.rot_dims,
                                batch.positions, slots, H, G, d, dv, qa=qa, talk=self.talk, scale=self.scale, qc=qc)
            if out is None:
                out = torch.empty((T, H * dv), dtype=qkv.dtype, device=qkv.device)
            args = (batch.req_of_token, batch.positions, R, self.window, 1.0)
            more = dict(select=(dv, H // G), out_scale=out_scale, score_from=R)     # R = G dv zeros lead the queries
            reach = min(batch.max_context_len, self.window) if self.window else batch.max_context_len
            chunks = -(-H // 64)
            if batch.decode_only:
                n = batch.num_tokens
                ops.latent_attention_mma(qa, out, cache.kv, table, None, None, n, *args,
                                         ops.latent_decode_splits(n, chunks, reach), **more)
                return out
            if flash:
                ops.talking_prefill_flash(qc, cache.kv, table, batch, G, d, dv, out, out_scale)
            elif batch.num_prefill_tiles:
                ops.latent_attention_mma(qa, out, cache.kv, table, batch.prefill_tiles, None, batch.num_prefill_tiles,
                                         *args, **more)
            if batch.num_decode_rows:
                n = batch.num_decode_rows
                ops.latent_attention_mma(qa, out, cache.kv, table, None, batch.decode_rows, n, *args,
                                         ops.latent_decode_splits(n, chunks, reach), **more)
            return out
        q = torch.empty((T, H, d), dtype=qkv.dtype, device=qkv.device)
        ops.talking_prepare(qkv, q, cache.kv, self.q_norm, self.k_norm, self.eps, self.freq, self.rot_dims,
                            batch.positions, slots, H, G, d, dv)
        return ops.talking_attention_general(q, cache.kv, self.talk, table, batch.req_of_token, batch.positions, G, dv,
                                             self.window, self.scale, out, out_scale)

    def forward(self, x, batch, cache, writes=True):
        w_o = self.w_o if self.w_o.is_contiguous() else self.w_o.contiguous()     # a share of a stacked matrix
        return ops.linear(self.mix(x, batch, cache, writes), w_o)


register_mixer("talking_attention", TalkingAttention)
