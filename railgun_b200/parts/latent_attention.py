"""Attention with a compressed key/value cache shared by all heads.

Per token the mixer keeps one vector c of ``kv_rank`` numbers (a
down-projection of its input, RMS-normed) and one rotated key part of
``rot_dim`` numbers; head h's keys and values are U_k[h] c and U_v[h] c.  A
head's score is scale * (q_plain . U_k[h] c + q_rot . k_rot), so with the
plain query part taken through U_k[h]^T once, every head reads the same
cache rows: scores over [c | k_rot], values = c, and the head's output is
U_v[h] applied to the weighted sum of c.  In this form nothing is expanded per head.

  proj          one product for the queries and the down-projection
  qa[:, h, :R]  = U_k[h]^T q_plain[h]          batched product (library)
  qa[:, h, R:]  = rotate(q_rot[h]);  cache row = [rmsnorm(c) | rotate(k_rot)]   (one kernel)
  o_lat         attention over the cache                                        (kernels)
  out           = W_o concat_h(U_v[h] o_lat[h])    batched product, product

That is the form single tokens always take.  Requests that bring several
tokens attend per head to expanded keys [U_k c | k_rot] and values U_v c
where that is cheaper and the sizes fit the flash kernel of ordinary paged
attention: the step expands those requests' contexts from the cache into
temporary key/value pages (``ops.latent_expand_context``) and rotates the
queries in place; the cache itself only ever holds the compressed rows.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache.manager import PagedKVNeed
from ..weights.loader import TensorSpec
from .base import Mixer
from .registry import register_mixer


def rotary_frequencies(dims: int, base: float) -> torch.Tensor:
    """f_i = base^(-2i/dims), i < dims/2, in 64-bit (the kernels multiply by the position in 64-bit too)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    return float(base) ** (-2.0 * i / dims)


class LatentAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``head_dim`` (unrotated query/key
    numbers per head), ``rot_dim`` (rotated ones), ``v_dim``, ``kv_rank``,
    ``scale``, ``rot_dims`` (how many of the rotated part's numbers are rotated),
    ``rot_layout`` ("half": pairs (i, i + rot_dims/2), the default; "interleaved":
    pairs (2i, 2i + 1)), ``rot_base``, ``eps`` (of the latent's norm), ``window``
    (0: none; else a query sees itself and the window - 1 positions before it),
    ``sink`` (optional: the name after the prefix of a tensor [heads]; exp of
    head h's number joins the denominator of h's softmax, with no key and no
    value), ``names`` (optional: tensor names after the prefix for q, dkv,
    dkv_norm, uk, uv, o)."""

    NAMES = dict(q="mix.q", dkv="mix.dkv", dkv_norm="mix.dkv.norm", uk="mix.uk", uv="mix.uv", o="mix.o")

    @classmethod
    def _names(cls, p, prefix):
        return {k: prefix + v for k, v in {**cls.NAMES, **(p.get("names") or {})}.items()}

    @classmethod
    def tensor_specs(cls, p, prefix):
        W, H, dn, dr, dv, R = (p["hidden_size"], p["num_heads"], p["head_dim"], p["rot_dim"], p["v_dim"],
                               p["kv_rank"])
        n = cls._names(p, prefix)
        sink = {prefix + p["sink"]: TensorSpec((H,))} if p.get("sink") else {}
        return {
            **sink,
            n["q"]: TensorSpec((H * (dn + dr), W)),
            n["dkv"]: TensorSpec((R + dr, W)),
            n["dkv_norm"]: TensorSpec((R,), init="norm"),
            n["uk"]: TensorSpec((H * dn, R)),
            n["uv"]: TensorSpec((H * dv, R)),
            n["o"]: TensorSpec((W, H * dv)),
        }

    @classmethod
    def cache_need(cls, p):
        D = p["kv_rank"] + p["rot_dim"]
        return PagedKVNeed(1, D, int(p.get("window") or 0), page_shape=("page", D))

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        self.H, self.dn, self.dr, self.dv, self.R = (p["num_heads"], p["head_dim"], p["rot_dim"], p["v_dim"],
                                                     p["kv_rank"])
        self.D = self.R + self.dr
        self.rot_dims = int(p["rot_dims"])
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.dr:
            raise ValueError(f"{self.rot_dims} rotated numbers do not fit a rotated part of {self.dr}")
        if self.R > 1024:
            raise ValueError(f"a latent of {self.R} numbers is above the attention kernels' limit of 1024")
        self.window = int(p.get("window") or 0)
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        layout = p.get("rot_layout") or "half"
        if layout not in ("half", "interleaved"):
            raise ValueError(f"rotation layout {layout!r} is not known: 'half' or 'interleaved'")
        self.interleaved = layout == "interleaved"
        self.sink = tensors.get(prefix + p["sink"], torch.float32).contiguous() if p.get("sink") else None
        n = self._names(p, prefix)
        self.w_proj = torch.cat([tensors.get(n["q"], env.dtype), tensors.get(n["dkv"], env.dtype)], dim=0).contiguous()
        tensors.drop(n["q"], n["dkv"])
        self.kv_off = self.H * (self.dn + self.dr)
        self.norm_w = tensors.get(n["dkv_norm"], torch.float32)
        self.w_uk = tensors.get(n["uk"], env.dtype).view(self.H, self.dn, self.R)                      # [H, dn, R]
        self.w_uv_t = tensors.get(n["uv"], env.dtype).view(self.H, self.dv, self.R).transpose(1, 2)    # [H, R, dv]
        self.w_o = tensors.get(n["o"], env.dtype)
        self.freq = tensors.shared_part(("rotary_frequencies", self.rot_dims, float(p["rot_base"])),
                                        lambda: rotary_frequencies(self.rot_dims, p["rot_base"]).to(env.device))
        # Prompts attend in the expanded form (keys [U_k c | k_rot], values U_v c per head: dn + dr + dv numbers
        # per key and head instead of 2 R + dr) through the dense model's flash kernel, where the sizes fit it.
        d = self.dn + self.dr
        self.expands_prompts = (env.dtype == torch.bfloat16 and d % 16 == 0 and 16 <= d <= 256 and self.dv <= d
                                and self.window == 0 and self.sink is None and d + self.dv < 2 * self.R + self.dr)
        if self.expands_prompts:
            self.w_uk_flat = tensors.get(n["uk"], env.dtype)                                # [H dn, R]
            self.w_uv_flat = tensors.get(n["uv"], env.dtype)                                # [H dv, R]
            pad = torch.zeros((self.w_o.shape[0], self.H, d), dtype=env.dtype, device=self.w_o.device)
            pad[:, :, :self.dv] = self.w_o.view(-1, self.H, self.dv)
            self.w_o_padded = pad.view(-1, self.H * d).contiguous()                         # zero columns behind each head's dv

    def forward(self, x, batch, cache, writes=True):
        H, dn, dr, dv, R, D = self.H, self.dn, self.dr, self.dv, self.R, self.D
        T = x.shape[0]
        proj = ops.linear(x, self.w_proj)                                                  # [T, H (dn + dr) + R + dr]
        slots = batch.slot_mapping[cache.group] if writes else None
        if self._expand_this_step(batch, cache, T):
            return self._forward_expanded(proj, batch, cache, slots)
        qa = torch.empty((T, H, D), dtype=proj.dtype, device=proj.device)
        q_plain = proj[:, :self.kv_off].view(T, H, dn + dr)[:, :, :dn].transpose(0, 1)     # [H, T, dn], no copy
        torch.bmm(q_plain, self.w_uk, out=qa[:, :, :R].transpose(0, 1))
        ops.latent_rope_cache(proj, self.kv_off, qa, cache.kv, self.norm_w, self.eps, self.freq, self.rot_dims,
                              batch.positions, slots, H, dn, dr, R, interleaved=self.interleaved)
        o_lat = self.attend(qa, batch, cache)                                              # [T, H, R]
        heads = torch.empty((T, H * dv), dtype=proj.dtype, device=proj.device)
        torch.bmm(o_lat.transpose(0, 1), self.w_uv_t, out=heads.view(T, H, dv).transpose(0, 1))
        return ops.linear(heads, self.w_o)

    def _expand_this_step(self, batch, cache, T) -> bool:
        """Prompts go through the expanded form when the step has some and the temporary pages (every request of
        the step at the block table's width) stay within a few times the step's tokens."""
        if not self.expands_prompts or batch.decode_only or not batch.num_prefill_tiles:
            return False
        table = batch.block_table[cache.group]
        return table.shape[0] * table.shape[1] * cache.page_size <= max(8192, 4 * T)

    def _forward_expanded(self, proj, batch, cache, slots):
        H, dn, dr, dv, R, D = self.H, self.dn, self.dr, self.dv, self.R, self.D
        T, d = proj.shape[0], self.dn + self.dr
        table = batch.block_table[cache.group]
        out = torch.zeros((T, H * d), dtype=proj.dtype, device=proj.device)
        qa = None
        if batch.num_decode_rows:
            # the step's single tokens stay in the compressed form; their rows of `out` are filled first
            qa = torch.empty((T, H, D), dtype=proj.dtype, device=proj.device)
            q_plain = proj[:, :self.kv_off].view(T, H, d)[:, :, :dn].transpose(0, 1)
            torch.bmm(q_plain, self.w_uk, out=qa[:, :, :R].transpose(0, 1))
        ops.latent_rope_cache(proj, self.kv_off, qa, cache.kv, self.norm_w, self.eps, self.freq, self.rot_dims,
                              batch.positions, slots, H, dn, dr, R, q_in_place=True, interleaved=self.interleaved)
        if batch.num_decode_rows:
            n = batch.num_decode_rows
            o_lat = torch.zeros((T, H, R), dtype=proj.dtype, device=proj.device)
            if ops.latent_attention_mma_ok(qa.dtype, H, R, D):
                ops.latent_attention_mma(qa, o_lat, cache.kv, table, None, batch.decode_rows, n, batch.req_of_token,
                                         batch.positions, R, self.window, self.scale,
                                         ops.latent_decode_splits(n, -(-H // 64), batch.max_context_len))
            else:
                o_lat = ops.latent_attention_general(qa, cache.kv, table, batch.req_of_token, batch.positions, R,
                                                     self.window, self.scale)
            torch.bmm(o_lat.transpose(0, 1), self.w_uv_t, out=out.view(T, H, d)[:, :, :dv].transpose(0, 1))
        kv, kv_table = ops.latent_expand_context(cache.kv, table, batch.cu_seqlens, batch.context_lens, self.w_uk_flat,
                                                 self.w_uv_flat, H, dn, dr, dv, R)
        ops.prefill_attention(proj, proj.stride(0), out, kv, kv_table, batch.prefill_tiles, batch.positions, H, H, d,
                              0, self.scale)
        return ops.linear(out, self.w_o_padded)

    def attend(self, qa, batch, cache):
        """bfloat16 with sizes in steps of 16 runs on the tensor cores (requests with several tokens in tiles of
        64 / heads tokens, single tokens with their contexts cut into shares); everything else, and all of the
        32-bit path, through the general kernel."""
        table = batch.block_table[cache.group]
        if not ops.latent_attention_mma_ok(qa.dtype, self.H, self.R, self.D):
            return ops.latent_attention_general(qa, cache.kv, table, batch.req_of_token, batch.positions, self.R,
                                                self.window, self.scale, self.sink)
        out = torch.empty((qa.shape[0], self.H, self.R), dtype=qa.dtype, device=qa.device)
        chunks = -(-self.H // 64)
        args = (batch.req_of_token, batch.positions, self.R, self.window, self.scale)
        # a single token sees at most its window: that is what its context is cut into shares by
        reach = min(batch.max_context_len, self.window) if self.window else batch.max_context_len
        if batch.decode_only:
            n = batch.num_tokens
            ops.latent_attention_mma(qa, out, cache.kv, table, None, None, n, *args,
                                     ops.latent_decode_splits(n, chunks, reach), sink=self.sink)
            return out
        if batch.num_prefill_tiles:
            ops.latent_attention_mma(qa, out, cache.kv, table, batch.prefill_tiles, None, batch.num_prefill_tiles, *args,
                                     sink=self.sink)
        if batch.num_decode_rows:
            n = batch.num_decode_rows
            ops.latent_attention_mma(qa, out, cache.kv, table, None, batch.decode_rows, n, *args,
                                     ops.latent_decode_splits(n, chunks, reach), sink=self.sink)
        return out


register_mixer("latent_attention", LatentAttention)
