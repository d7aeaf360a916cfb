"""Rupulix as a description in parts.

Embedding; layers in the order the configuration lists them.  A layer is a
mixer and (unless it has none) a feed-forward, each behind an RMS norm, wired
around ``streams`` copies of the residual stream by hyper-connections
(arrangement "hyper"): the part reads a weighted sum of the copies, and every
copy becomes a mix of all copies plus its own multiple of the part's output.
Without ``streams`` the block is the plain pre-norm one.  Mixers: attention
over a compressed key/value cache with a sliding window and a sink in the
softmax ("latent_attention"), or two branches side by side ("parallel"): an
attention whose heads' scores are mixed before the softmax, with a norm on q
and k ("talking_attention"), and a gated linear recurrence behind a short
convolution ("gated_recurrence").  Feed-forward: down(relu(up x)^2).  A span
of layers may run several times in a row with the same weights and a cache of
its own per pass.  Final norm over the sum of the copies; the head is the
embedding matrix, its logits times ``logit_scale``.

Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.hc1|hc2.in|out|mix``,
``l<i>.mix.*``, ``l<i>.mlp.up|down``, ``final.norm``.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.rupulix import RupulixConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, SubLayer, looped_run_order


def _mixer_spec(c: RupulixConfig, L) -> PartSpec:
    W, m = c.width, L.mixer
    if L.type == "latent_attention":
        return PartSpec("latent_attention", dict(
            hidden_size=W, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, v_dim=m.vdim, kv_rank=m.kv_rank,
            scale=m.scale, rot_dims=m.rot_dims, rot_base=m.rot_base, rot_layout="interleaved", eps=c.norm_eps,
            window=m.window, sink="mix.sink"))
    a, r = m.left, m.right
    left = PartSpec("talking_attention", dict(
        hidden_size=W, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, v_dim=a.vdim, scale=a.scale,
        rot_dims=a.rot_dims, rot_base=a.rot_base, eps=c.norm_eps, window=a.window, base="mix.left."))
    right = PartSpec("gated_recurrence", dict(
        hidden_size=W, width=r.width, blocks=r.blocks, taps=r.conv, base="mix.right."))
    return PartSpec("parallel", dict(branches=((left, m.left_scale), (right, m.right_scale))))


def rupulix_model_spec(c: RupulixConfig) -> ModelSpec:
    W = c.width

    def norm(name, mult=None):
        return PartSpec("rmsnorm", dict(size=W, eps=c.norm_eps, name=name, mult=mult))

    def hyper(name):
        return dict(streams=c.streams, name=name) if c.streams else None

    layers = []
    for i, L in enumerate(c.layers):
        subs = [SubLayer(norm("norm1"), _mixer_spec(c, L), "mixer", wiring=hyper("hc1"))]
        if L.mlp is not None:
            ffn = PartSpec("dense_mlp", dict(hidden_size=W, intermediate_size=L.mlp.ff, activation="relu2",
                                             names=("mlp.up", "mlp.down")))
            subs.append(SubLayer(norm("norm2"), ffn, "ffn", wiring=hyper("hc2")))
        layers.append(LayerSpec(prefix=f"l{i}.", sublayers=tuple(subs), arrangement="hyper" if c.streams else "prenorm"))
    return ModelSpec(
        hidden_size=W, vocab_size=c.vocab, max_position=c.max_position,
        embedding=PartSpec("token_embedding", dict(vocab_size=c.vocab, hidden_size=W, name="embed")),
        layers=tuple(layers),
        # the logits' constant factor is part of the final norm's weight (32-bit, folded at load)
        final_norm=norm("final.norm", mult=c.logit_scale),
        head=PartSpec("lm_head", dict(vocab_size=c.vocab, hidden_size=W, name="embed")),
        schedule=looped_run_order(len(c.layers), c.loop),
    )


RUPULIX = register_architecture(Architecture(
    name="Rupulix",
    config_from_dict=RupulixConfig.from_dict,
    model_spec=rupulix_model_spec,
    description="looped decoder on hyper-connected residual streams: windowed latent-cache attention with a sink, "
                "and talking-heads attention beside a gated linear recurrence",
    family="Rupulix",
), replace=True)
