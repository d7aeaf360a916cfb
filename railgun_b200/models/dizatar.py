"""Dizatar as a description in parts.

Embedding; layers in the order the configuration lists them, each a
"sandwich" block: x += m * ls1 * norm1b(mixer(norm1(x))), then
x += m * ls2 * norm2b(ff(norm2(x))) (m the residual multiplier, ls the
per-feature layer scales; a layer may have no feed-forward); the mixer is
attention over a compressed key/value cache, the feed-forward a mixture of
gated experts with identity experts and a shared one.  A span of layers runs
several times in a row with the same weights and a cache of its own per pass;
each pass starts with x <- W_in [x; x0], x0 the embedding's output.  Final
norm, head, soft cap on the logits.

Tensor names: ``embed``, ``loop.in``, ``l<i>.norm1|norm2|norm1b|norm2b``,
``l<i>.ls1|ls2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.dizatar import DizatarConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, SubLayer, looped_run_order


def dizatar_run_order(n_layers: int, loop) -> tuple:
    """Schedule entries: the layers before the span, the span ``times`` times
    (every pass with caches of its own, its first layer behind stream
    operation 0), the layers after it."""
    return looped_run_order(n_layers, loop, before=0)


def dizatar_model_spec(c: DizatarConfig) -> ModelSpec:
    W = c.width

    def norm(name, scale_name=None, mult=None):
        return PartSpec("rmsnorm", dict(size=W, eps=c.norm_eps, name=name, scale_name=scale_name, mult=mult))

    layers = []
    for i, L in enumerate(c.layers):
        m = L.mixer
        mixer = PartSpec(L.type, dict(
            hidden_size=W, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, v_dim=m.vdim, kv_rank=m.kv_rank,
            scale=m.scale, rot_dims=m.rot_dims, rot_base=m.rot_base, eps=c.norm_eps, window=0))
        subs = [SubLayer(norm("norm1"), mixer, "mixer", norm("norm1b", "ls1", c.residual_mult))]
        if L.mlp is not None:
            f = L.mlp
            ffn = PartSpec("routed_experts", dict(
                hidden_size=W, experts=f.experts, identity=f.identity, top=f.top, expert_size=f.expert_ff,
                shared_size=f.shared_ff, base="mlp."))
            subs.append(SubLayer(norm("norm2"), ffn, "ffn", norm("norm2b", "ls2", c.residual_mult)))
        layers.append(LayerSpec(prefix=f"l{i}.", sublayers=tuple(subs), arrangement="sandwich"))
    return ModelSpec(
        hidden_size=W, vocab_size=c.vocab, max_position=c.max_position,
        embedding=PartSpec("token_embedding", dict(vocab_size=c.vocab, hidden_size=W, name="embed")),
        layers=tuple(layers),
        final_norm=PartSpec("rmsnorm", dict(size=W, eps=c.norm_eps, name="final.norm")),
        head=PartSpec("lm_head", dict(vocab_size=c.vocab, hidden_size=W, name="head", softcap=c.logit_softcap)),
        schedule=dizatar_run_order(len(c.layers), c.loop),
        stream_ops=(PartSpec("reinject", dict(hidden_size=W, name="loop.in")),) if c.loop is not None else (),
    )


DIZATAR = register_architecture(Architecture(
    name="Dizatar",
    config_from_dict=DizatarConfig.from_dict,
    model_spec=dizatar_model_spec,
    description="looped decoder: latent-cache attention, routed experts with identity and shared experts, "
                "norms on both sides of every part",
    family="Dizatar",
), replace=True)
