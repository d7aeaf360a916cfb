"""Typed reading of a Dizatar model's config.json.

The file lists the layers one by one (``layers``: each with ``type``, the
mixer's sizes under ``mixer`` and the feed-forward under ``mlp``, null for
none), names a span of layers that runs several times in a row (``loop``:
``start``, ``stop``, ``times``), and gives the constants that differ between
models: ``norm.eps``, ``residual_mult``, ``logit_softcap``, ``width``,
``vocab``.  ``architecture`` (a string) names the design.  ``max_position``
is optional (default 2^20: positions are computed, not tabulated).
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, KeyReader

DEFAULT_MAX_POSITION = 1 << 20


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int                # unrotated query/key numbers per head
    rot_dim: int            # rotated ones
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float

    @staticmethod
    def from_reader(r: KeyReader) -> "LatentMixerConfig":
        rot = r.obj("rot")
        if rot is None:
            raise ConfigError(f"{r.where}: required key 'rot' is missing")
        c = LatentMixerConfig(
            heads=r.integer("heads", minimum=1), dim=r.integer("dim", minimum=1),
            rot_dim=r.integer("rot_dim", minimum=0), vdim=r.integer("vdim", minimum=1),
            kv_rank=r.integer("kv_rank", minimum=1), scale=r.number("scale", positive=True),
            rot_dims=rot.integer("dims", minimum=0), rot_base=rot.number("base", positive=True))
        if c.rot_dims % 2 or c.rot_dims > c.rot_dim:
            raise ConfigError(f"{r.where}: rot.dims {c.rot_dims} must be even and at most rot_dim {c.rot_dim}")
        return c

    def to_dict(self) -> dict:
        return dict(dim=self.dim, heads=self.heads, kv_rank=self.kv_rank,
                    rot=dict(base=self.rot_base, dims=self.rot_dims), rot_dim=self.rot_dim, scale=self.scale,
                    vdim=self.vdim)


@dataclass(frozen=True)
class ExpertMixtureConfig:
    experts: int
    identity: int
    top: int
    expert_ff: int
    shared_ff: int | None

    @staticmethod
    def from_reader(r: KeyReader) -> "ExpertMixtureConfig":
        kind = r.string("kind")
        if kind != "moe":
            raise ConfigError(f"{r.where}: feed-forward kind {kind!r} is not known; known: ['moe']")
        router, expert, shared = r.obj("router"), r.obj("expert"), r.obj("shared")
        if router is None or expert is None:
            raise ConfigError(f"{r.where}: 'router' and 'expert' are required")
        c = ExpertMixtureConfig(
            experts=router.integer("experts", minimum=0), identity=router.integer("identity", 0, minimum=0),
            top=router.integer("top", minimum=1), expert_ff=expert.integer("ff", minimum=1),
            shared_ff=shared.integer("ff", minimum=1) if shared is not None else None)
        if c.top > c.experts + c.identity:
            raise ConfigError(f"{r.where}: top {c.top} is more than the router's {c.experts + c.identity} outputs")
        return c

    def to_dict(self) -> dict:
        return dict(expert=dict(ff=self.expert_ff), kind="moe",
                    router=dict(experts=self.experts, identity=self.identity, top=self.top),
                    shared=dict(ff=self.shared_ff) if self.shared_ff else None)


@dataclass(frozen=True)
class DizatarLayerConfig:
    type: str
    mixer: LatentMixerConfig
    mlp: ExpertMixtureConfig | None

    MIXERS = ("latent_attention",)

    @staticmethod
    def from_reader(r: KeyReader) -> "DizatarLayerConfig":
        kind = r.string("type")
        if kind not in DizatarLayerConfig.MIXERS:
            raise ConfigError(f"{r.where}: layer type {kind!r} is not known; known: {list(DizatarLayerConfig.MIXERS)}")
        mixer, mlp = r.obj("mixer"), r.obj("mlp")
        if mixer is None:
            raise ConfigError(f"{r.where}: required key 'mixer' is missing")
        return DizatarLayerConfig(kind, LatentMixerConfig.from_reader(mixer),
                                  ExpertMixtureConfig.from_reader(mlp) if mlp is not None else None)

    def to_dict(self) -> dict:
        return dict(mixer=self.mixer.to_dict(), mlp=self.mlp.to_dict() if self.mlp else None, type=self.type)


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass
class DizatarConfig:
    architecture: str
    width: int
    vocab: int
    layers: tuple
    loop: LoopConfig | None
    norm_eps: float
    residual_mult: float = 1.0
    logit_softcap: float | None = None
    max_position: int = DEFAULT_MAX_POSITION
    eos_token_id: tuple = field(default_factory=tuple)

    ARCHITECTURE = "Dizatar"

    @staticmethod
    def from_dict(data: dict, where: str = "config.json") -> "DizatarConfig":
        r = KeyReader(data, where)
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers = tuple(DizatarLayerConfig.from_reader(KeyReader(x, f"{where}:layers[{i}]"))
                       for i, x in enumerate(raw_layers))
        norm = r.obj("norm")
        if norm is None:
            raise ConfigError(f"{where}: required key 'norm' is missing")
        loop = None
        lr = r.obj("loop")
        if lr is not None:
            loop = LoopConfig(lr.integer("start", minimum=0), lr.integer("stop", minimum=0),
                              lr.integer("times", minimum=1))
            if not loop.start <= loop.stop <= len(layers):          # an empty span (start == stop) loops nothing
                raise ConfigError(f"{where}: loop {loop.start}..{loop.stop} does not name layers of the {len(layers)}")
        cap = r.number("logit_softcap", None)
        return DizatarConfig(
            architecture=r.string("architecture", DizatarConfig.ARCHITECTURE),
            width=r.integer("width", minimum=1), vocab=r.integer("vocab", minimum=1), layers=layers, loop=loop,
            norm_eps=norm.number("eps", positive=True), residual_mult=r.number("residual_mult", 1.0),
            logit_softcap=cap if cap else None,
            max_position=r.integer("max_position", DEFAULT_MAX_POSITION, minimum=1),
            eos_token_id=r.int_list("eos_token_id", ()))

    def to_dict(self) -> dict:
        d = dict(architecture=self.architecture, layers=[x.to_dict() for x in self.layers],
                 logit_softcap=self.logit_softcap,
                 loop=dict(start=self.loop.start, stop=self.loop.stop, times=self.loop.times) if self.loop else None,
                 norm=dict(eps=self.norm_eps), residual_mult=self.residual_mult, vocab=self.vocab, width=self.width)
        if self.max_position != DEFAULT_MAX_POSITION:
            d["max_position"] = self.max_position
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d
