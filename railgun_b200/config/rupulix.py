"""Typed reading of a Rupulix model's config.json.

``layers`` lists the layers one by one: ``type`` names the mixer
("latent_attention" or "parallel"), ``mixer`` holds its sizes and ``mlp`` the
feed-forward (``kind`` "dense" with ``ff``; null for a layer without one).
``loop`` (``start``, ``stop``, ``times``) names a span of layers that runs
several times in a row.  ``streams`` is the number of copies of the residual
stream that the layers' hyper-connections mix (absent: one stream with plain
residual additions).  Constants: ``norm.eps``, ``logit_scale``, ``width``,
``vocab``.  ``architecture`` (a string) names the design; ``max_position`` is
optional (default 2^20: positions are computed, not tabulated).
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, KeyReader

DEFAULT_MAX_POSITION = 1 << 20


def _rotation(r: KeyReader, limit: int, what: str):
    """(dims, base) of a mixer's ``rot`` object; no object means no rotation."""
    rot = r.obj("rot")
    if rot is None:
        return 0, 10000.0
    dims, base = rot.integer("dims", minimum=0), rot.number("base", positive=True)
    if dims % 2 or dims > limit:
        raise ConfigError(f"{r.where}: rot.dims {dims} must be even and at most {what} {limit}")
    return dims, base


def _window(r: KeyReader) -> int:
    """``mask.size``: how many positions a query sees, itself included (0: all before it)."""
    mask = r.obj("mask")
    return mask.integer("size", minimum=1) if mask is not None else 0


def _rot_dict(dims, base):
    return dict(base=base, dims=dims)


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
    window: int

    @staticmethod
    def from_reader(r: KeyReader) -> "LatentMixerConfig":
        rot_dim = r.integer("rot_dim", minimum=0)
        dims, base = _rotation(r, rot_dim, "rot_dim")
        return LatentMixerConfig(
            heads=r.integer("heads", minimum=1), dim=r.integer("dim", minimum=1), rot_dim=rot_dim,
            vdim=r.integer("vdim", minimum=1), kv_rank=r.integer("kv_rank", minimum=1),
            scale=r.number("scale", positive=True), rot_dims=dims, rot_base=base, window=_window(r))

    def to_dict(self) -> dict:
        d = dict(dim=self.dim, heads=self.heads, kv_rank=self.kv_rank, rot=_rot_dict(self.rot_dims, self.rot_base),
                 rot_dim=self.rot_dim, scale=self.scale, vdim=self.vdim)
        if self.window:
            d["mask"] = dict(size=self.window)
        return d


@dataclass(frozen=True)
class TalkingAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float
    window: int

    @staticmethod
    def from_reader(r: KeyReader) -> "TalkingAttentionConfig":
        dim = r.integer("dim", minimum=1)
        dims, base = _rotation(r, dim, "dim")
        c = TalkingAttentionConfig(
            heads=r.integer("heads", minimum=1), kv_heads=r.integer("kv_heads", minimum=1), dim=dim,
            vdim=r.integer("vdim", minimum=1), scale=r.number("scale", positive=True), rot_dims=dims, rot_base=base,
            window=_window(r))
        if c.heads % c.kv_heads:
            raise ConfigError(f"{r.where}: {c.heads} heads cannot share {c.kv_heads} key/value heads")
        return c

    def to_dict(self) -> dict:
        d = dict(dim=self.dim, heads=self.heads, kv_heads=self.kv_heads, rot=_rot_dict(self.rot_dims, self.rot_base),
                 scale=self.scale, vdim=self.vdim)
        if self.window:
            d["mask"] = dict(size=self.window)
        return d


@dataclass(frozen=True)
class RecurrentConfig:
    width: int
    blocks: int
    conv: int               # taps of the causal convolution

    @staticmethod
    def from_reader(r: KeyReader) -> "RecurrentConfig":
        c = RecurrentConfig(width=r.integer("width", minimum=1), blocks=r.integer("blocks", minimum=1),
                            conv=r.integer("conv", minimum=1))
        if c.width % c.blocks:
            raise ConfigError(f"{r.where}: width {c.width} does not split into {c.blocks} equal blocks")
        return c

    def to_dict(self) -> dict:
        return dict(blocks=self.blocks, conv=self.conv, width=self.width)


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: TalkingAttentionConfig
    right: RecurrentConfig
    left_scale: float
    right_scale: float

    @staticmethod
    def from_reader(r: KeyReader) -> "ParallelMixerConfig":
        left, right = r.obj("left"), r.obj("right")
        if left is None or right is None:
            raise ConfigError(f"{r.where}: 'left' and 'right' are required")
        return ParallelMixerConfig(TalkingAttentionConfig.from_reader(left), RecurrentConfig.from_reader(right),
                                   r.number("left_scale", 1.0), r.number("right_scale", 1.0))

    def to_dict(self) -> dict:
        return dict(left=self.left.to_dict(), left_scale=self.left_scale, right=self.right.to_dict(),
                    right_scale=self.right_scale)


@dataclass(frozen=True)
class DenseMLPConfig:
    ff: int

    @staticmethod
    def from_reader(r: KeyReader) -> "DenseMLPConfig":
        kind = r.string("kind")
        if kind != "dense":
            raise ConfigError(f"{r.where}: feed-forward kind {kind!r} is not known; known: ['dense']")
        return DenseMLPConfig(ff=r.integer("ff", minimum=1))

    def to_dict(self) -> dict:
        return dict(ff=self.ff, kind="dense")


_MIXERS = {"latent_attention": LatentMixerConfig, "parallel": ParallelMixerConfig}


@dataclass(frozen=True)
class RupulixLayerConfig:
    type: str
    mixer: object
    mlp: DenseMLPConfig | None

    @staticmethod
    def from_reader(r: KeyReader) -> "RupulixLayerConfig":
        kind = r.string("type")
        if kind not in _MIXERS:
            raise ConfigError(f"{r.where}: layer type {kind!r} is not known; known: {sorted(_MIXERS)}")
        mixer, mlp = r.obj("mixer"), r.obj("mlp")
        if mixer is None:
            raise ConfigError(f"{r.where}: required key 'mixer' is missing")
        return RupulixLayerConfig(kind, _MIXERS[kind].from_reader(mixer),
                                  DenseMLPConfig.from_reader(mlp) if mlp is not None else None)

    def to_dict(self) -> dict:
        return dict(mixer=self.mixer.to_dict(), mlp=self.mlp.to_dict() if self.mlp else None, type=self.type)


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass
class RupulixConfig:
    architecture: str
    width: int
    vocab: int
    layers: tuple
    loop: LoopConfig | None
    norm_eps: float
    streams: int = 0                    # 0: one stream with plain residual additions
    logit_scale: float = 1.0
    max_position: int = DEFAULT_MAX_POSITION
    eos_token_id: tuple = field(default_factory=tuple)

    ARCHITECTURE = "Rupulix"

    @staticmethod
    def from_dict(data: dict, where: str = "config.json") -> "RupulixConfig":
        r = KeyReader(data, where)
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers = tuple(RupulixLayerConfig.from_reader(KeyReader(x, f"{where}:layers[{i}]"))
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
        return RupulixConfig(
            architecture=r.string("architecture", RupulixConfig.ARCHITECTURE),
            width=r.integer("width", minimum=1), vocab=r.integer("vocab", minimum=1), layers=layers, loop=loop,
            norm_eps=norm.number("eps", positive=True), streams=r.integer("streams", 0, minimum=1) or 0,
            logit_scale=r.number("logit_scale", 1.0),
            max_position=r.integer("max_position", DEFAULT_MAX_POSITION, minimum=1),
            eos_token_id=r.int_list("eos_token_id", ()))

    def to_dict(self) -> dict:
        d = dict(architecture=self.architecture, layers=[x.to_dict() for x in self.layers],
                 logit_scale=self.logit_scale,
                 loop=dict(start=self.loop.start, stop=self.loop.stop, times=self.loop.times) if self.loop else None,
                 norm=dict(eps=self.norm_eps), vocab=self.vocab, width=self.width)
        if self.streams:
            d["streams"] = self.streams
        if self.max_position != DEFAULT_MAX_POSITION:
            d["max_position"] = self.max_position
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d
