"""Typed configuration of the Meresun design, read from its config.json.

The file is nested like Robazen's and Samusun's: `layers` is a list of {type, mixer, mlp}, `loop` = {start, stop,
times} names a run of layers that is repeated with the same weights, `norm` = {eps, groups}; beside those
`embedding.scale` and `token_side.dim`.  A layer's `type` is 'latent_attention'; its `mlp` is null, a dense
feed-forward {kind: dense, ff} or routed experts {kind: moe, expert: {ff, limit}, router: {experts, top, groups:
{count, keep}}}.  Every size and every constant that can differ between two models of the design is read here; a
missing or ill-typed key raises ConfigError with the key's path.  What a file leaves out does not exist: no window
(`mask`), no rotation (`rot`), no scaling of its frequencies (`rot.scaling`), no groups of experts, no token side
input, no loop; `norm.groups` and `embedding.scale` default to 1.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from .errors import ConfigError
from .robazen import LoopConfig, _get

NAME = "Meresun"
LAYER_TYPES = ("latent_attention",)


@dataclass(frozen=True)
class FrequencyScaling:
    """Rotary frequencies stretched for longer contexts: pairs that turn more than `fast` times over `original`
    positions keep their frequency, pairs that turn fewer than `slow` times have it divided by `factor`."""
    factor: float
    original: float
    fast: float
    slow: float

    @staticmethod
    def read(d, where):
        c = FrequencyScaling(factor=_get(d, "factor", float, where), original=_get(d, "original", float, where),
                             fast=_get(d, "fast", float, where), slow=_get(d, "slow", float, where))
        if c.factor <= 0 or c.original <= 0 or c.fast <= 0 or c.slow <= 0:
            raise ConfigError(f"config.json: '{where}' needs positive factor, original, fast and slow")
        return c

    def to_dict(self):
        return dict(factor=self.factor, fast=self.fast, original=self.original, slow=self.slow)


@dataclass(frozen=True)
class LatentAttentionConfig:
    """The 'latent_attention' mixer: queries through a latent of q_rank, keys and values through one latent of
    kv_rank and one rotated key part of rot_dim shared by the heads; a window; a sink per head."""
    heads: int
    dim: int                  # unrotated query / key elements of a head
    rot_dim: int              # rotated ones
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: Optional[int]
    rot_dims: int             # how many of the rot_dim elements are rotated (0: none)
    rot_base: float
    scaling: Optional[FrequencyScaling]

    @staticmethod
    def read(d, where):
        mask = _get(d, "mask", dict, where, required=False)
        rot = _get(d, "rot", dict, where, required=False)
        rot_dim = _get(d, "rot_dim", int, where, required=False, default=0)
        scaling = None if rot is None else _get(rot, "scaling", dict, where + ".rot", required=False)
        c = LatentAttentionConfig(
            heads=_get(d, "heads", int, where, positive=True), dim=_get(d, "dim", int, where, positive=True),
            rot_dim=rot_dim, vdim=_get(d, "vdim", int, where, positive=True),
            q_rank=_get(d, "q_rank", int, where, positive=True), kv_rank=_get(d, "kv_rank", int, where, positive=True),
            scale=_get(d, "scale", float, where),
            window=None if mask is None else _get(mask, "size", int, where + ".mask", positive=True),
            rot_dims=0 if rot is None else _get(rot, "dims", int, where + ".rot"),
            rot_base=10000.0 if rot is None else _get(rot, "base", float, where + ".rot"),
            scaling=None if scaling is None else FrequencyScaling.read(scaling, where + ".rot.scaling"))
        if c.rot_dim < 0:
            raise ConfigError(f"config.json: '{where}.rot_dim' must not be negative, got {c.rot_dim}")
        if c.rot_dims % 2 or not 0 <= c.rot_dims <= c.rot_dim:
            raise ConfigError(f"config.json: '{where}.rot.dims' ({c.rot_dims}) must be even and at most rot_dim ({c.rot_dim})")
        if c.rot_base <= 0:
            raise ConfigError(f"config.json: '{where}.rot.base' must be positive, got {c.rot_base}")
        return c

    def to_dict(self):
        d = dict(dim=self.dim, heads=self.heads, kv_rank=self.kv_rank, q_rank=self.q_rank, rot_dim=self.rot_dim,
                 scale=self.scale, vdim=self.vdim)
        if self.window is not None:
            d["mask"] = dict(size=self.window)
        if self.rot_dims:
            d["rot"] = dict(base=self.rot_base, dims=self.rot_dims)
            if self.scaling is not None:
                d["rot"]["scaling"] = self.scaling.to_dict()
        return d


@dataclass(frozen=True)
class FeedForwardConfig:
    """kind 'dense': one feed-forward of `ff` with the polynomial activation; 'moe': `experts` clamped gated
    feed-forwards of `ff` each, `top` a token, chosen inside `keep` of `groups` groups (groups 0: no groups)."""
    kind: str
    ff: int
    limit: float = 0.0
    experts: int = 0
    top: int = 0
    groups: int = 0
    keep: int = 0

    @staticmethod
    def read(d, where):
        kind = _get(d, "kind", str, where)
        if kind == "dense":
            return FeedForwardConfig("dense", _get(d, "ff", int, where, positive=True))
        if kind == "moe":
            expert = _get(d, "expert", dict, where)
            router = _get(d, "router", dict, where)
            groups = _get(router, "groups", dict, where + ".router", required=False)
            c = FeedForwardConfig("moe", _get(expert, "ff", int, where + ".expert", positive=True),
                                  limit=_get(expert, "limit", float, where + ".expert"),
                                  experts=_get(router, "experts", int, where + ".router", positive=True),
                                  top=_get(router, "top", int, where + ".router", positive=True),
                                  groups=0 if groups is None else _get(groups, "count", int, where + ".router.groups", positive=True),
                                  keep=0 if groups is None else _get(groups, "keep", int, where + ".router.groups", positive=True))
            if not c.limit > 0:
                raise ConfigError(f"config.json: '{where}.expert.limit' must be positive, got {c.limit}")
            if c.top > c.experts:
                raise ConfigError(f"config.json: '{where}.router.top' ({c.top}) is above experts ({c.experts})")
            if c.groups:
                if c.experts % c.groups or c.keep > c.groups:
                    raise ConfigError(f"config.json: '{where}.router.groups' ({c.groups}, keep {c.keep}) does not fit "
                                      f"{c.experts} experts")
                if c.top > (c.experts // c.groups) * c.keep:
                    raise ConfigError(f"config.json: '{where}.router.top' ({c.top}) is above the experts of {c.keep} groups")
            return c
        raise ConfigError(f"config.json: '{where}.kind' is {kind!r}; known: dense, moe")

    def to_dict(self):
        if self.kind == "dense":
            return dict(ff=self.ff, kind="dense")
        router = dict(experts=self.experts, top=self.top)
        if self.groups:
            router["groups"] = dict(count=self.groups, keep=self.keep)
        return dict(expert=dict(ff=self.ff, limit=self.limit), kind="moe", router=router)


@dataclass(frozen=True)
class MeresunLayer:
    type: str
    mixer: LatentAttentionConfig
    mlp: Optional[FeedForwardConfig]          # None: the layer has no feed-forward

    def to_dict(self):
        return dict(mixer=self.mixer.to_dict(), mlp=None if self.mlp is None else self.mlp.to_dict(), type=self.type)


@dataclass
class MeresunConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int = 1
    embedding_scale: float = 1.0
    side_dim: int = 0                          # 0: no token side input
    layers: List[MeresunLayer] = field(default_factory=list)
    loop: Optional[LoopConfig] = None

    @staticmethod
    def from_dict(d: dict) -> "MeresunConfig":
        vocab = _get(d, "vocab", int, "", positive=True)
        width = _get(d, "width", int, "", positive=True)
        norm = _get(d, "norm", dict, "")
        eps = _get(norm, "eps", float, "norm")
        groups = _get(norm, "groups", int, "norm", positive=True, required=False, default=1)
        if width % groups:
            raise ConfigError(f"config.json: 'norm.groups' ({groups}) does not divide width ({width})")
        emb = _get(d, "embedding", dict, "", required=False, default={})
        emb_scale = _get(emb, "scale", float, "embedding", required=False, default=1.0)
        side = _get(d, "token_side", dict, "", required=False)
        side_dim = 0 if side is None else _get(side, "dim", int, "token_side", positive=True)
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]"
            kind = _get(L, "type", str, where)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: '{where}.type' is {kind!r}; known: {', '.join(LAYER_TYPES)}")
            mixer = LatentAttentionConfig.read(_get(L, "mixer", dict, where), where + ".mixer")
            mlp = None if L.get("mlp") is None else FeedForwardConfig.read(L["mlp"], where + ".mlp")
            layers.append(MeresunLayer(kind, mixer, mlp))
        loop = None
        if d.get("loop") is not None:
            lp = _get(d, "loop", dict, "")
            loop = LoopConfig(_get(lp, "start", int, "loop"), _get(lp, "stop", int, "loop"),
                              _get(lp, "times", int, "loop", positive=True))
            if not 0 <= loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json: 'loop' names layers {loop.start}..{loop.stop - 1} of {len(layers)}")
        return MeresunConfig(vocab=vocab, width=width, norm_eps=eps, norm_groups=groups, embedding_scale=emb_scale,
                             side_dim=side_dim, layers=layers, loop=loop)

    def to_dict(self) -> dict:
        d = dict(architecture=NAME, embedding=dict(scale=self.embedding_scale), layers=[L.to_dict() for L in self.layers],
                 norm=dict(eps=self.norm_eps, groups=self.norm_groups), vocab=self.vocab, width=self.width)
        if self.side_dim:
            d["token_side"] = dict(dim=self.side_dim)
        if self.loop is not None:
            d["loop"] = dict(start=self.loop.start, stop=self.loop.stop, times=self.loop.times)
        return d
