"""Typed configuration of the Nalizen design, read from its config.json.

The file is nested like Robazen's, Samusun's and Meresun's: `layers` is a list of {type, mixer, mlp}, `norm` = {eps};
beside those `embedding.scale` and `token_side.dim`.  A layer's `type` is 'attention' or 'hgrn2'; its `mlp` is null, a
dense gated feed-forward {kind: dense, ff} or routed experts {kind: moe, expert: {ff}, router: {experts, top}}.  An
attention mixer may read the keys and values of an earlier attention layer (`kv_from`).  Every size and every constant
that can differ between two models of the design is read here; a missing or ill-typed key raises ConfigError with the
key's path.  What a file leaves out does not exist: no window (`mask`), no rotation (`rot`), no scaling of its
frequencies (`rot.scaling`), no token side input; `kv_heads` defaults to `heads`, `vdim` to `dim`, `embedding.scale`
to 1.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from .errors import ConfigError
from .robazen import _get

NAME = "Nalizen"
LAYER_TYPES = ("attention", "hgrn2")


@dataclass(frozen=True)
class BandScaling:
    """Rotary frequencies rescaled by wavelength: a wavelength below original / high keeps its frequency, one above
    original / low has it divided by `factor`, the band between is blended linearly in original / wavelength."""
    factor: float
    low: float
    high: float
    original: float

    @staticmethod
    def read(d, where):
        c = BandScaling(factor=_get(d, "factor", float, where), low=_get(d, "low", float, where),
                        high=_get(d, "high", float, where), original=_get(d, "original", float, where))
        if c.factor <= 0 or c.low <= 0 or c.high <= 0 or c.original <= 0:
            raise ConfigError(f"config.json: '{where}' needs positive factor, low, high and original")
        return c

    def to_dict(self):
        return dict(factor=self.factor, high=self.high, low=self.low, original=self.original)


@dataclass(frozen=True)
class GatedAttentionConfig:
    """The 'attention' mixer: grouped queries, rotation of a head's leading elements, unit norm of q and k behind the
    rotation, a sliding window, a sigmoid gate on the heads' outputs; `kv_from`: the layer whose keys and values it reads."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    rot_dims: int
    rot_base: float
    scaling: Optional[BandScaling]
    kv_from: Optional[int]

    @staticmethod
    def read(d, where):
        mask = _get(d, "mask", dict, where, required=False)
        rot = _get(d, "rot", dict, where, required=False)
        scaling = None if rot is None else _get(rot, "scaling", dict, where + ".rot", required=False)
        heads = _get(d, "heads", int, where, positive=True)
        dim = _get(d, "dim", int, where, positive=True)
        c = GatedAttentionConfig(
            heads=heads, kv_heads=_get(d, "kv_heads", int, where, positive=True, required=False, default=heads),
            dim=dim, vdim=_get(d, "vdim", int, where, positive=True, required=False, default=dim),
            scale=_get(d, "scale", float, where),
            window=None if mask is None else _get(mask, "size", int, where + ".mask", positive=True),
            rot_dims=0 if rot is None else _get(rot, "dims", int, where + ".rot"),
            rot_base=10000.0 if rot is None else _get(rot, "base", float, where + ".rot"),
            scaling=None if scaling is None else BandScaling.read(scaling, where + ".rot.scaling"),
            kv_from=_get(d, "kv_from", int, where, required=False))
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: '{where}.heads' ({c.heads}) is not a multiple of kv_heads ({c.kv_heads})")
        if c.rot_dims % 2 or not 0 <= c.rot_dims <= c.dim:
            raise ConfigError(f"config.json: '{where}.rot.dims' ({c.rot_dims}) must be even and at most dim ({c.dim})")
        if c.rot_base <= 0:
            raise ConfigError(f"config.json: '{where}.rot.base' must be positive, got {c.rot_base}")
        return c

    def to_dict(self):
        d = dict(dim=self.dim, heads=self.heads, kv_heads=self.kv_heads, scale=self.scale, vdim=self.vdim)
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        if self.window is not None:
            d["mask"] = dict(size=self.window)
        if self.rot_dims:
            d["rot"] = dict(base=self.rot_base, dims=self.rot_dims)
            if self.scaling is not None:
                d["rot"]["scaling"] = self.scaling.to_dict()
        return d


@dataclass(frozen=True)
class Hgrn2Config:
    """The 'hgrn2' mixer: a matrix state per head whose forget gate also weighs what is written."""
    heads: int
    dim: int
    vdim: int

    @staticmethod
    def read(d, where):
        return Hgrn2Config(heads=_get(d, "heads", int, where, positive=True), dim=_get(d, "dim", int, where, positive=True),
                           vdim=_get(d, "vdim", int, where, positive=True))

    def to_dict(self):
        return dict(dim=self.dim, heads=self.heads, vdim=self.vdim)


@dataclass(frozen=True)
class FeedForwardConfig:
    """kind 'dense': one gated feed-forward of `ff`; 'moe': `experts` plain feed-forwards of `ff` each, `top` a token."""
    kind: str
    ff: int
    experts: int = 0
    top: int = 0

    @staticmethod
    def read(d, where):
        kind = _get(d, "kind", str, where)
        if kind == "dense":
            return FeedForwardConfig("dense", _get(d, "ff", int, where, positive=True))
        if kind == "moe":
            router = _get(d, "router", dict, where)
            c = FeedForwardConfig("moe", _get(_get(d, "expert", dict, where), "ff", int, where + ".expert", positive=True),
                                  _get(router, "experts", int, where + ".router", positive=True),
                                  _get(router, "top", int, where + ".router", positive=True))
            if c.top > c.experts:
                raise ConfigError(f"config.json: '{where}.router.top' ({c.top}) is above experts ({c.experts})")
            return c
        raise ConfigError(f"config.json: '{where}.kind' is {kind!r}; known: dense, moe")

    def to_dict(self):
        if self.kind == "dense":
            return dict(ff=self.ff, kind="dense")
        return dict(expert=dict(ff=self.ff), kind="moe", router=dict(experts=self.experts, top=self.top))


@dataclass(frozen=True)
class NalizenLayer:
    type: str
    mixer: object
    mlp: Optional[FeedForwardConfig]          # None: the layer has no feed-forward

    def to_dict(self):
        return dict(mixer=self.mixer.to_dict(), mlp=None if self.mlp is None else self.mlp.to_dict(), type=self.type)


@dataclass
class NalizenConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float = 1.0
    side_dim: int = 0
    layers: List[NalizenLayer] = field(default_factory=list)

    @staticmethod
    def from_dict(d: dict) -> "NalizenConfig":
        vocab = _get(d, "vocab", int, "", positive=True)
        width = _get(d, "width", int, "", positive=True)
        eps = _get(_get(d, "norm", dict, ""), "eps", float, "norm")
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
            m = _get(L, "mixer", dict, where)
            mixer = (GatedAttentionConfig if kind == "attention" else Hgrn2Config).read(m, where + ".mixer")
            mlp = None if L.get("mlp") is None else FeedForwardConfig.read(L["mlp"], where + ".mlp")
            layers.append(NalizenLayer(kind, mixer, mlp))
        for i, L in enumerate(layers):
            j = getattr(L.mixer, "kv_from", None)
            if j is None:
                continue
            where = f"layers[{i}].mixer.kv_from"
            if not 0 <= j < i or layers[j].type != "attention":
                raise ConfigError(f"config.json: '{where}' ({j}) must name an earlier attention layer")
            src = layers[j].mixer
            if src.kv_from is not None:
                raise ConfigError(f"config.json: '{where}' names layer {j}, which keeps no keys and values of its own")
            same = (src.kv_heads, src.dim, src.vdim, src.rot_dims, src.rot_base, src.scaling) == \
                   (L.mixer.kv_heads, L.mixer.dim, L.mixer.vdim, L.mixer.rot_dims, L.mixer.rot_base, L.mixer.scaling)
            if not same:
                raise ConfigError(f"config.json: '{where}': layer {j}'s key/value heads, sizes and rotation differ from layer {i}'s")
        return NalizenConfig(vocab=vocab, width=width, norm_eps=eps, embedding_scale=emb_scale, side_dim=side_dim,
                             layers=layers)

    def to_dict(self) -> dict:
        d = dict(architecture=NAME, embedding=dict(scale=self.embedding_scale), layers=[L.to_dict() for L in self.layers],
                 norm=dict(eps=self.norm_eps), vocab=self.vocab, width=self.width)
        if self.side_dim:
            d["token_side"] = dict(dim=self.side_dim)
        return d
