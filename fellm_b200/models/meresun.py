"""Meresun: how the design is put together from parts.

A layer is `h = norm1(x); x += mixer(h) * sigmoid(W_1 h + b_1) + ff(h) * sigmoid(W_2 h + b_2)`: one norm (RMS in
groups, parts/rmsnorm.py), mixer and feed-forward side by side, each through a gate of its own on its way into the
stream (the 'parallel_gated' arrangement, parts/residual_gate.py); then every token adds an input of its own, read
from a slice of a table shared by the layers (parts/token_side.py).  A layer may have no feed-forward.
  mixer         latent attention: queries through a normed latent, one normed key-value latent and one rotated key
                part per token shared by the heads, frequencies scaled for long contexts, a sliding window, a sink
                per head in the softmax's denominator                                     (parts/latent_attention.py)
  feed-forward  dense with a polynomial activation over unit powers (parts/polynorm.py), or routed experts with
                sigmoid scores, a correction for the choice, groups of experts ranked by their two best, weights
                over their sum, clamped gated experts                                     (parts/moe.py)
`loop` repeats a run of layers with the same weights, each pass with caches of its own; every pass but the first
opens with x <- x + (the embedding's output) (parts/connector.py, 'add_embedding').  The embedding is scaled.

Tensor names of the safetensors file: embed, side.embed, head, final.norm, and per layer i: l<i>.norm1,
l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,o}, l<i>.mlp.{up,down,act} (dense) or l<i>.mlp.{router,correction}
and l<i>.mlp.e<j>.{gate,up,down} (experts), l<i>.rg1{,.b}, l<i>.rg2{,.b}, l<i>.side.{gate,proj,norm}.
"""
from __future__ import annotations

from ..config.meresun import NAME, MeresunConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run

MAX_POSITION = 1 << 20        # nothing ends a context but memory
GROUP_BEST = 2                # a group of experts is ranked by the sum of this many of its largest choice scores
EXPERT_ALPHA = 1.702          # an expert's gate is g sigmoid(EXPERT_ALPHA g)
SIDE_TABLE = "side.embed"


def _norm(name: str, d: int, eps: float, groups: int) -> PartSpec:
    if groups == 1:
        return PartSpec.make("rmsnorm", names={"weight": name}, size=d, eps=eps)
    return PartSpec.make("rmsnorm_groups", names={"weight": name}, size=d, eps=eps, groups=groups)


def _mixer(p: str, d: int, m, eps: float) -> PartSpec:
    names = {f"{t}.weight": p + t for t in ("dq", "uq", "dkv", "uk", "uv", "o")}
    names.update({"dq.norm": p + "dq.norm", "dkv.norm": p + "dkv.norm", "sink": p + "sink"})
    position = PartSpec.make("none")
    if m.rot_dims:
        s = m.scaling
        position = PartSpec.make("rope", rot_dim=m.rot_dims, theta=m.rot_base, pairing="adjacent", table64=True,
                                 scaling=None if s is None else (s.factor, s.original, s.fast, s.slow))
    return PartSpec.make("latent_attention", names=names, size=d, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim,
                         v_dim=m.vdim, q_rank=m.q_rank, kv_rank=m.kv_rank, scale=m.scale, norm_eps=eps,
                         position=position, window=m.window, sink=True)


def _feed_forward(p: str, d: int, f, eps: float) -> PartSpec:
    if f.kind == "dense":
        return PartSpec.make("polynorm", names={"up.weight": p + "up", "down.weight": p + "down", "act": p + "act"},
                             size=d, ff=f.ff, eps=eps)
    names = {"router.weight": p + "router", "correction": p + "correction"}
    for e in range(f.experts):
        names.update({f"e{e}.{t}.weight": f"{p}e{e}.{t}" for t in ("gate", "up", "down")})
    return PartSpec.make("moe", names=names, size=d, ff=f.ff, experts=f.experts, top=f.top, renormalize=True,
                         score="sigmoid", correction=True,
                         groups=(f.groups, f.keep, GROUP_BEST) if f.groups else None,
                         act=("clamped", f.limit, EXPERT_ALPHA))


def build_spec(cfg: MeresunConfig) -> ModelSpec:
    d, eps, groups = cfg.width, cfg.norm_eps, cfg.norm_groups
    layers = []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        ffn = None if L.mlp is None else _feed_forward(p + "mlp.", d, L.mlp, eps)
        names = {"0.weight": p + "rg1", "0.bias": p + "rg1.b"}
        if ffn is not None:
            names.update({"1.weight": p + "rg2", "1.bias": p + "rg2.b"})
        gate = PartSpec.make("sigmoid", names=names, size=d, sublayers=1 if ffn is None else 2)
        side = None
        if cfg.side_dim:
            side = PartSpec.make("token_gated", names={"gate.weight": p + "side.gate", "proj.weight": p + "side.proj",
                                                       "norm.weight": p + "side.norm"},
                                 size=d, dim=cfg.side_dim, offset=i * cfg.side_dim, eps=eps, table=SIDE_TABLE)
        layers.append(LayerSpec(norm1=_norm(p + "norm1", d, eps, groups), mixer=_mixer(p + "mix.", d, L.mixer, eps),
                                norm2=None, ffn=ffn, arrangement="parallel_gated", gate=gate, side=side))
    schedule, connectors = None, []
    if cfg.loop is not None:
        lp = cfg.loop
        connectors = [PartSpec.make("add_embedding", size=d)]
        schedule = [Run(i) for i in range(lp.start)]
        for t in range(lp.times):
            schedule += [Run(i, before=(0, t) if (i == lp.start and t > 0) else None) for i in range(lp.start, lp.stop)]
        schedule += [Run(i) for i in range(lp.stop, len(cfg.layers))]
    shared = []
    if cfg.side_dim:
        shared = [PartSpec.make("table", names={"weight": SIDE_TABLE}, vocab=cfg.vocab, width=len(cfg.layers) * cfg.side_dim)]
    return ModelSpec(architecture=NAME, hidden_size=d, vocab_size=cfg.vocab, max_position=MAX_POSITION,
                     embedding=PartSpec.make("table", names={"weight": "embed"}, vocab=cfg.vocab, size=d,
                                             scale=cfg.embedding_scale),
                     layers=layers, final_norm=_norm("final.norm", d, eps, groups),
                     head=PartSpec.make("linear", names={"weight": "head"}, vocab=cfg.vocab, size=d, tied=False),
                     schedule=schedule or [], connectors=connectors, shared=shared)


register_architecture(NAME, MeresunConfig.from_dict, build_spec)
