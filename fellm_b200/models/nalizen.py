"""Nalizen: how the design is put together from parts.

A layer is `x += LN1(mixer(shift(x))); x += LN2(ff(x)); x += side(x, token)`: the sublayers read the residual stream
itself and a LayerNorm with weight and bias stands on each sublayer's OUTPUT (the 'outnorm' arrangement,
parts/layernorm.py); in front of every mixer the stream is mixed with the previous token's (parts/shifted.py); after
the feed-forward every token adds an input of its own, read from a slice of a table shared by the layers
(parts/token_side.py).  A layer may have no feed-forward.
  mixer 'attention'  grouped queries, rotation of a head's leading elements (pairs i, i + r/2) with frequencies
                     rescaled by wavelength, q and k over their root mean square behind the rotation, a sliding
                     window, a sigmoid gate on the heads' outputs; a layer may read the keys and values of an
                     earlier attention layer (`kv_from`: a schedule entry with cache_of)      (parts/attention.py)
  mixer 'hgrn2'      a matrix state per head whose forget gate also weighs what is written     (parts/hgrn2.py)
  feed-forward       dense, W_down (gelu_tanh(W_gate x) * (W_up x)) (parts/swiglu.py), or routed plain experts
                     W_down relu(W_up x)^2 with a biased router and the softmax over the chosen logits (parts/moe.py)
The embedding is scaled; the head is the embedding matrix itself, without the scale, behind the final LayerNorm.

Tensor names of the safetensors file: embed, side.embed, final.norm{,.b}, and per layer i: l<i>.norm1{,.b},
l<i>.norm2{,.b}, l<i>.shift, l<i>.mix.{q,k,v,g,o} (attention; no k, v where the layer reads another's) or
l<i>.mix.{q,f,f.b,lower,v,norm,o} (hgrn2), l<i>.mlp.{gate,up,down} (dense) or l<i>.mlp.{router,router.b} and
l<i>.mlp.e<j>.{up,down} (experts), l<i>.side.{gate,proj,norm}.
"""
from __future__ import annotations

from ..config.nalizen import NAME, NalizenConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run

MAX_POSITION = 1 << 20        # nothing ends a context but memory: windows slide and states have a fixed size
SIDE_TABLE = "side.embed"


def _norm(name: str, d: int, eps: float) -> PartSpec:
    return PartSpec.make("layernorm", names={"weight": name, "bias": name + ".b"}, size=d, eps=eps)


def _attention(p: str, d: int, m, eps: float, cache_window) -> PartSpec:
    names = {"q_proj.weight": p + "q", "k_proj.weight": p + "k", "v_proj.weight": p + "v", "out_gate.weight": p + "g",
             "out_proj.weight": p + "o"}
    position = PartSpec.make("none")
    if m.rot_dims:
        s = m.scaling
        position = PartSpec.make("rope", rot_dim=m.rot_dims, theta=m.rot_base, pairing="split_half",
                                 bands=None if s is None else (s.factor, s.low, s.high, s.original),
                                 table64=True)
    return PartSpec.make("attention", names=names, size=d, heads=m.heads, kv_heads=m.kv_heads, head_dim=m.dim,
                         v_dim=m.vdim, qk_norm=False, unit_qk_norm=True, out_gate=True, norm_eps=eps, position=position,
                         window=m.window, cache_window=cache_window, scale=m.scale, shares_cache=m.kv_from is not None)


def _hgrn2(p: str, d: int, m, eps: float) -> PartSpec:
    names = {"q.weight": p + "q", "f.weight": p + "f", "f.bias": p + "f.b", "lower": p + "lower", "v.weight": p + "v",
             "norm.weight": p + "norm", "o.weight": p + "o"}
    return PartSpec.make("hgrn2", names=names, size=d, heads=m.heads, key_dim=m.dim, value_dim=m.vdim, norm_eps=eps)


def _feed_forward(p: str, d: int, f) -> PartSpec:
    if f.kind == "dense":
        return PartSpec.make("swiglu", names={"gate.weight": p + "gate", "up.weight": p + "up", "down.weight": p + "down"},
                             size=d, ff=f.ff, act="gelu_tanh")
    names = {"router.weight": p + "router", "router.bias": p + "router.b"}
    for e in range(f.experts):
        names.update({f"e{e}.{t}.weight": f"{p}e{e}.{t}" for t in ("up", "down")})
    return PartSpec.make("moe", names=names, size=d, ff=f.ff, experts=f.experts, top=f.top, renormalize=True,
                         router_bias=True, plain="relu2")


def _kept_windows(cfg: NalizenConfig):
    """Per attention layer that keeps pages: the window they are kept for, the widest among the layer itself and the
    layers that read its pages (None: no window, nothing is given back before the request ends)."""
    kept = {}
    for i, L in enumerate(cfg.layers):
        if L.type != "attention":
            continue
        src = i if L.mixer.kv_from is None else L.mixer.kv_from
        w = L.mixer.window
        if src not in kept:
            kept[src] = w
        elif kept[src] is not None:
            kept[src] = None if w is None else max(kept[src], w)
    return kept


def build_spec(cfg: NalizenConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    kept = _kept_windows(cfg)
    layers, schedule = [], []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        if L.type == "attention":
            own = L.mixer.kv_from is None
            inner = _attention(p + "mix.", d, L.mixer, eps, kept[i] if own else "same")
            schedule.append(Run(i, cache_of=L.mixer.kv_from))          # (layers run once each: entry j is layer j)
        else:
            inner = _hgrn2(p + "mix.", d, L.mixer, eps)
            schedule.append(Run(i))
        mixer = PartSpec.make("token_shifted", names={"shift": p + "shift"}, size=d, inner=inner)
        ffn = None if L.mlp is None else _feed_forward(p + "mlp.", d, L.mlp)
        side = None
        if cfg.side_dim:
            side = PartSpec.make("token_gated", names={"gate.weight": p + "side.gate", "proj.weight": p + "side.proj",
                                                       "norm.weight": p + "side.norm"},
                                 size=d, dim=cfg.side_dim, offset=i * cfg.side_dim, eps=eps, table=SIDE_TABLE)
        layers.append(LayerSpec(norm1=_norm(p + "norm1", d, eps), mixer=mixer,
                                norm2=None if ffn is None else _norm(p + "norm2", d, eps), ffn=ffn,
                                arrangement="outnorm", side=side))
    shared = []
    if cfg.side_dim:
        shared = [PartSpec.make("table", names={"weight": SIDE_TABLE}, vocab=cfg.vocab, width=len(cfg.layers) * cfg.side_dim)]
    return ModelSpec(architecture=NAME, hidden_size=d, vocab_size=cfg.vocab, max_position=MAX_POSITION,
                     embedding=PartSpec.make("table", names={"weight": "embed"}, vocab=cfg.vocab, size=d,
                                             scale=cfg.embedding_scale),
                     layers=layers, final_norm=_norm("final.norm", d, eps),
                     head=PartSpec.make("linear", names={"weight": "head"}, vocab=cfg.vocab, size=d, tied=True),
                     schedule=schedule, shared=shared)


register_architecture(NAME, NalizenConfig.from_dict, build_spec)
