"""Small Nalizen configurations for the tests, their model folders (random weights in a temporary folder), and helpers
that run the engine and the plain implementation (tests/plain_nalizen.py) side by side.

The configurations differ from one another in every size: key and value sizes of a head that are equal and not, that
are and are not multiples of 8, one key/value head and as many as query heads, windows smaller and larger than a cache
page (of ONE position, and none at all), rotations of a whole head, of a part and none, frequencies rescaled and not,
layers that read another layer's keys and values through a wider, a narrower and an equal window, attention as the
first layer and as the last, layers without a feed-forward, routers that keep one expert, all experts, and the only
one, a token side input of one element, of many, and none."""
from __future__ import annotations

import functools
import json
import tempfile
from pathlib import Path

import numpy as np
import torch


def attention(heads, kv_heads, dim, vdim, window, scale, rot=None, base=10000.0, scaling=None, kv_from=None):
    m = dict(dim=dim, heads=heads, kv_heads=kv_heads, scale=scale, vdim=vdim)
    if window is not None:
        m["mask"] = dict(size=window)
    if rot:
        m["rot"] = dict(base=base, dims=rot)
        if scaling is not None:
            factor, low, high, original = scaling
            m["rot"]["scaling"] = dict(factor=factor, high=high, low=low, original=original)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="attention", mixer=m)


def hgrn2(heads, dim, vdim):
    return dict(type="hgrn2", mixer=dict(dim=dim, heads=heads, vdim=vdim))


def dense(ff):
    return dict(ff=ff, kind="dense")


def moe(ff, experts, top):
    return dict(expert=dict(ff=ff), kind="moe", router=dict(experts=experts, top=top))


def layer(mix, mlp=None):
    return dict(mix, mlp=mlp)


def config(vocab, width, layers, eps=1e-5, emb=1.0, side=None):
    d = dict(architecture="Nalizen", embedding=dict(scale=emb), layers=layers, norm=dict(eps=eps), vocab=vocab, width=width)
    if side:
        d["token_side"] = dict(dim=side)
    return d


_ROT_A = dict(rot=8, base=10000.0, scaling=(4.0, 1.0, 4.0, 64))
# A: recurrent layers around an attention layer whose pages a later layer reads through a WIDER window (21 and 50; pages
# of 16 divide neither); values smaller than keys, three query heads a key/value head; a layer without a feed-forward
CFG_A = config(211, 96, [
    layer(hgrn2(3, 20, 12), dense(160)),
    layer(attention(6, 2, 24, 16, 21, 0.21, **_ROT_A), moe(40, 6, 2)),
    layer(hgrn2(2, 8, 40), moe(24, 5, 3)),
    layer(attention(6, 2, 24, 16, 50, 0.21, kv_from=1, **_ROT_A)),
    layer(hgrn2(4, 16, 16), moe(40, 6, 2)),
], emb=2.5, side=5)

# B: attention first and last; no window at all; a window of ONE position; a rotation of the whole head, unscaled, and no
# rotation; as many key/value heads as heads, and one; a reader with a NARROWER window than the layer it reads; a router
# that keeps all its experts and one with a single expert; a side input of one element
CFG_B = config(300, 128, [
    layer(attention(4, 4, 16, 16, None, 0.3, rot=16, base=500.0), moe(24, 4, 4)),
    layer(attention(5, 1, 8, 40, 1, 0.35), dense(192)),
    layer(hgrn2(1, 64, 8), moe(56, 1, 1)),
    layer(attention(4, 4, 16, 16, 33, 0.3, rot=16, base=500.0, kv_from=0), moe(16, 3, 1)),
    layer(attention(2, 1, 32, 32, 4096, 0.15, rot=12, base=1e6, scaling=(8.0, 1.0, 32.0, 256)), dense(64)),
], emb=0.6, side=1)

# C: sizes that are multiples of nothing: width 72, vocabulary 101, heads of 5 and 9 and 7, seven experts of 9; a window
# equal to a page; readers of one layer's pages through equal windows; no side input
CFG_C = config(101, 72, [
    layer(hgrn2(3, 5, 7), dense(40)),
    layer(attention(3, 3, 10, 7, 16, 0.45, rot=6, base=77.0), moe(9, 7, 3)),
    layer(attention(3, 3, 10, 7, 16, 0.45, rot=6, base=77.0, kv_from=1), dense(24)),
    layer(hgrn2(9, 3, 5), moe(9, 7, 3)),
    layer(attention(3, 3, 10, 7, 16, 0.45, rot=6, base=77.0, kv_from=1)),
], eps=1e-6, emb=1.7)

# M: small, and of the sizes the tensor-core kernels of the bfloat16 engine take (keys and values of one size, a multiple
# of 16; a width of a multiple of 128; a side input of 16), run with pages of 64: windows longer and shorter than a page
CFG_M = config(180, 128, [
    layer(attention(4, 2, 32, 32, 70, 0.2, rot=16, scaling=(4.0, 1.0, 4.0, 64)), dense(96)),
    layer(hgrn2(2, 32, 64), moe(24, 4, 2)),
    layer(attention(4, 2, 32, 32, 33, 0.2, rot=16, scaling=(4.0, 1.0, 4.0, 64), kv_from=0), moe(32, 8, 3)),
    layer(attention(2, 1, 48, 48, 200, 0.15, rot=48, base=500000.0)),
], emb=1.5, side=16)

# W: not tiny: the sizes at which the products and the experts' grouped products run on their tensor-core kernels
CFG_W = config(256, 1024, [
    layer(hgrn2(8, 64, 128), dense(2048)),
    layer(attention(16, 4, 64, 64, 100, 0.125, rot=32, scaling=(8.0, 1.0, 4.0, 128)), moe(512, 8, 2)),
    layer(attention(16, 4, 64, 64, 4096, 0.125, rot=32, scaling=(8.0, 1.0, 4.0, 128), kv_from=1), moe(256, 16, 4)),
], side=16)

# O: a width and a vocabulary that are odd (no 8- or 16-byte row anywhere: every kernel's scalar form), odd head sizes
CFG_O = config(97, 37, [
    layer(attention(3, 1, 7, 5, 9, 0.4, rot=6, base=50.0, scaling=(2.0, 0.5, 2.0, 16)), moe(11, 5, 2)),
    layer(hgrn2(2, 9, 3), dense(21)),
    layer(attention(2, 1, 7, 5, 30, 0.4, rot=6, base=50.0, scaling=(2.0, 0.5, 2.0, 16), kv_from=0), dense(13)),
], emb=3.0, side=3)

CONFIGS = {"A": (CFG_A, 41), "B": (CFG_B, 42), "C": (CFG_C, 43), "M": (CFG_M, 44), "W": (CFG_W, 45), "O": (CFG_O, 46)}
PAGE_TOKENS = {"M": 64, "W": 64}          # (the other small configurations run with pages of 16)
_tmp = tempfile.TemporaryDirectory(prefix="fellm_b200_nalizen_")

# random weights as the framework's random mode makes them, then some scaled so that no mechanism hides behind small
# numbers: experts and dense feed-forwards whose outputs differ, routers whose logits differ, gates away from one half
SCALES = ((".mlp.e", 4.0), (".mlp.gate", 3.0), (".mlp.up", 3.0), (".mix.g", 6.0), (".mix.f", 8.0), (".mix.q", 3.0), (".mix.k", 3.0))


def write_folder(folder, cfg, seed, scales=SCALES):
    from fellm_b200.config.registry import config_from_dict
    from fellm_b200.models.model import build_model
    from fellm_b200.weights.random_init import random_tensors
    from fellm_b200.weights.safetensors_io import write_safetensors
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    arch, typed = config_from_dict(cfg)
    tensors = random_tensors(build_model(arch.build_spec(typed), "float32"), seed)
    for name in tensors:
        for pat, s in scales:
            if pat in name and tensors[name].dim() == 2:
                tensors[name] = (tensors[name].float() * s).bfloat16()
    (folder / "config.json").write_text(json.dumps(typed.to_dict(), indent=1))
    write_safetensors(folder / "model.safetensors", tensors)
    return str(folder)


@functools.lru_cache(maxsize=None)
def model_folder(name: str) -> str:
    cfg, seed = CONFIGS[name]
    return write_folder(Path(_tmp.name) / f"nalizen_{name}", cfg, seed)


def load_folder(folder):
    """(config dict, {name: float64 array}) read with the safetensors reader."""
    from fellm_b200.weights.safetensors_io import SafetensorsFile
    cfg = json.loads((Path(folder) / "config.json").read_text())
    f = SafetensorsFile(Path(folder) / "model.safetensors")
    w = {n: f.tensor(n).clone().double().numpy() for n in f.names()}
    f.close()
    return cfg, w


@functools.lru_cache(maxsize=None)
def plain_model(name: str):
    return load_folder(model_folder(name))


def tokens(name: str, length: int, seed: int):
    cfg, _ = CONFIGS[name]
    rng = np.random.default_rng(7000 + seed)
    return [int(t) for t in rng.integers(0, cfg["vocab"], size=length)]


def plain_run(cfg, w, toks) -> torch.Tensor:
    import plain_nalizen
    return torch.from_numpy(plain_nalizen.run(cfg, w, toks))


@functools.lru_cache(maxsize=None)
def plain_logits(name: str, length: int, seed: int) -> torch.Tensor:
    cfg, w = plain_model(name)
    return plain_run(cfg, w, tokens(name, length, seed))


def make_engine(name_or_folder: str, dtype: str, **opts):
    from fellm_b200.config.options import EngineOptions
    from fellm_b200.engine import Engine
    folder = model_folder(name_or_folder) if name_or_folder in CONFIGS else name_or_folder
    o = dict(dtype=dtype, n_ctx=1024, ctx_past_model=True, max_requests=4, max_tokens=2048,
             page_tokens=PAGE_TOKENS.get(name_or_folder, 16), cuda_graphs=False, n_batch=2048)
    o.update(opts)
    return Engine.open(folder, EngineOptions(**o))


def row_distances(got, want) -> torch.Tensor:
    """Row by row: the root mean square difference of the logits with their means taken off, relative to the root mean
    square of all the wanted logits."""
    got, want = got.double().cpu(), want.double().cpu()
    got = got - got.mean(-1, keepdim=True)
    want = want - want.mean(-1, keepdim=True)
    return (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()


def distance(got, want) -> float:
    return float(row_distances(got, want).max())


# (bfloat16: these models are 72 to 144 wide and norm every sublayer's OUTPUT: the rounding of a product of so few terms does
# not average out, and a small output is divided by its own size; the float32 engine is the sharp comparison)
LIMIT = {"float32": 1e-4, "bfloat16": 1e-1}


def assert_close(got, want, dtype: str, times: float = 1.0, note=None):
    """In 32-bit every row is within the limit.  In bfloat16 a router's close call may go the other way for a token
    (its input is rounded), and experts that differ by design then move that row, and faintly the rows that read it, far
    beyond rounding: nine rows in ten are within the limit and the median row within a third of it, which no fault of
    a mechanism passes (a fault moves every row)."""
    assert got.shape == want.shape, (got.shape, want.shape)
    d = row_distances(got, want)
    limit = LIMIT[dtype] * times
    if dtype == "float32":
        assert float(d.max()) < limit, (note, float(d.max()), int(d.argmax()))
    else:
        assert float(torch.quantile(d, 0.9)) < limit and float(d.median()) < limit / 3, (note, float(torch.quantile(d, 0.9)), float(d.median()))


def run_cuts(engine, req, toks, cuts):
    """Feeds toks in portions of the given sizes (the rest one by one) and returns the logits of every position."""
    from fellm_b200.engine import StepItem
    engine.add_request(req)
    out, at = [], 0
    sizes = list(cuts)
    while at < len(toks):
        n = sizes.pop(0) if sizes else 1
        n = min(n, len(toks) - at)
        out.append(engine.step([StepItem(req, toks[at:at + n], list(range(n)))]).clone())
        at += n
    engine.check_status()
    engine.release(req)
    return torch.cat(out)


def random_config(seed: int):
    """A configuration drawn at random: 1 to 6 layers of either kind in any order, heads and sizes that are and are not
    multiples of anything, windows from 1 to beyond the prompt or none, readers of earlier layers' pages, any
    feed-forward or none, a side input or none."""
    rng = np.random.default_rng(9100 + seed)
    pick = lambda xs: xs[int(rng.integers(0, len(xs)))]
    width = int(pick([48, 72, 96, 120, 144]))
    n_layers = int(rng.integers(1, 7))
    layers, owners = [], []
    for i in range(n_layers):
        if rng.random() < 0.5:
            mix = hgrn2(int(pick([1, 2, 3, 5])), int(pick([3, 4, 8, 16, 20, 48])), int(pick([2, 8, 12, 32, 33])))
        elif owners and rng.random() < 0.4:
            j = int(pick(owners))
            m = dict(layers[j]["mixer"])
            m["kv_from"] = j
            m["heads"] = m["kv_heads"] * int(pick([1, 2, 3]))
            m["scale"] = float(rng.uniform(0.05, 0.5))
            window = pick([1, 5, 16, 17, 40, 100, None])
            m.pop("mask", None)
            if window is not None:
                m["mask"] = dict(size=window)
            mix = dict(type="attention", mixer=m)
        else:
            G = int(pick([1, 2, 3]))
            dim = int(pick([4, 6, 8, 16, 24, 32, 48]))
            vdim = dim if rng.random() < 0.5 else int(pick([3, 8, 12, 16, 40]))
            rot = int(pick([0, 2, 4, dim, dim // 2 * 2]))
            scaling = None
            if rot and rng.random() < 0.6:
                scaling = (float(pick([2.0, 4.0, 8.0])), float(pick([0.5, 1.0])), float(pick([2.0, 4.0, 32.0])), float(pick([16, 64, 512])))
            mix = attention(G * int(pick([1, 2, 4])), G, dim, vdim, pick([1, 2, 15, 16, 17, 31, 64, 100, 1000, None]),
                            float(rng.uniform(0.05, 0.5)), rot=rot, base=float(pick([10.0, 10000.0, 5e5])), scaling=scaling)
            owners.append(i)
        r = rng.random()
        if r < 0.2:
            mlp = None
        elif r < 0.5:
            mlp = dense(int(pick([8, 24, 40, 64, 100])))
        else:
            experts = int(pick([1, 2, 3, 5, 8, 12]))
            mlp = moe(int(pick([8, 9, 16, 24, 40])), experts, int(rng.integers(1, experts + 1)))
        layers.append(layer(mix, mlp))
    return config(int(pick([50, 101, 128, 200, 333])), width, layers, eps=float(pick([1e-5, 1e-6])),
                  emb=float(rng.uniform(0.5, 8.0)), side=int(pick([0, 1, 4, 7, 16])))
