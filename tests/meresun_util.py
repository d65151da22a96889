"""Small Meresun configurations for the tests, their model folders (random weights in a temporary folder), and
helpers that run the engine and the plain implementation side by side.

The configurations differ from one another in every size: unrotated, rotated and value sizes of a head that are and
are not multiples of 8, latents smaller and larger than a head, windows smaller and larger than a cache page (and of
ONE position, and longer than any prompt), frequencies scaled and not, groups of experts of which one, some or all are
kept (and groups of one expert), layers without a feed-forward, a loop over the first, the last or all layers, one
norm group and several, a token side input of one element and of many, and none."""
from __future__ import annotations

import functools
import json
import tempfile
from pathlib import Path

import numpy as np
import torch


def mixer(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, scale, base=10000.0, scaling=None):
    m = dict(dim=dim, heads=heads, kv_rank=kv_rank, q_rank=q_rank, rot_dim=rot_dim, scale=scale, vdim=vdim)
    if window is not None:
        m["mask"] = dict(size=window)
    if rot_dim:
        m["rot"] = dict(base=base, dims=rot_dim)
        if scaling is not None:
            factor, original, fast, slow = scaling
            m["rot"]["scaling"] = dict(factor=factor, fast=fast, original=original, slow=slow)
    return m


def dense(ff):
    return dict(ff=ff, kind="dense")


def moe(ff, experts, top, groups=None, limit=0.3):
    router = dict(experts=experts, top=top)
    if groups is not None:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    return dict(expert=dict(ff=ff, limit=limit), kind="moe", router=router)


def layer(m, mlp=None):
    return dict(type="latent_attention", mixer=m, mlp=mlp)


def config(vocab, width, layers, loop=None, eps=1e-5, groups=1, emb=1.0, side=None):
    d = dict(architecture="Meresun", embedding=dict(scale=emb), layers=layers, norm=dict(eps=eps, groups=groups),
             vocab=vocab, width=width)
    if side:
        d["token_side"] = dict(dim=side)
    if loop is not None:
        d["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return d


# A: a loop of two passes over layers 1..2, a window of 21 (pages of 16 do not divide it) and one of 50, three norm
# groups, scaled frequencies whose ramp lies inside the pairs, six experts in three groups of which two are kept, a
# layer without a feed-forward
CFG_A = config(211, 96, [
    layer(mixer(3, 20, 8, 12, 24, 40, 21, 0.21, 10000.0, (4.0, 64, 8.0, 1.0)), moe(40, 6, 2, (3, 2))),
    layer(mixer(4, 16, 16, 24, 48, 32, 50, 0.17, 500000.0, (8.0, 256, 32.0, 1.0)), dense(160)),
    layer(mixer(2, 24, 4, 16, 16, 56, 21, 0.3)),
], loop=(1, 3, 2), groups=3, emb=2.5, side=5)

# B: no loop; a window of ONE position and a window longer than any prompt; no rotated part at all in one layer; one
# norm group; groups of ONE expert; every group kept; a side input of one element
CFG_B = config(300, 128, [
    layer(mixer(2, 40, 8, 40, 32, 24, 1, 0.15), moe(24, 4, 2, (4, 2), limit=0.2)),
    layer(mixer(5, 8, 0, 8, 20, 16, 4096, 0.35), dense(192)),
    layer(mixer(8, 16, 32, 16, 64, 64, 4096, 0.125, 1000.0, (2.0, 32, 4.0, 2.0)), moe(56, 6, 3, (2, 2), limit=5.0)),
    layer(mixer(1, 64, 16, 48, 8, 8, 33, 0.11), moe(16, 3, 1)),
], emb=0.6, side=1)

# C: the loop is the whole model, three passes; a window equal to a page; one head; no side input; two norm groups
CFG_C = config(128, 64, [
    layer(mixer(1, 32, 16, 64, 16, 48, 16, 0.18, 100.0, (16.0, 16, 2.0, 0.5)), moe(32, 2, 2, (1, 1))),
    layer(mixer(2, 16, 2, 4, 32, 24, 17, 0.25), dense(96)),
], loop=(0, 2, 3), eps=1e-6, groups=2)

# D: sizes that are multiples of nothing: width 72, vocabulary 101, heads of 5 + 6, values of 7, latents of 9 and 13,
# a loop of one pass over the last layer, seven experts of 9 without groups, four norm groups
CFG_D = config(101, 72, [
    layer(mixer(3, 5, 6, 7, 9, 13, 9, 0.45, 77.0), dense(40)),
    layer(mixer(3, 20, 2, 3, 11, 10, 15, 0.22), moe(9, 7, 3, limit=0.15)),
    layer(mixer(9, 3, 10, 20, 30, 21, 33, 0.22, 10000.0, (3.0, 40, 5.0, 0.8)), dense(24)),
], loop=(2, 3, 1), groups=4, emb=1.7, side=3)

# W: not tiny: the sizes at which the products run on their tensor-core kernels and the experts' grouped products on
# theirs; a latent wider than a head, as the design is used
CFG_W = config(256, 1024, [
    layer(mixer(16, 64, 32, 64, 384, 256, 100, 0.1, 10000.0, (8.0, 128, 32.0, 1.0)), dense(2048)),
    layer(mixer(8, 128, 64, 128, 512, 192, 4096, 0.07), moe(512, 8, 2, (4, 2), limit=0.5)),
], groups=2, side=16)

# M: small, and of the sizes the tensor-core kernels of the bfloat16 engine take (latents of a multiple of 32, cache rows
# of a multiple of 16, a width of a multiple of 128, a side input of 16), run with pages of 64: windows longer and
# shorter than a page, a layer without a rotated part's scaling, a loop of two passes over the first two layers
CFG_M = config(180, 128, [
    layer(mixer(5, 24, 16, 16, 40, 64, 70, 0.2, 10000.0, (4.0, 64, 8.0, 1.0)), dense(96)),
    layer(mixer(3, 16, 32, 24, 24, 32, 33, 0.25), moe(24, 4, 2, (2, 1), limit=0.3)),
    layer(mixer(2, 32, 16, 40, 32, 96, 200, 0.15, 500000.0, (8.0, 256, 32.0, 1.0))),
], loop=(0, 2, 2), groups=2, emb=1.5, side=16)

CONFIGS = {"A": (CFG_A, 31), "B": (CFG_B, 32), "C": (CFG_C, 33), "D": (CFG_D, 34), "W": (CFG_W, 35), "M": (CFG_M, 36)}
PAGE_TOKENS = {"M": 64}          # (the other small configurations run with pages of 16)
_tmp = tempfile.TemporaryDirectory(prefix="fellm_b200_meresun_")

# random weights as the framework's random mode makes them, then some scaled so that no mechanism hides behind small
# numbers: experts that reach their clamps, a router whose logits differ, side inputs and gates that matter
SCALES = ((".mlp.e", 6.0), (".mlp.router", 1.0), (".rg", 8.0), (".mlp.up", 3.0), (".mix.dq", 2.0), (".mix.dkv", 2.0))


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
    return write_folder(Path(_tmp.name) / f"meresun_{name}", cfg, seed)


def load_folder(folder):
    """(config dict, {name: float64 tensor}) read with the safetensors reader."""
    from fellm_b200.weights.safetensors_io import SafetensorsFile
    cfg = json.loads((Path(folder) / "config.json").read_text())
    f = SafetensorsFile(Path(folder) / "model.safetensors")
    w = {n: f.tensor(n).clone().double() for n in f.names()}
    f.close()
    return cfg, w


@functools.lru_cache(maxsize=None)
def plain_model(name: str):
    return load_folder(model_folder(name))


def tokens(name: str, length: int, seed: int):
    cfg, _ = CONFIGS[name]
    rng = np.random.default_rng(4000 + seed)
    return [int(t) for t in rng.integers(0, cfg["vocab"], size=length)]


@functools.lru_cache(maxsize=None)
def plain_logits(name: str, length: int, seed: int) -> torch.Tensor:
    import plain_meresun
    cfg, w = plain_model(name)
    return plain_meresun.forward(tokens(name, length, seed), w, cfg)


def make_engine(name_or_folder: str, dtype: str, **opts):
    from fellm_b200.config.options import EngineOptions
    from fellm_b200.engine import Engine
    folder = model_folder(name_or_folder) if name_or_folder in CONFIGS else name_or_folder
    o = dict(dtype=dtype, n_ctx=1024, ctx_past_model=True, max_requests=4, max_tokens=2048,
             page_tokens=PAGE_TOKENS.get(name_or_folder, 16), cuda_graphs=False, n_batch=2048)
    o.update(opts)
    return Engine.open(folder, EngineOptions(**o))


def distance(got, want) -> float:
    """The largest, over the rows, root mean square difference of the logits with their means taken off,
    relative to the root mean square of the wanted logits."""
    got, want = got.double().cpu(), want.double().cpu()
    got = got - got.mean(-1, keepdim=True)
    want = want - want.mean(-1, keepdim=True)
    return float(((got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()).max())


LIMIT = {"float32": 1e-4, "bfloat16": 6e-2}


def row_distances(got, want) -> torch.Tensor:
    """distance() row by row."""
    got, want = got.double().cpu(), want.double().cpu()
    got = got - got.mean(-1, keepdim=True)
    want = want - want.mean(-1, keepdim=True)
    return (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()


def assert_close(got, want, dtype: str, times: float = 1.0, note=None):
    """In 32-bit every row is within the limit.  In bfloat16 a router's close call may go the other way for a token
    (its input is rounded), and experts that differ by design then move that row, and faintly the rows that read it, far
    beyond rounding: nine rows in ten are within the limit and the median row within a third of it, which no fault of
    a mechanism passes (a fault moves every row)."""
    d = row_distances(got, want)
    limit = LIMIT[dtype] * times
    if dtype == "float32":
        assert float(d.max()) < limit, (note, float(d.max()))
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
    """A configuration drawn at random: 1 to 5 layers, heads and sizes that are and are not multiples of anything,
    windows from 1 to beyond the prompt, any feed-forward or none, a loop or none, any norm groups, a side input or none."""
    rng = np.random.default_rng(9000 + seed)
    pick = lambda xs: xs[int(rng.integers(0, len(xs)))]
    groups = int(pick([1, 1, 2, 3, 4, 6]))
    width = int(pick([48, 72, 96, 120, 144]))
    n_layers = int(rng.integers(1, 6))
    layers = []
    for _ in range(n_layers):
        dr = int(pick([0, 2, 4, 8, 10, 16, 32]))
        scaling = None
        if dr and rng.random() < 0.6:
            scaling = (float(pick([2.0, 4.0, 8.0, 40.0])), int(pick([16, 64, 1024, 4096])), float(pick([4.0, 32.0])), float(pick([0.5, 1.0, 2.0])))
        m = mixer(int(pick([1, 2, 3, 4, 6, 7])), int(pick([4, 5, 8, 16, 24, 32, 48])), dr, int(pick([3, 8, 12, 16, 40, 64])),
                  int(pick([4, 9, 16, 32, 48])), int(pick([6, 8, 16, 24, 40, 72])), pick([1, 2, 5, 15, 16, 17, 31, 40, 64, 100, 1000, None]),
                  float(rng.uniform(0.05, 0.5)), float(pick([10.0, 10000.0, 5e5])), scaling)
        r = rng.random()
        if r < 0.2:
            mlp = None
        elif r < 0.5:
            mlp = dense(int(pick([8, 24, 40, 64, 100, 160])))
        else:
            count = int(pick([1, 2, 3, 4]))
            per = int(pick([1, 2, 3, 4]))
            keep = int(rng.integers(1, count + 1))
            top = int(rng.integers(1, per * keep + 1))
            mlp = moe(int(pick([8, 9, 16, 24, 40, 64])), count * per, top, (count, keep) if rng.random() < 0.8 else None,
                      limit=float(pick([0.1, 0.3, 1.0, 7.0])))
        layers.append(layer(m, mlp))
    loop = None
    if rng.random() < 0.6:
        a = int(rng.integers(0, n_layers))
        b = int(rng.integers(a + 1, n_layers + 1))
        loop = (a, b, int(rng.integers(1, 4)))
    return config(int(pick([50, 101, 128, 200, 333])), width, layers, loop=loop, eps=float(pick([1e-5, 1e-6])), groups=groups,
                  emb=float(rng.uniform(0.3, 3.0)), side=int(pick([0, 1, 4, 7, 16])))
