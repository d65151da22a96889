"""Meresun on the GPU against the plain implementation (tests/plain_meresun.py).

First each mechanism alone, through its kernel's Python face with inputs made so that a fault shows (norm groups of
very different magnitude, one old key that would win the softmax if the window let it in, a sink that outweighs every
key, experts whose outputs differ by orders of magnitude and reach their clamps, choice scores that are all negative);
then whole models of four small configurations and a wide one: whole prompts, layer by layer, prompts against
token-by-token decoding, portions down to two tokens, unequal batches against each request alone, pages and slots that
are freed and come again, long decoding past every window, and greedy generation through the scheduler and the
command line."""
from __future__ import annotations

import copy
import json
import math
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import meresun_util as U
import plain_meresun as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _i32(xs):
    return torch.tensor(xs, dtype=torch.int32, device=DEV)


# ----------------------------------------------------------------------------- mechanisms alone

@pytest.mark.parametrize("T,d,groups", [(1, 96, 3), (5, 72, 4), (40, 128, 1), (3, 250, 2), (2, 2048, 8), (7, 6, 6)])
def test_norm_in_groups(T, d, groups):
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(d)
    mags = torch.tensor([10.0 ** (k - 1) for k in range(groups)]).repeat_interleave(d // groups)
    x = torch.randn(T, d, generator=g) * mags                         # parts of very different size: one root for all would show
    w = torch.randn(d, generator=g)
    want = P.grouped_rms_norm(x.double(), w.double(), 1e-6, groups)
    got = ops.rmsnorm_groups(x.to(DEV), w.to(DEV), 1e-6, groups, torch.float32)
    assert (got.double().cpu() - want).abs().max() < 1e-5 * float(want.abs().max())
    rows = [T - 1, 0]
    got = ops.rmsnorm_groups(x.to(DEV), w.to(DEV), 1e-6, groups, torch.bfloat16, rows=_i32(rows))
    assert (got.double().cpu() - want[rows]).abs().max() < 1e-2 * float(want.abs().max())


@pytest.mark.parametrize("T,F", [(1, 40), (6, 160), (3, 2048), (2, 9), (70, 384)])
def test_polynomial_activation(T, F):
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(F)
    z = torch.randn(T, F, generator=g) * 3.0
    coef = torch.tensor([0.7, -1.3, 0.4, 0.25])
    want = P.poly_norm(z.double(), coef.double(), 1e-5)
    got = ops.poly_norm(z.to(DEV), coef.to(DEV), 1e-5, torch.float32)
    assert (got.double().cpu() - want).abs().max() < 1e-5 * float(want.abs().max())
    got = ops.poly_norm(z.to(DEV), coef.to(DEV), 1e-5, torch.bfloat16)
    assert (got.double().cpu() - want).abs().max() < 1e-2 * float(want.abs().max())
    # each power has a root mean square of its own: a row of one large element has N(z) = N(z^3) there, up to sign
    z = torch.zeros(1, F)
    z[0, 3] = -50.0
    got = ops.poly_norm(z.to(DEV), torch.tensor([1.0, 10.0, 100.0, 0.5], device=DEV), 0.0, torch.float32).cpu()
    r = math.sqrt(F)
    assert abs(float(got[0, 3]) - (-r + 10 * r - 100 * r + 0.5)) < 1e-3 * r and float(got[0, 0]) == 0.5


def test_gated_sum_of_the_sublayers():
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(5)
    T, d = 9, 72
    x, a, b = (torch.randn(T, d, generator=g) for _ in range(3))
    zg = torch.randn(T, 2 * d + 8, generator=g) * 4
    want2 = x.double() + a.double() * torch.sigmoid(zg[:, :d].double()) + b.double() * torch.sigmoid(zg[:, d:2 * d].double())
    got = ops.gated_add(x.to(DEV).clone(), [a.to(DEV), b.to(DEV)], zg.to(DEV))
    assert (got.double().cpu() - want2).abs().max() < 1e-5
    want1 = x.double() + a.double() * torch.sigmoid(zg[:, :d].double())
    got = ops.gated_add(x.to(DEV).clone(), [a.to(DEV)], zg.to(DEV))
    assert (got.double().cpu() - want1).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,d,m,layer,n_layers", [(1, 96, 5, 1, 3), (7, 72, 1, 0, 2), (30, 320, 16, 3, 4), (3, 1024, 64, 2, 3)])
def test_token_side_input(dtype, T, d, m, layer, n_layers):
    """The layer's own part of the table (the parts beside it hold numbers a thousand times larger), gated by the stream,
    projected, over its root mean square, times the norm's weight, added to the stream."""
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(d + m)
    vocab = 37
    table = torch.randn(vocab, n_layers * m, generator=g) * 1000.0
    table[:, layer * m:(layer + 1) * m] = torch.randn(vocab, m, generator=g)
    W = {"side.embed": table.to(dtype).double(), "gate": (torch.randn(m, d, generator=g) * 0.3).to(dtype).double(),
         "proj": (torch.randn(d, m, generator=g) * 0.3).to(dtype).double(), "norm": torch.randn(d, generator=g).double()}
    x = torch.randn(T, d, generator=g)
    toks = [int(t) for t in torch.randint(0, vocab, (T,), generator=g)]
    toks[0] = vocab - 1
    want = x.double() + P.token_side_input(x.double(), toks, W, "", layer, m, 1e-6)
    got = ops.token_side(x.to(DEV).clone(), _i32(toks), W["side.embed"].to(dtype).to(DEV), layer * m, W["gate"].to(dtype).to(DEV),
                         W["proj"].to(dtype).to(DEV), W["norm"].float().to(DEV), 1e-6)
    # (bfloat16: the gate's product reads x rounded, as every product of the engine does)
    assert (got.double().cpu() - want).abs().max() < (1e-4 if dtype == torch.float32 else 3e-2 * max(1.0, float(want.abs().max())))


@pytest.mark.parametrize("n,base,scaling", [(8, 100.0, (4.0, 64, 8.0, 1.0)), (32, 250000.0, (6.0, 2048, 24.0, 1.0)), (6, 10.0, (2.0, 1.0, 1.0, 1.0)),
                                            (16, 10000.0, None), (64, 1e6, (40.0, 4096, 32.0, 1.0)), (2, 50.0, (3.0, 16, 4.0, 0.5))])
def test_scaled_frequencies_of_the_position_part(n, base, scaling):
    from fellm_b200.parts.base import build_part
    from fellm_b200.parts.spec import PartSpec
    part = build_part("position", PartSpec.make("rope", rot_dim=n, theta=base, pairing="adjacent", table64=True, scaling=scaling), "float32")
    sc = None if scaling is None else dict(zip(("factor", "original", "fast", "slow"), scaling))
    f, mag = P.scaled_frequencies(n, base, sc)
    assert torch.equal(part.inv_freq.cpu(), torch.tensor(f, dtype=torch.float64).float())
    assert abs(float(getattr(part, "magnitude", 1.0)) - mag) < 1e-12


def _latent_case(H, dn, dr, dv, rq, rk, n_rot, seed, dtype, sharp=None):
    """Random tensors of one latent-attention layer in the plain implementation's names, rounded to `dtype`."""
    g = torch.Generator().manual_seed(seed)
    d = 64
    r = lambda *s, k=1.0: (torch.randn(*s, generator=g) * k).to(dtype).double()
    W = {"dq": r(rq, d, k=0.2), "dq.norm": torch.rand(rq, generator=g).double() + 0.5, "uq": r(H * (dn + dr), rq, k=0.4),
         "dkv": r(rk + dr, d, k=0.2), "dkv.norm": torch.rand(rk, generator=g).double() + 0.5, "uk": r(H * dn, rk, k=0.4),
         "uv": r(H * dv, rk, k=0.4), "sink": torch.randn(H, generator=g).double(), "o": r(d, H * dv, k=0.3)}
    if sharp:
        W["uq"], W["uk"] = W["uq"] * sharp, W["uk"] * sharp
    return W, d


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dn,dr,dv,rq,rk,n_rot,window,page", [
    (3, 20, 8, 12, 24, 40, 8, 21, 16), (2, 40, 8, 40, 32, 24, 8, 1, 16), (5, 8, 0, 8, 20, 16, 0, None, 16), (1, 64, 16, 48, 8, 8, 16, 33, 32),
    (4, 16, 16, 24, 48, 32, 16, 16, 16), (3, 5, 6, 7, 9, 13, 6, 17, 16), (8, 16, 32, 16, 64, 64, 32, 64, 64), (2, 24, 10, 16, 16, 56, 4, 15, 16)])
def test_latent_attention_kernels_against_per_head_keys_and_values(dtype, H, dn, dr, dv, rq, rk, n_rot, window, page):
    """The kernels between the layer's products (the norms of both latents, the rotation of the key part and of the
    queries' rotated parts, the cache row, the queries taken into the latent's space, attention over the cached rows
    with a sink, the values read out of the latent) against the plain mixer, which writes every head's keys and values
    out.  The sinks outweigh most keys; in 32-bit the queries and keys are scaled so that the softmax is sharp: the key just
    outside the window must not count and the oldest inside must.  Rows come as two requests whose pages interleave,
    in portions that end before, on and behind the edges of pages and windows, single rows among them."""
    from fellm_b200 import ops
    from fellm_b200.parts.base import build_part
    from fellm_b200.parts.spec import PartSpec
    T = min(2 * max(window or 40, page) + 7, 140)
    W, d = _latent_case(H, dn, dr, dv, rq, rk, n_rot, 11 * H + dn, dtype, sharp=4.0 if dtype == torch.float32 else None)
    W["sink"] = W["sink"] + 2.0
    m = dict(heads=H, dim=dn, rot_dim=dr, vdim=dv, q_rank=rq, kv_rank=rk, scale=0.3)
    scaling = (4.0, 32, 8.0, 1.0) if n_rot >= 8 else None
    if window is not None:
        m["mask"] = dict(size=window)
    if n_rot:
        m["rot"] = dict(base=100.0, dims=n_rot)
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    freq, mag = None, 1.0
    if n_rot:
        part = build_part("position", PartSpec.make("rope", rot_dim=n_rot, theta=100.0, pairing="adjacent", table64=True, scaling=scaling), "float32")
        freq, mag = part.inv_freq.to(DEV), float(part.magnitude)
    n_pages = -(-T // page)
    pool = torch.zeros(2 * n_pages + 1, 2, page * (rk + dr), dtype=dtype, device=DEV)      # two layers a page; this one is layer 1
    table = torch.full((2, n_pages), -1, dtype=torch.int32, device=DEV)
    for r in range(2):
        table[r] = torch.arange(n_pages, dtype=torch.int32) * 2 + (1 - r)
    cache = SimpleNamespace(pool=pool, block_table=table, page_tokens=page, layer=1)
    dev = lambda t, dt=dtype: t.to(dt).to(DEV)
    down = dev(torch.cat([W["dq"], W["dkv"]], 0))
    ukT = dev(W["uk"].view(H, dn, rk).transpose(1, 2).contiguous())
    uv = dev(W["uv"].view(H, dv, rk).contiguous())
    g = torch.Generator().manual_seed(window or 0)
    for r in range(2):
        h = torch.randn(T, d, generator=g).to(dtype)
        want = P.latent_attention_mixer(h.double(), {**W, "o": torch.eye(H * dv, dtype=torch.float64)}, "", m, 1e-5)      # before W_o
        got, at = [], 0
        for n in [1, 2, page - 1, 1, 1, (window or 7) + 1, 2, T]:
            n = min(max(n, 1), T - at)
            if n <= 0:
                break
            pos, slot = _i32(list(range(at, at + n))), _i32([r] * n)
            z = (dev(h[at:at + n]).float() @ down.float().T).contiguous()
            cq = ops.latent_prep(z, 0, rq, rq, rk, rq + rk, dr, dev(W["dq.norm"], torch.float32), dev(W["dkv.norm"], torch.float32), 1e-5,
                                 freq, n_rot, mag, pos, slot, cache, dtype)
            q = (cq.float() @ dev(W["uq"]).float().T).to(dtype).contiguous()
            qa = torch.zeros(n, H * (rk + dr), dtype=dtype, device=DEV)
            ops.head_gemm(q, ukT, qa, a_head=dn + dr, out_head=rk + dr)
            ops.latent_rotate_q(q, H, dn, dr, qa, rk, freq, n_rot, mag, pos)
            a = ops.paged_attention_general(qa, H, rk + dr, 0, pool, table, pos, slot, 1, page, 1, 0.3, window=window,
                                            warps=1 + (window or 2) % 4, sinks=dev(W["sink"], torch.float32), out_dim=rk)
            o = torch.empty(n, H * dv, dtype=dtype, device=DEV)
            ops.head_gemm(a, uv, o, a_head=rk, out_head=dv)
            got.append(o)
            at += n
        got = torch.cat(got).double().cpu()
        assert float(pool[:, 0].float().abs().sum()) == 0.0                                   # the other layer's records are untouched
        tol = 2e-4 if dtype == torch.float32 else 6e-2          # (bfloat16: the latent, both queries and the read-out are rounded)
        assert got.shape == want.shape
        assert (got - want).abs().max() < tol * max(1.0, float(want.abs().max())), (r, float((got - want).abs().max()))


def _latent_pool(rows, page, n_req, g):
    """Cache rows [n_req][T][D] bfloat16 -> (pool of one layer, pages in a random order and interleaved between the requests, block table)."""
    T, D = rows.shape[1], rows.shape[2]
    n_pages = -(-T // page)
    perm = torch.randperm(n_req * n_pages + 2, generator=g)[:n_req * n_pages].view(n_req, n_pages)
    pool = torch.full((n_req * n_pages + 2, 1, page * D), float("nan"), dtype=torch.bfloat16, device=DEV)       # bits of pages never written
    padded = torch.full((n_req, n_pages * page, D), float("nan"), dtype=torch.bfloat16)
    padded[:, :T] = rows
    for r in range(n_req):
        pool[perm[r].to(DEV), 0] = padded[r].view(n_pages, page * D).to(DEV)
    return pool, perm.to(torch.int32).to(DEV)


@pytest.mark.parametrize("H,rk,dr,window,page,T", [(3, 32, 16, 21, 64, 150), (6, 64, 0, None, 64, 200), (16, 512, 64, 100, 64, 260), (5, 96, 16, 64, 128, 300),
                                                  (20, 128, 32, 65, 64, 140), (1, 192, 64, 1, 64, 70), (8, 256, 32, 129, 256, 400)])
def test_latent_attention_on_tensor_cores(H, rk, dr, window, page, T):
    """The tensor-core kernel against the float32 kernel on the same bfloat16 rows and queries: two requests whose pages
    interleave (pages that hold NaN behind a request's end), portions that start and end before, on and behind the
    edges of pages, key tiles and windows, single tokens (with the key walk split and not) beside portions in one step,
    sinks that outweigh most keys, and scores scaled so that the softmax is sharp: the oldest key a window keeps must
    count and the one before it must not."""
    from fellm_b200 import ops
    D = rk + dr
    g = torch.Generator().manual_seed(H * 1000 + rk + T)
    rows = torch.randn(2, T, D, generator=g).bfloat16()
    q = (torch.randn(2, T, H, D, generator=g) * 1.5).bfloat16()
    if window is not None and window > 1:
        for r in range(2):
            for i in range(window, T, 7):          # query i points at the oldest key it sees and, twice as hard, at the one before it
                q[r, i, 0] = (rows[r, i - window + 1].float() * 0.8 + rows[r, i - window].float() * 1.6).bfloat16()
    sinks = (torch.randn(H, generator=g) + 2.0).to(DEV)
    pool, table = _latent_pool(rows, page, 2, g)
    pool32 = torch.nan_to_num(pool.float(), nan=0.0)
    scale = 2.0 / math.sqrt(D)
    flat = q.view(2, T, H * D).to(DEV)

    def both(items):
        """items: [(request, first position, rows)] of one step -> (tensor cores, float32 kernel)"""
        pos = _i32([p for r, a, n in items for p in range(a, a + n)])
        slot = _i32([r for r, a, n in items for _ in range(n)])
        qa = torch.cat([flat[r, a:a + n] for r, a, n in items]).contiguous()
        starts = _i32([0] + list(np.cumsum([n for _, _, n in items])))
        got = ops.latent_attention(qa, H, rk, dr, pool, table, pos, slot, starts, len(items), max(n for _, _, n in items),
                                   max(a + n for _, a, n in items), 0, page, scale, window=window, sinks=sinks)
        want = ops.paged_attention_general(qa.float(), H, D, 0, pool32, table, pos, slot, 0, page, 1, scale, window=window, warps=2,
                                           sinks=sinks, out_dim=rk)
        return got.float(), want

    steps, at = [], 0
    for n in [1, 2, 29, 1, 31, 1, 1, 64, 3, (window or 40) + 1, 2, T]:
        n = min(n, T - at)
        if n <= 0:
            break
        steps.append([(0, at, n), (1, at, n)] if n > 2 else [(1, at, n), (0, at, n)])
        at += n
    steps.append([(0, T - 1, 1), (1, 5, 9)])                                   # a single token beside a portion
    steps.append([(0, T - 1, 1)])                                              # one token alone: its key walk is split
    steps.append([(1, T // 2, 1), (0, T - 3, 1)])
    for items in steps:
        got, want = both(items)
        assert torch.isfinite(got).all(), items
        err = (got - want).abs().max()
        assert err < 2e-2 * max(1.0, float(want.abs().max())), (items, float(err))
    if dr:
        # the queries' rotated parts read from the query product's rows and rotated inside the kernel: the same as
        # rotating them into place in front of it
        dn, n_rot = 24, dr - 8 * (H % 2)                                    # (heads of 24 + dr; all or all but 8 elements rotated)
        freq = (1.0 / (50.0 ** (torch.arange(n_rot // 2, dtype=torch.float32) / max(n_rot // 2, 1)))).to(DEV)
        for items in ([(0, 3, 60), (1, 0, 9)], [(1, T - 1, 1), (0, 17, 1)]):
            n_tok = sum(n for _, _, n in items)
            pos = _i32([p for r, a, n in items for p in range(a, a + n)])
            slot = _i32([r for r, a, n in items for _ in range(n)])
            starts = _i32([0] + list(np.cumsum([n for _, _, n in items])))
            qp = (torch.randn(n_tok, H * (dn + dr) + 8, generator=g) * 1.5).bfloat16().to(DEV)[:, :H * (dn + dr)]      # rows wider than the heads
            qa = (torch.randn(n_tok, H, rk, generator=g) * 1.5).bfloat16().to(DEV)
            full = torch.zeros(n_tok, H, D, dtype=torch.bfloat16, device=DEV)
            full[:, :, :rk] = qa
            full = full.view(n_tok, H * D)
            ops.latent_rotate_q(qp, H, dn, dr, full, rk, freq, n_rot, 1.07, pos)
            args = (pool, table, pos, slot, starts, len(items), max(n for _, _, n in items), max(a + n for _, a, n in items), 0, page, scale)
            a = ops.latent_attention(full, H, rk, dr, *args, window=window, sinks=sinks).float()
            b = ops.latent_attention(qa.view(n_tok, H * rk).contiguous(), H, rk, dr, *args, window=window, sinks=sinks,
                                     q_rot=(qp, dn + dr, dn, freq, n_rot, 1.07)).float()
            assert torch.isfinite(b).all() and (a - b).abs().max() < 1e-2 * max(1.0, float(a.abs().max())), items
    if window is not None and window > 1:
        # a window one position longer lets the key before the oldest in: the rows that point at it change
        i = window + 7 * ((T - 1 - window) // 7)
        qa = flat[0, i:i + 1].contiguous()
        args = (pool, table, _i32([i]), _i32([0]), _i32([0, 1]), 1, 1, i + 1, 0, page, scale)
        a = ops.latent_attention(qa, H, rk, dr, *args, window=window, sinks=sinks).float()
        b = ops.latent_attention(qa, H, rk, dr, *args, window=window + 1, sinks=sinks).float()
        assert float((a - b)[0, :rk].abs().max()) > 0.1


@pytest.mark.parametrize("T,H,N,K,a_head,out_head", [(1, 3, 40, 16, 24, 48), (70, 6, 96, 64, 96, 128), (300, 16, 512, 128, 192, 576), (9, 2, 8, 24, 24, 8)])
def test_head_products_on_tensor_cores(T, H, N, K, a_head, out_head):
    """One product per head on column blocks of the same rows, blocks wider than the product's operands: what lies
    between the blocks of the result stays as it was."""
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(T + N)
    a = torch.randn(T, H * a_head, generator=g).bfloat16()
    w = (torch.randn(H, N, K, generator=g) * 0.2).bfloat16()
    out = torch.full((T, H * out_head), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.head_gemm(a.to(DEV), w.to(DEV), out, a_head=a_head, out_head=out_head)
    want = torch.full((T, H * out_head), 7.0, dtype=torch.float64)
    for h in range(H):
        want[:, h * out_head:h * out_head + N] = a[:, h * a_head:h * a_head + K].double() @ w[h].double().T
    assert (out.double().cpu() - want).abs().max() < 2e-2 * float(want.abs().max())


@pytest.mark.parametrize("T,d,m,layer,n_layers", [(1, 64, 16, 1, 3), (37, 128, 32, 0, 2), (300, 1024, 64, 2, 3), (16, 2048, 48, 1, 2), (17, 192, 16, 0, 1), (9, 1024, 64, 0, 2), (3, 384, 80, 1, 2)])
def test_token_side_input_on_tensor_cores(T, d, m, layer, n_layers):
    """The side input's kernel for bfloat16 tables (16 rows a block; 16 warps instead of 8 for a single block of a
    width that is a multiple of 128): a last block that is not full, rows whose x differ by orders of magnitude, the
    layer's own part of the table."""
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(d + m)
    vocab = 37
    table = torch.randn(vocab, n_layers * m, generator=g) * 1000.0
    table[:, layer * m:(layer + 1) * m] = torch.randn(vocab, m, generator=g)
    W = {"side.embed": table.bfloat16().double(), "gate": (torch.randn(m, d, generator=g) * 0.3).bfloat16().double(),
         "proj": (torch.randn(d, m, generator=g) * 0.3).bfloat16().double(), "norm": torch.randn(d, generator=g).double()}
    x = (torch.randn(T, d, generator=g) * (10.0 ** torch.randint(-1, 2, (T, 1), generator=g))).bfloat16().float()
    toks = [int(t) for t in torch.randint(0, vocab, (T,), generator=g)]
    toks[0] = vocab - 1
    want = x.double() + P.token_side_input(x.double(), toks, W, "", layer, m, 1e-6)
    got = ops.token_side(x.to(DEV).clone(), _i32(toks), W["side.embed"].bfloat16().to(DEV), layer * m, W["gate"].bfloat16().to(DEV),
                         W["proj"].bfloat16().to(DEV), W["norm"].float().to(DEV), 1e-6)
    assert (got.double().cpu() - want).abs().max() < 3e-2 * max(1.0, float(want.abs().max()))
    # with the layer's gated results handed on: the same as adding them first
    for n_sub in (1, 2):
        ys = [torch.randn(T, d, generator=g).to(DEV) for _ in range(n_sub)]
        zg = (torch.randn(T, 2 * d + 4, generator=g) * 3.0).to(DEV)
        base = ops.gated_add(x.to(DEV).clone(), ys, zg)
        want2 = base.double().cpu() + P.token_side_input(base.double().cpu(), toks, W, "", layer, m, 1e-6)
        got2 = ops.token_side(x.to(DEV).clone(), _i32(toks), W["side.embed"].bfloat16().to(DEV), layer * m, W["gate"].bfloat16().to(DEV),
                              W["proj"].bfloat16().to(DEV), W["norm"].float().to(DEV), 1e-6, pending=(ys, zg))
        assert (got2.double().cpu() - want2).abs().max() < 3e-2 * max(1.0, float(want2.abs().max())), n_sub


def test_a_sink_counts_once_and_unscaled():
    """One key (the row's own) with a score of exactly 0: the output is the value over 1 + exp(sink), whatever the scale."""
    from fellm_b200 import ops
    H, D, page = 3, 8, 16
    pool = torch.zeros(2, 1, page * D, device=DEV)
    key = torch.arange(1, D + 1, dtype=torch.float32)
    pool[1, 0, :D] = key.to(DEV)
    table = _i32([[1]])
    sinks = torch.tensor([0.0, 1.5, -2.0])
    for scale in (1.0, 0.01, 30.0):
        out = ops.paged_attention_general(torch.zeros(1, H * D, device=DEV), H, D, 0, pool, table, _i32([0]), _i32([0]), 0, page, 1, scale,
                                          window=4, sinks=sinks.to(DEV), out_dim=5).cpu().view(H, 5)
        for h in range(H):
            assert torch.allclose(out[h], key[:5] / (1.0 + math.exp(float(sinks[h]))), rtol=1e-6)
    # a sink far above the scores leaves nothing; one far below changes nothing
    out = ops.paged_attention_general(torch.zeros(1, H * D, device=DEV), H, D, 0, pool, table, _i32([0]), _i32([0]), 0, page, 1, 1.0,
                                      sinks=torch.tensor([80.0, -80.0, -1e4]).to(DEV), out_dim=D).cpu().view(H, D)
    assert float(out[0].abs().max()) < 1e-30 and torch.equal(out[1], key) and torch.equal(out[2], key)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,page", [(None, 16), (700, 64), (300, 16)])
def test_a_far_key_among_hundreds(dtype, window, page):
    """640 cached rows of small numbers and one, at position 5 or at the window's far edge, that the last queries point
    at: it takes most of the softmax when it is seen (and when the window ends one position after it, nothing of it is
    left).  The last rows come as a portion and as single rows."""
    from fellm_b200 import ops
    H, D, od, T = 2, 24, 16, 640
    g = torch.Generator().manual_seed(page)
    rows = (torch.randn(T, D, generator=g) * 0.1).to(dtype)
    far = 5 if window is None or window > T else T - window            # the oldest position the LAST query sees
    rows[far] = torch.randn(D, generator=g).to(dtype) * 2.0
    q = (torch.randn(T, H, D, generator=g) * 0.1).to(dtype)
    q[T - 4:] = rows[far].float().view(1, 1, D).to(dtype) * 1.5
    n_pages = T // page
    perm = torch.randperm(n_pages, generator=g)
    pool = torch.zeros(n_pages, 1, page * D, dtype=dtype, device=DEV)
    pool[perm.to(DEV), 0] = rows.view(n_pages, page * D).to(DEV)
    table = perm.to(torch.int32).view(1, n_pages).to(DEV)
    sinks = torch.tensor([0.3, -0.4])
    # the plain attention over all rows is slow in Python: only the last eight queries are compared
    def plain_row(i):
        lo = 0 if window is None else max(0, i - window + 1)
        out = []
        for h in range(H):
            s = rows.double()[lo:i + 1] @ q.double()[i, h]
            mx = torch.maximum(s.max(), sinks.double()[h])
            e = torch.exp(s - mx)
            out.append((e @ rows.double()[lo:i + 1, :od]) / (e.sum() + torch.exp(sinks.double()[h] - mx)))
        return torch.stack(out)
    want = torch.stack([plain_row(i) for i in range(T - 8, T)])
    seen = torch.stack([plain_row(T - 1)[0], rows.double()[far, :od]])
    assert float((seen[0] - seen[1]).abs().max()) < 0.5 * float(seen[1].abs().max())          # the far key carries the last row
    flat = q.view(T, H * D).to(DEV)
    got = [ops.paged_attention_general(flat[T - 8:T - 3], H, D, 0, pool, table, _i32(list(range(T - 8, T - 3))), _i32([0] * 5), 0, page, 1,
                                       1.0, window=window, warps=3, sinks=sinks.to(DEV), out_dim=od)]
    for i in range(T - 3, T):
        got.append(ops.paged_attention_general(flat[i:i + 1], H, D, 0, pool, table, _i32([i]), _i32([0]), 0, page, 1, 1.0, window=window,
                                               warps=3, sinks=sinks.to(DEV), out_dim=od))
    got = torch.cat(got).double().cpu().view(8, H, od)
    assert (got - want).abs().max() < (1e-5 if dtype == torch.float32 else 2e-2) * float(want.abs().max())
    if window is not None and window < T:
        # one position on, the key has left the window: what is left of the softmax is small numbers
        assert float(plain_row(T - 1).abs().max()) > 5 * float(torch.stack([plain_row(i) for i in range(T - 8, T - 4)]).abs().max())


@pytest.mark.parametrize("E,top,groups", [(6, 2, (3, 2)), (12, 3, (2, 1)), (4, 2, (4, 2)), (8, 3, None), (6, 3, (2, 2)), (2, 2, (1, 1)),
                                          (9, 2, (3, 1)), (16, 8, (4, 3))])
def test_router_choice_in_groups(E, top, groups):
    """Sigmoid scores, the correction in the choice and not in the weights, groups ranked by their two best choice
    scores, experts outside the kept groups never chosen although every choice score is negative."""
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(E * 10 + top)
    T, d = 300, 32
    h = torch.randn(T, d, generator=g)
    wr = torch.randn(E, d, generator=g) * 0.5
    router = dict(experts=E, top=top)
    if groups:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    for shift in (0.0, -3.0):
        corr = torch.randn(E, generator=g) * 0.3 + shift
        z = h.double() @ wr.double().T
        want_idx, want_w = P.route(z, corr.double(), router)
        idx, w = ops.moe_router(h.to(DEV), wr.to(DEV), top, True, score="sigmoid", correction=corr.to(DEV),
                                groups=None if groups is None else (groups[0], groups[1], 2))
        a, b = torch.sort(idx.cpu().long(), 1), torch.sort(want_idx, 1)
        same = (a.values == b.values).all(1)
        assert float(same.float().mean()) > 0.98                                  # (a close call may go the other way)
        ga = torch.gather(w.cpu().double(), 1, a.indices)
        gb = torch.gather(want_w, 1, b.indices)
        assert (ga - gb)[same].abs().max() < 1e-5
        assert (w.sum(1) - 1).abs().max() < 1e-5
        if groups:
            per = E // groups[0]
            assert int((torch.div(idx.cpu().long(), per, rounding_mode="floor")[:, :, None] ==
                        torch.div(idx.cpu().long(), per, rounding_mode="floor")[:, None, :]).sum(-1).min()) >= 1
            n_groups_used = torch.tensor([len(set((row // per).tolist())) for row in idx.cpu().long()])
            assert int(n_groups_used.max()) <= groups[1]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,d,ff,E,top,groups,limit", [(1, 64, 24, 4, 2, (2, 1), 0.3), (3, 96, 40, 6, 2, (3, 2), 0.2), (70, 72, 9, 7, 3, None, 0.15),
                                                       (700, 128, 56, 6, 3, (2, 2), 5.0), (1300, 64, 32, 8, 2, (4, 2), 0.5), (300, 64, 24, 1, 1, (1, 1), 1.0)])
def test_clamped_experts_from_the_router_to_the_weighted_sum(dtype, T, d, ff, E, top, groups, limit):
    """Routing, the plan, both grouped products with the clamped activation and the combine against the plain mixture.
    The experts' inputs are large, so that most gate and up values reach their clamps (a gate clamped from below too, or
    an up branch without its + 1, would be far off); expert e's down projection is scaled by 2^e."""
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(T + E)
    W = {"router": (torch.randn(E, d, generator=g) * 0.5).to(dtype).double(), "correction": torch.randn(E, generator=g).double() * 0.2}
    for e in range(E):
        W[f"e{e}.gate"] = (torch.randn(ff, d, generator=g) * 0.2).to(dtype).double()
        W[f"e{e}.up"] = (torch.randn(ff, d, generator=g) * 0.2).to(dtype).double()
        W[f"e{e}.down"] = (torch.randn(d, ff, generator=g) * 0.1 * 2.0 ** e).to(dtype).double()
    h = torch.randn(T, d, generator=g).to(dtype)
    router = dict(experts=E, top=top)
    if groups:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    mlp = dict(expert=dict(ff=ff, limit=limit), router=router)
    gv = h.double() @ W["e0.gate"].T
    assert limit > 1 or float((gv.abs() > limit).float().mean()) > 0.05
    idx, score = ops.moe_router(h.to(DEV), W["router"].to(dtype).to(DEV), top, True, score="sigmoid", correction=W["correction"].float().to(DEV),
                                groups=None if groups is None else (groups[0], groups[1], 2))
    # the plain mixture with the kernel's own choice (a close call of the router is not this test's matter)
    s = torch.sigmoid(h.double() @ W["router"].T)
    chosen = idx.cpu().long()
    wt = torch.gather(s, 1, chosen)
    wt = wt / (wt.sum(-1, keepdim=True) + 1e-20)
    assert (score.cpu().double() - wt).abs().max() < 1e-5
    want = torch.zeros(T, d, dtype=torch.float64)
    for e in range(E):
        y = P.clamped_glu_expert(h.double(), W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"], limit)
        want += y * (wt * (chosen == e)).sum(-1, keepdim=True)
    if T <= 70:
        ci, _ = P.route(h.double() @ W["router"].T, W["correction"], router)
        if torch.equal(torch.sort(ci, 1).values, torch.sort(chosen, 1).values):
            assert torch.allclose(P.routed_experts(h.double(), W, "", mlp), want, atol=1e-9)
    gate_up = [(W[f"e{e}.gate"].to(dtype).to(DEV), W[f"e{e}.up"].to(dtype).to(DEV)) for e in range(E)]
    dn = torch.stack([W[f"e{e}.down"] for e in range(E)]).to(dtype).to(DEV)
    modes = [("fma", 64, False)]
    if dtype == torch.bfloat16:
        modes.append(("mma", 64, False))
        if ff % 8 == 0:
            modes += [("mma", 64, True), ("umma", 128, True)]
    x = torch.randn(T, d, generator=g)
    for mode, row_tile, inter in modes:
        plan = ops.moe_plan(idx, E, row_tile)
        if inter:
            gu = torch.stack([ops.interleave_gate_up(a, b) for a, b in gate_up]).contiguous()
        else:
            gu = torch.stack([torch.cat([a, b]) for a, b in gate_up]).contiguous()
        ops.MOE_MMA = mode != "fma"
        try:
            a = ops.moe_gemm(h.to(DEV), gu, plan, gated=True, gather=True, interleaved=inter, act=(limit, 1.702))
            y = ops.moe_gemm(a, dn, plan, gated=False, gather=False)
        finally:
            ops.MOE_MMA = True
        out = x.to(DEV).clone()
        ops.moe_combine(out, y, plan, score)
        ops.check_umma_status(DEV)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        err = (out.double().cpu() - x.double() - want).abs().max()
        assert err < tol * max(1.0, float(want.abs().max())), (mode, inter, float(err))


# ----------------------------------------------------------------------------- whole models

@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def engines(request):
    made = {}

    def get(name, **opts):
        key = (name, tuple(sorted(opts.items())))
        if key not in made:
            made[key] = U.make_engine(name, request.param, **opts)
        return made[key]
    get.dtype = request.param
    yield get
    made.clear()


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "M"])
def test_whole_prompt(engines, name):
    T = 150
    got = U.run_cuts(engines(name), "a", U.tokens(name, T, 0), [T])
    U.assert_close(got, U.plain_logits(name, T, 0), engines.dtype)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_layers_one_by_one(engines, name):
    """The residual stream after every layer run (the token's side input included) against the plain implementation's."""
    from fellm_b200.models import model as M
    cfg, w = U.plain_model(name)
    toks = U.tokens(name, 40, 1)
    want = []
    P.forward(toks, w, cfg, want)
    want = torch.stack(want)
    kept, orig = [], M.Block.forward

    def fwd(self, x, *a, **k):
        r = orig(self, x, *a, **k)
        kept.append(x.clone())
        return r
    M.Block.forward = fwd
    try:
        U.run_cuts(engines(name), "a", toks, [40])
    finally:
        M.Block.forward = orig
    got = torch.stack(kept).double().cpu()
    assert got.shape == want.shape
    tol = 1e-4 if engines.dtype == "float32" else 6e-2
    for i in range(got.shape[0]):
        err = (got[i] - want[i]).abs().amax(-1) / want[i].abs().max()
        # (in bfloat16 a router's close call may move a row: see meresun_util.assert_close)
        assert float(err.max() if engines.dtype == "float32" else torch.quantile(err, 0.9)) < tol, (i, float(err.max()))


@pytest.mark.parametrize("name", ["A", "B", "D", "M"])
def test_prompt_against_token_by_token(engines, name):
    T = 90
    eng = engines(name)
    toks = U.tokens(name, T, 2)
    whole = U.run_cuts(eng, "a", toks, [T])
    single = U.run_cuts(eng, "b", toks, [])
    U.assert_close(single, whole, engines.dtype)
    U.assert_close(single, U.plain_logits(name, T, 2), engines.dtype)


@pytest.mark.parametrize("name,cuts", [("A", [2, 2, 3, 17, 2, 21, 1, 1, 23, 2, 48]), ("B", [7, 2, 71, 2, 9, 64, 3]),
                                       ("C", [15, 2, 1, 16, 17, 2, 33]), ("D", [8, 2, 9, 1, 10, 65]), ("M", [31, 2, 30, 1, 2, 63, 2, 7]),
                                       ("M", [64, 2, 69])])
def test_portions_of_many_sizes(engines, name, cuts):
    T = 170
    eng = engines(name)
    toks = U.tokens(name, T, 3)
    got = U.run_cuts(eng, "a", toks, cuts)
    U.assert_close(got, U.plain_logits(name, T, 3), engines.dtype)


@pytest.mark.parametrize("name", ["A", "B", "M"])
def test_unequal_batch_against_each_alone_with_slots_and_pages_that_come_again(engines, name):
    """Four requests of different lengths share steps (portions beside single tokens), end at different times and
    are followed by new ones in the slots and pages they gave back; the pool holds less than all of them together."""
    from fellm_b200.engine import StepItem
    eng = engines(name, max_tokens=640 if name == "M" else 448)          # (M's pages hold 64 tokens: ten of them)
    lengths = [97, 5, 140, 33, 61, 120, 2, 75]
    plans = {i: (U.tokens(name, n, 10 + i), [3, 1, 2, 40, 1, 1, 17, 2, 64][i % 3:]) for i, n in enumerate(lengths)}
    waiting, live, got = list(plans), {}, {i: [] for i in plans}
    step = 0
    while waiting or live:
        while waiting and len(live) < 4 and eng.cache.free_pages() * eng.cache.page_tokens >= lengths[waiting[0]] + 16 * len(live):
            i = waiting.pop(0)
            eng.add_request(i)
            live[i] = [0, list(plans[i][1])]
        items = []
        for i, st in live.items():
            if (step + i) % 5 == 4:
                continue                                    # left out of this step, goes on later
            n = min(st[1].pop(0) if st[1] else 1, len(plans[i][0]) - st[0])
            items.append((i, StepItem(i, plans[i][0][st[0]:st[0] + n], list(range(n)))))
            st[0] += n
        if items:
            lg = eng.step([it for _, it in items])
            at = 0
            for i, it in items:
                got[i].append(lg[at:at + len(it.tokens)].clone())
                at += len(it.tokens)
        for i in [i for i, st in live.items() if st[0] == len(plans[i][0])]:
            eng.release(i)
            del live[i]
        eng.cache.audit()
        step += 1
    eng.check_status()
    cfg, w = U.plain_model(name)
    alone = engines(name)
    for i in plans:
        want = P.forward(plans[i][0], w, cfg)
        U.assert_close(torch.cat(got[i]), want, engines.dtype, note=i)
        if i in (1, 3):
            single = U.run_cuts(alone, f"alone{i}", plans[i][0], [len(plans[i][0])])
            U.assert_close(torch.cat(got[i]), single, engines.dtype, 0.1 if engines.dtype == "float32" else 1.0, note=i)


def test_wide_model(engines):
    """Width 1,024, latents of 256 and 192 under heads of 64 + 32 and 128 + 64, pages of 64 tokens: the sizes at which the
    products and the experts' grouped products run on their tensor-core kernels; portions, then token by token, the
    window of 100 passed in both."""
    name, T = "W", 150
    toks = U.tokens(name, T, 7)
    got = U.run_cuts(engines(name, page_tokens=64), "a", toks, [140, 2, 5])
    U.assert_close(got, U.plain_logits(name, T, 7), engines.dtype)


def test_long_decoding(engines):
    """420 tokens, most of them one by one: every window slides over decoded tokens, pages are given back on the way."""
    name, T = "A", 420
    toks = U.tokens(name, T, 5)
    got = U.run_cuts(engines(name, max_tokens=256), "a", toks, [20])
    U.assert_close(got, U.plain_logits(name, T, 5), engines.dtype)


def test_scaled_queries_and_keys_show_a_wrong_window_or_a_lost_sink(engines):
    """Queries and keys scaled so that a softmax is nearly one-hot: a key let in from outside its window or the oldest
    key inside left out would change the logits far beyond rounding; sinks raised so that they hold a good part of
    every denominator.  Also with the window at one position more and less than a page."""
    from fellm_b200.weights.safetensors_io import write_safetensors
    for n_case, window in enumerate([21, 15, 17] if engines.dtype == "float32" else [21]):
        cfg = copy.deepcopy(U.CFG_A)
        cfg["layers"][0]["mixer"]["mask"]["size"] = window
        cfg["layers"][2]["mixer"]["mask"]["size"] = window + 1
        _, w = U.plain_model("A")
        w = {n: t.clone() for n, t in w.items()}
        for n in ("l0.mix.uq", "l0.mix.uk", "l1.mix.uq", "l2.mix.uq", "l2.mix.uk"):
            w[n] = (w[n].float() * 8).bfloat16().double()
        for i in range(3):
            w[f"l{i}.mix.sink"] = (w[f"l{i}.mix.sink"].float() + 3.0).bfloat16().double()
        folder = Path(U._tmp.name) / f"sharp_{engines.dtype}_{n_case}"
        folder.mkdir(exist_ok=True)
        (folder / "config.json").write_text(json.dumps(cfg))
        write_safetensors(folder / "model.safetensors", {n: t.bfloat16() for n, t in w.items()})
        eng = U.make_engine(str(folder), engines.dtype)
        toks = U.tokens("A", 80, 6)
        got = U.run_cuts(eng, "a", toks, [3, 2, 11, 1, 1, 30])
        want = P.forward(toks, w, cfg)
        # without the sinks, or with a window one position off, the same comparison is off by parts in ten
        for broken in ("sink", "window"):
            w2, cfg2 = dict(w), copy.deepcopy(cfg)
            if broken == "sink":
                for i in range(3):
                    w2[f"l{i}.mix.sink"] = torch.full_like(w[f"l{i}.mix.sink"], -1e4)
            else:
                cfg2["layers"][0]["mixer"]["mask"]["size"] = window + 1
            # (rows that are longer than the window: the ones before it see every key either way)
            assert float(U.row_distances(P.forward(toks, w2, cfg2), want)[window + 1:].median()) > 0.02, broken
        U.assert_close(got, want, engines.dtype, 5.0 if engines.dtype == "float32" else 1.0, note=window)


@pytest.mark.parametrize("seed", range(10))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_configurations_drawn_at_random(seed, dtype):
    """Ten models of random shape, each under three regimes: the whole prompt, portions down to two tokens followed by
    single tokens, and two unequal requests sharing every step."""
    from fellm_b200.engine import StepItem
    cfg = U.random_config(seed)
    folder = U.write_folder(Path(U._tmp.name) / f"random_{seed}", cfg, 500 + seed)
    _, w = U.load_folder(folder)
    eng = U.make_engine(folder, dtype, max_tokens=512)
    rng = np.random.default_rng(seed)
    T = 75
    toks = [int(t) for t in rng.integers(0, cfg["vocab"], T)]
    other = [int(t) for t in rng.integers(0, cfg["vocab"], 41)]
    want, want_other = P.forward(toks, w, cfg), P.forward(other, w, cfg)
    times = 3.0 if dtype == "bfloat16" else 1.0                       # (several passes of a loop add up their rounding)
    U.assert_close(U.run_cuts(eng, "whole", toks, [T]), want, dtype, times, note=cfg)
    U.assert_close(U.run_cuts(eng, "cut", toks, [2, 17, 2, 3, 31]), want, dtype, times, note=cfg)
    eng.add_request("a")
    eng.add_request("b")
    got_a, got_b, at_a, at_b = [], [], 0, 0
    sizes_a, sizes_b = [5, 1, 30, 2], [1, 1, 16, 7, 2]
    while at_a < T or at_b < len(other):
        items = []
        na = min(sizes_a.pop(0) if sizes_a else 1, T - at_a)
        nb = min(sizes_b.pop(0) if sizes_b else 1, len(other) - at_b)
        if na > 0:
            items.append(StepItem("a", toks[at_a:at_a + na], list(range(na))))
        if nb > 0:
            items.append(StepItem("b", other[at_b:at_b + nb], list(range(nb))))
        lg = eng.step(items)
        if na > 0:
            got_a.append(lg[:na].clone())
        if nb > 0:
            got_b.append(lg[max(na, 0):max(na, 0) + nb].clone())
        at_a, at_b = at_a + max(na, 0), at_b + max(nb, 0)
    eng.check_status()
    U.assert_close(torch.cat(got_a), want, dtype, times, note=cfg)
    U.assert_close(torch.cat(got_b), want_other, dtype, times, note=cfg)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_scheduler(name):
    """Engine.generate_batch (scheduler, sampler, CUDA graphs on) in float32 against the plain implementation's greedy
    continuation; prompts longer than a portion so that the scheduler cuts them."""
    from fellm_b200.engine import GenParams
    eng = U.make_engine(name, "float32", cuda_graphs=True, n_ubatch=32, n_batch=64, max_tokens=1024)
    cfg, w = U.plain_model(name)
    prompts = [U.tokens(name, n, 20 + i) for i, n in enumerate([70, 3, 41])]
    outs, stats = eng.generate_batch(prompts, GenParams.greedy(12))
    for p, got in zip(prompts, outs):
        seq = list(p)
        for k in range(12):
            lg = P.forward(seq, w, cfg)[-1]
            top = torch.topk(lg, 2).values
            if int(lg.argmax()) != got[k]:
                assert float(top[0] - top[1]) < 1e-4 * float(lg.abs().max()), (k, got, int(lg.argmax()))
                break
            seq.append(got[k])
    assert all(s is not None for s in stats)


def test_command_line_runs_the_design(capsys):
    from fellm_b200 import cli
    folder = U.model_folder("A")
    assert cli.main(["inspect", "--model", folder]) == 0
    out = capsys.readouterr().out
    assert "architecture: Meresun" in out and "l0.mlp.e3.up" in out and "l1.mix.dkv.norm" in out
    assert cli.main(["run", folder, "--prompt", "5 17 3 9 100", "--max-tokens", "6", "--temperature", "0", "--repetition-penalty", "1.0",
                     "--dtype", "float32", "--page-tokens", "16", "-c", "256", "--kv-device-budget", "4194304"]) == 0
    toks = [int(t) for t in capsys.readouterr().out.split()]
    cfg, w = U.plain_model("A")
    seq = [5, 17, 3, 9, 100]
    for t in toks:
        lg = P.forward(seq, w, cfg)[-1]
        top = torch.topk(lg, 2).values
        assert int(lg.argmax()) == t or float(top[0] - top[1]) < 1e-4 * float(lg.abs().max())
        seq.append(t)
    assert len(toks) == 6


def test_bfloat16_generation_runs_through_the_entry_point():
    from fellm_b200.engine import GenParams
    eng = U.make_engine("C", "bfloat16", cuda_graphs=True, n_ubatch=16, n_batch=64)
    out = list(eng.generate(U.tokens("C", 50, 30), GenParams.greedy(20)))
    assert len(out) == 20 and all(0 <= t < U.CFG_C["vocab"] for t in out)


def test_trace_replay_program(tmp_path):
    """bin/trace_run on a written folder: steps of portions beside single tokens, a request that ends and one that
    takes its slot; the logits it writes are the plain implementation's."""
    import subprocess
    import sys
    root = Path(__file__).resolve().parent.parent
    folder = U.model_folder("D")
    cfg, w = U.plain_model("D")
    a, b, c = U.tokens("D", 40, 40), U.tokens("D", 9, 41), U.tokens("D", 30, 42)
    steps = [dict(step=0, entries=[dict(id="a", tokens=a[:33], want=[0, 32]), dict(id="b", tokens=b[:2], want=[])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=a[33:34], want=[0]), dict(id="b", tokens=b[2:], want=[6])], end=["b"]),
             dict(step=2, entries=[dict(id="c", tokens=c, want=[29])], end=[]),
             dict(step=3, entries=[dict(id="a", tokens=a[34:], want=[5])], end=["a", "c"])]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "128"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    wa, wb, wc = P.forward(a, w, cfg), P.forward(b, w, cfg), P.forward(c, w, cfg)
    want = {0: torch.stack([wa[0], wa[32]]), 1: torch.stack([wa[33], wb[8]]), 2: wc[29:30], 3: wa[39:40]}
    for i, wt in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
        assert U.distance(got, wt) < U.LIMIT["float32"], i
