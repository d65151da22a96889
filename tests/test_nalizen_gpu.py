"""Nalizen on the GPU against the plain implementation (tests/plain_nalizen.py).

First each mechanism alone, through its kernel's Python face with inputs made so that a fault shows (rows with a large
mean under the LayerNorm, a previous row that must come from the slot and not from the batch, heads whose rotated and
unrotated parts differ by orders of magnitude, a forget gate at its bounds, a router whose bias decides); then whole
models of four small configurations and a wide one: whole prompts, layer by layer, prompts against token-by-token
decoding, portions down to two tokens, unequal batches against each request alone, pages and slots that are freed and
come again, long decoding past every window, scores sharpened until one key decides, and greedy generation through the
scheduler, the command line and the replay program."""
from __future__ import annotations

import copy
import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import nalizen_util as U
import plain_nalizen as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _i32(xs):
    return torch.tensor(xs, dtype=torch.int32, device=DEV)


def _np(t):
    return t.detach().double().cpu().numpy()


# ----------------------------------------------------------------------------- mechanisms alone

@pytest.mark.parametrize("T,d", [(1, 96), (5, 72), (40, 128), (3, 250), (2, 2048), (7, 6), (300, 1024)])
def test_layer_norm_and_its_sum_into_the_stream(T, d):
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(d)
    y = torch.randn(T, d, generator=g) * 3.0 + 500.0                 # a large mean: E[y^2] - mean^2 would lose the variance
    w, b, x = torch.randn(d, generator=g), torch.randn(d, generator=g), torch.randn(T, d, generator=g)
    want = P.layer_norm(_np(y), _np(w), _np(b), 1e-5)
    got = ops.layernorm(y.to(DEV), w.to(DEV), b.to(DEV), 1e-5, torch.float32)
    assert np.abs(_np(got) - want).max() < 2e-3 * np.abs(want).max()       # (float32 holds 500 +- 3 to seven digits)
    y2 = torch.randn(T, d, generator=g) * 3.0 + 1.0
    want = P.layer_norm(_np(y2), _np(w), _np(b), 1e-5)
    rows = [T - 1, 0]
    got = ops.layernorm(y2.to(DEV), w.to(DEV), b.to(DEV), 1e-5, torch.bfloat16, rows=_i32(rows))
    assert np.abs(_np(got) - want[rows]).max() < 1e-2 * np.abs(want).max()
    xs, cast = x.to(DEV).clone(), torch.empty(T, d, dtype=torch.bfloat16, device=DEV)
    ops.add_layernorm(xs, y2.to(DEV), w.to(DEV), b.to(DEV), 1e-5, cast=cast)
    assert np.abs(_np(xs) - (_np(x) + want)).max() < 1e-5 * np.abs(want).max()
    assert torch.equal(cast, xs.bfloat16())


@pytest.mark.parametrize("d,with_items", [(40, False), (40, True), (128, True), (42, True)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_token_shift_reads_the_row_before_from_the_batch_or_from_the_slot(out_dtype, d, with_items):
    """with_items: the rows' items are handed over, which lets widths of a multiple of 4 take 16-byte loads."""
    from fellm_b200 import ops
    slots = 4
    g = torch.Generator().manual_seed(1)
    mu = torch.rand(d, generator=g)
    mu[0], mu[1] = 0.0, 1.0
    state = torch.zeros(slots, 3, d, device=DEV)[:, 1]                 # a view with a slot stride of its own
    seqs = {2: torch.randn(70, d, generator=g) * 5, 0: torch.randn(9, d, generator=g) * 5}
    at = {2: 0, 0: 0}
    got = {2: [], 0: []}
    for step, sizes in enumerate([(3, 1), (1, 2), (64, 1), (2, 5)]):
        rows, starts, sl = [], [0], []
        for s, n in zip((2, 0), sizes):
            rows.append(seqs[s][at[s]:at[s] + n])
            starts.append(starts[-1] + n)
            sl.append(s)
        x = torch.cat(rows).to(DEV)
        row_item = _i32([k for k in range(2) for _ in range(sizes[k])]) if with_items else None
        out = ops.token_shift(x, mu.to(DEV), state, _i32(starts), _i32(sl), 2, max(sizes), out_dtype, row_item=row_item)
        for k, (s, n) in enumerate(zip((2, 0), sizes)):
            got[s].append(out[starts[k]:starts[k + 1]].float().cpu())
            at[s] += n
    for s in (2, 0):
        n = at[s]
        prev = torch.cat([torch.zeros(1, d), seqs[s][:n - 1]])
        want = P.token_shift(_np(seqs[s][:n]), _np(prev), _np(mu))
        tol = 1e-6 if out_dtype == torch.float32 else 1e-2
        assert np.abs(_np(torch.cat(got[s])) - want).max() < tol * np.abs(want).max()
        assert torch.equal(state[s].cpu(), seqs[s][n - 1])           # the slot keeps the unshifted float32 row
    assert float(state[1].abs().max()) == 0.0 and float(state[3].abs().max()) == 0.0


@pytest.mark.parametrize("n,base,scaling", [(8, 100.0, (4.0, 1.0, 4.0, 64)), (32, 250000.0, (8.0, 1.0, 4.0, 8192)), (6, 10.0, (2.0, 0.5, 2.0, 16)),
                                            (64, 10000.0, (32.0, 1.0, 32.0, 2048)), (12, 5e5, None)])
def test_rescaled_frequencies_of_the_position_part(n, base, scaling):
    from fellm_b200.parts.base import build_part
    from fellm_b200.parts.spec import PartSpec
    part = build_part("position", PartSpec.make("rope", rot_dim=n, theta=base, pairing="split_half", table64=True, bands=scaling), "float32")
    sc = None if scaling is None else dict(zip(("factor", "low", "high", "original"), scaling))
    want = P.rotary_frequencies(n, base, sc)
    assert np.allclose(_np(part.inv_freq), want, rtol=1e-6, atol=0)
    if scaling is not None:
        assert not np.allclose(want, P.rotary_frequencies(n, base))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,rot,extra", [(6, 2, 24, 8, 16), (3, 3, 10, 6, 7), (4, 1, 128, 64, 0), (2, 2, 16, 16, 5), (5, 0, 48, 0, 3), (1, 1, 200, 120, 8),
                                              (4, 1, 128, 64, 5), (6, 2, 64, 32, 2), (3, 1, 32, 16, 5), (2, 1, 256, 0, 5), (5, 3, 64, 64, 7)])
def test_rotation_then_unit_norm_in_place(dtype, H, G, hd, rot, extra):
    """Heads whose rotated part is a thousand times their unrotated part (and the other way round): a norm over the wrong
    elements, or taken in front of a rotation that did not keep the length, would show; positions up to 100,000 (the angle
    is the float32 product of position and frequency, as the design computes it)."""
    from fellm_b200 import ops
    T = 9
    g = torch.Generator().manual_seed(hd)
    cols = (H + G) * hd + G * 3 + extra
    x = torch.randn(T, cols, generator=g)
    mag = torch.ones(hd)
    mag[:rot] = 1000.0 if hd % 3 else 0.001
    for h in range(H + G):
        x[:, h * hd:(h + 1) * hd] *= mag
    x = x.to(dtype)
    pos = [0, 1, 7, 100000, 33, 4095, 2, 511, 64][:T]
    freqs = P.rotary_frequencies(rot, 10000.0, dict(factor=4.0, low=1.0, high=4.0, original=64)) if rot else np.zeros(0)
    inv = torch.tensor(freqs, dtype=torch.float64).float().to(DEV) if rot else None
    y = x.to(DEV).clone()
    ops.qk_rotate_norm(y, H, G, H * hd, hd, rot, inv, "split_half", _i32(pos), 1e-5, unit_norm=True)
    xs = _np(x)
    for t in range(T):
        heads = xs[t, :(H + G) * hd].reshape(H + G, hd)
        want = P.unit_rms(P.rotate(heads, pos[t], _np(inv) if rot else np.zeros(0)), 1e-5)
        got = _np(y[t, :(H + G) * hd]).reshape(H + G, hd)
        tol = 2e-5 if dtype == torch.float32 else 1e-2
        assert np.abs(got - want).max() < tol * np.abs(want).max(), (t, pos[t])
    assert torch.equal(y[:, (H + G) * hd:], x.to(DEV)[:, (H + G) * hd:])           # values and what lies behind them are not touched


@pytest.mark.parametrize("block,prepared", [(0, False), (0, True), (16, True), (64, False), (0, None)])
@pytest.mark.parametrize("H,dk,dv", [(3, 20, 12), (1, 64, 8), (9, 3, 5), (2, 128, 64), (4, 48, 32), (2, 5, 33)])
def test_gated_write_recurrence_over_portions_and_slots(H, dk, dv, block, prepared):
    """The scan in portions of 1, 2, 17, ... tokens of two requests in interleaved slots against the token-by-token
    recurrence; the gate's logits reach both bounds (f = lower and f = 1) and a state written at the first token is read
    three hundred tokens later through gates close to one.  block > 0: portions longer than a block run in blocks side by
    side (beside a request's single token in the same step), which must give the same outputs and leave the same state.
    prepared: the gates are computed by a kernel in front, in place (None: the choice by the step's longest portion)."""
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(dk * dv)
    n, m = H * dk, H * dv
    pad = 5
    lower = torch.rand(n, generator=g) * 0.9
    lower[0] = 0.0
    bias = torch.randn(n, generator=g)
    state = torch.zeros(4, H, dk, dv, device=DEV)
    seqs = {}
    for s, T in ((3, 330), (1, 40)):
        z = torch.randn(T, 2 * n + m + pad, generator=g)
        z[:, n:2 * n] *= 6.0                                     # gates at both bounds
        z[1:300, n:2 * n] = 12.0                                 # ... then a long stretch that forgets almost nothing
        seqs[s] = z
    at, got = {3: 0, 1: 0}, {3: [], 1: []}
    sizes = [(1, 1), (2, 2), (17, 1), (64, 5), (1, 1), (200, 20), (45, 10)]
    for a, b in sizes:
        rows, starts, sl = [], [0], []
        for s, k in ((3, a), (1, b)):
            k = min(k, len(seqs[s]) - at[s])
            if k:
                rows.append(seqs[s][at[s]:at[s] + k])
                starts.append(starts[-1] + k)
                sl.append(s)
        z = torch.cat(rows).to(DEV)             # (a copy: the prepared form writes into it)
        o = ops.gated_write_scan(z, n, 2 * n, lower.to(DEV), bias.to(DEV), state, _i32(starts), _i32(sl), len(sl), H, dk, dv,
                                 max_item_rows=max(starts[i + 1] - starts[i] for i in range(len(sl))), block=block,
                                 prepared=prepared)
        for i, s in enumerate(sl):
            got[s].append(o[starts[i]:starts[i + 1]].cpu())
            at[s] += starts[i + 1] - starts[i]
    lo, bi = _np(lower), _np(bias)
    for s in (3, 1):
        S = np.zeros((H, dk, dv))
        z = _np(seqs[s])
        want = []
        for t in range(at[s]):
            q = P.silu(z[t, :n]).reshape(H, dk)
            f = (lo + (1 - lo) * P.sigmoid(z[t, n:2 * n] + bi)).reshape(H, dk)
            S, o = P.hgrn2_step(S, q, f, z[t, 2 * n:2 * n + m].reshape(H, dv))
            want.append(o.reshape(-1))
        want = np.stack(want)
        assert at[s] == len(seqs[s])
        assert np.abs(_np(torch.cat(got[s])) - want).max() < 2e-5 * np.abs(want).max(), s
    assert float(state[0].abs().max()) == 0.0 and float(state[2].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_elementwise_steps(dtype):
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(3)
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    gu = (torch.randn(7, 2 * 40 + 8, generator=g) * 3).to(dtype)
    want = P.gelu_tanh(_np(gu[:, :44])) * _np(gu[:, 44:88])
    got = ops.act_mul(gu.to(DEV)[:, :88], "gelu_tanh")
    assert np.abs(_np(got) - want).max() < tol * np.abs(want).max()
    want = P.silu(_np(gu[:, :44])) * _np(gu[:, 44:88])
    assert np.abs(_np(ops.act_mul(gu.to(DEV)[:, :88], "silu")) - want).max() < tol * np.abs(want).max()
    a, z = torch.randn(5, 24, generator=g).to(dtype), (torch.randn(5, 64, generator=g) * 4).to(dtype)
    want = _np(a) * P.sigmoid(_np(z[:, 8:32]))
    got = ops.gate_mul(a.to(DEV).clone(), z.to(DEV)[:, 8:32])
    assert np.abs(_np(got) - want).max() < tol * np.abs(want).max()
    r = torch.randn(6, 33, generator=g) * 2
    assert np.abs(_np(ops.relu2(r.to(DEV), dtype)) - np.maximum(_np(r), 0) ** 2).max() < tol * 16
    x = torch.randn(3, 50, generator=g)
    assert torch.equal(ops.cast_rows(x.to(DEV), dtype).cpu(), x.to(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,d,ff,E,top", [(1, 64, 24, 4, 2), (3, 96, 40, 6, 6), (70, 72, 9, 7, 3), (300, 128, 64, 16, 4), (5, 64, 16, 1, 1), (40, 1024, 512, 8, 2)])
def test_plain_experts_from_the_biased_router_to_the_weighted_sum(dtype, T, d, ff, E, top):
    """Logits a hundred times smaller than the biases: the bias decides the choice, and a weight that left it out (or a
    softmax over all the experts) would be far off; the experts' outputs differ by orders of magnitude."""
    from fellm_b200.parts.base import build_part
    from fellm_b200.parts.spec import PartSpec
    g = torch.Generator().manual_seed(T * E + top)
    part = build_part("feed_forward", PartSpec.make("moe", size=d, ff=ff, experts=E, top=top, renormalize=True, router_bias=True,
                                                     plain="relu2"), "float32" if dtype == torch.float32 else "bfloat16")
    rt = lambda *s: torch.randn(*s, generator=g).bfloat16().float()
    router, rb = rt(E, d) * 0.01, torch.linspace(-2.0, 2.0, E)[torch.randperm(E, generator=g)]
    ups = [rt(ff, d) * 0.2 * (1.0 + e) for e in range(E)]
    downs = [rt(d, ff) * 0.1 for e in range(E)]
    tensors = {"router.weight": router.to(dtype), "router.bias": rb}
    for e in range(E):
        tensors[f"e{e}.up.weight"], tensors[f"e{e}.down.weight"] = ups[e].to(dtype), downs[e].to(dtype)
    part.bind({k: v.to(DEV) for k, v in tensors.items()})
    x = rt(T, d)
    out = torch.zeros(T, d, device=DEV)
    part.forward(x.to(dtype).to(DEV), None, out)
    want = np.stack([P.routed_ff(_np(x[t]), _np(router), _np(rb), [_np(u) for u in ups], [_np(w) for w in downs], top) for t in range(T)])
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert np.abs(_np(out) - want).max() < tol * np.abs(want).max()
    if top < E:
        others = np.stack([P.routed_ff(_np(x[t]), _np(router), np.zeros(E), [_np(u) for u in ups], [_np(w) for w in downs], top) for t in range(T)])
        assert np.abs(others - want).max() > 0.1 * np.abs(want).max()            # (the bias matters in this case)


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


@pytest.mark.parametrize("name", ["A", "B", "C", "M", "O"])
def test_whole_prompt(engines, name):
    T = 150
    got = U.run_cuts(engines(name), "a", U.tokens(name, T, 0), [T])
    U.assert_close(got, U.plain_logits(name, T, 0), engines.dtype)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_layers_one_by_one(engines, name):
    """The residual stream after every layer (the token's side input included) against the plain implementation's."""
    cfg, w = U.plain_model(name)
    toks = U.tokens(name, 40, 1)
    plain = P.Plain(cfg, w)
    want = []
    for t in toks:
        s = []
        plain.step(t, s)
        want.append(np.stack(s))
    want = torch.from_numpy(np.stack(want, 1))                    # [layers, tokens, width]
    eng = engines(name)
    kept = []
    eng.model.after_run = lambda n, x: kept.append(x.clone())
    try:
        U.run_cuts(eng, "a", toks, [40])
    finally:
        eng.model.after_run = None
    got = torch.stack(kept).double().cpu()
    assert got.shape == want.shape
    tol = U.LIMIT[engines.dtype]
    for i in range(got.shape[0]):
        err = (got[i] - want[i]).abs().amax(-1) / want[i].abs().max()
        assert float(err.max() if engines.dtype == "float32" else torch.quantile(err, 0.9)) < tol, (i, float(err.max()))


@pytest.mark.parametrize("name", ["A", "B", "C", "M"])
def test_prompt_against_token_by_token(engines, name):
    T = 90
    eng = engines(name)
    toks = U.tokens(name, T, 2)
    whole = U.run_cuts(eng, "a", toks, [T])
    single = U.run_cuts(eng, "b", toks, [])
    U.assert_close(single, whole, engines.dtype)
    U.assert_close(single, U.plain_logits(name, T, 2), engines.dtype)


@pytest.mark.parametrize("name,cuts", [("A", [2, 2, 3, 17, 2, 21, 1, 1, 23, 2, 48]), ("B", [7, 2, 71, 2, 9, 64, 3]),
                                       ("C", [15, 2, 1, 16, 17, 2, 33]), ("M", [31, 2, 30, 1, 2, 63, 2, 7]), ("M", [64, 2, 69]),
                                       ("O", [2, 9, 1, 8, 2, 31, 16])])
def test_portions_of_many_sizes(engines, name, cuts):
    T = 170
    eng = engines(name)
    toks = U.tokens(name, T, 3)
    got = U.run_cuts(eng, "a", toks, cuts)
    U.assert_close(got, U.plain_logits(name, T, 3), engines.dtype)


@pytest.mark.parametrize("name", ["A", "C", "M"])
def test_unequal_batch_against_each_alone_with_slots_and_pages_that_come_again(engines, name):
    """Requests of different lengths share steps (portions beside single tokens), end at different times and are followed
    by new ones in the slots and pages they gave back; the pool holds less than all of them together.  A new request in a
    used slot starts from a zero state and a zero previous row."""
    from fellm_b200.engine import StepItem
    eng = engines(name, max_tokens=640 if name == "M" else 448)
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
        want = U.plain_run(cfg, w, plans[i][0])
        U.assert_close(torch.cat(got[i]), want, engines.dtype, note=i)
        if i in (1, 3):
            single = U.run_cuts(alone, f"alone{i}", plans[i][0], [len(plans[i][0])])
            U.assert_close(torch.cat(got[i]), single, engines.dtype, 0.1 if engines.dtype == "float32" else 1.0, note=i)


def test_wide_model(engines):
    """Width 1,024, heads of 64 and pages of 64 tokens: the sizes at which the products, the attention of portions and the
    experts' grouped products run on their tensor-core kernels; portions, then token by token, the window of 100 passed
    in both."""
    name, T = "W", 150
    toks = U.tokens(name, T, 7)
    got = U.run_cuts(engines(name), "a", toks, [140, 2, 5])
    # (float32: a plain expert's output is a sum of squares of what passes its relu, and where little passes, the LayerNorm
    # behind it divides that little by its own size: single rows at ten times the median row's distance)
    U.assert_close(got, U.plain_logits(name, T, 7), engines.dtype, 2.0 if engines.dtype == "float32" else 1.0)


def test_long_decoding(engines):
    """420 tokens, most of them one by one: every window slides over decoded tokens, pages are given back on the way, and
    the recurrent states and previous rows go through four hundred single steps."""
    name, T = "A", 420
    toks = U.tokens(name, T, 5)
    got = U.run_cuts(engines(name, max_tokens=256), "a", toks, [20])
    U.assert_close(got, U.plain_logits(name, T, 5), engines.dtype)


def test_sharp_scores_show_a_window_that_is_one_off(engines):
    """Queries and keys have unit length, so the score's scale alone decides how sharp a softmax is: raised until one key
    takes nearly all the weight, a key let in from outside its window or the oldest key inside left out moves the logits
    far beyond rounding.  Also with the windows one position under and over a page, in portions and token by token."""
    from fellm_b200.weights.safetensors_io import write_safetensors
    for n_case, window in enumerate([21, 15, 17] if engines.dtype == "float32" else [21]):
        cfg = copy.deepcopy(U.CFG_A)
        for i, wnd in ((1, window), (3, window + 12)):
            cfg["layers"][i]["mixer"]["mask"]["size"] = wnd
            cfg["layers"][i]["mixer"]["scale"] = 0.9
        _, w = U.plain_model("A")
        folder = Path(U._tmp.name) / f"sharp_{engines.dtype}_{n_case}"
        folder.mkdir(exist_ok=True)
        (folder / "config.json").write_text(json.dumps(cfg))
        write_safetensors(folder / "model.safetensors", {n: torch.from_numpy(t).bfloat16() for n, t in w.items()})
        eng = U.make_engine(str(folder), engines.dtype)
        toks = U.tokens("A", 100, 6)
        got = U.run_cuts(eng, "a", toks, [3, 2, 11, 1, 1, 30, 2, 17])
        want = U.plain_run(cfg, w, toks)
        for layer, delta in ((1, 1), (1, -1), (3, 1), (3, -1)):
            cfg2 = copy.deepcopy(cfg)
            cfg2["layers"][layer]["mixer"]["mask"]["size"] += delta
            off = U.row_distances(U.plain_run(cfg2, w, toks), want)[window + 14:]
            assert float(off.median()) > 0.01, (layer, delta, float(off.median()))
        U.assert_close(got, want, engines.dtype, 5.0 if engines.dtype == "float32" else 1.0, note=window)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,page", [(None, 16), (700, 64), (300, 16)])
def test_a_far_key_among_hundreds(dtype, window, page):
    """One attention layer with a sharp score: the token at position 3 comes again at the end, 600 positions later, and
    its query finds its own old key among hundreds (inside a window of 700 or none) or must not (a window of 300)."""
    from fellm_b200.weights.safetensors_io import write_safetensors
    cfg = U.config(64, 64, [U.layer(U.attention(2, 1, 32, 16, window, 1.5), None)], emb=4.0)
    folder = U.write_folder(Path(U._tmp.name) / f"far_{window}", cfg, 77, scales=((".mix.q", 4.0), (".mix.k", 4.0)))
    cfg, w = U.load_folder(folder)
    w["l0.mix.k"] = w["l0.mix.q"][:32].copy()                     # a token's key is its first head's query: it finds itself
    w["l0.shift"] = np.zeros_like(w["l0.shift"])
    write_safetensors(Path(folder) / "model.safetensors", {n: torch.from_numpy(t).bfloat16() for n, t in w.items()})
    rng = np.random.default_rng(5)
    toks = [int(t) for t in rng.integers(1, 64, 604)]
    toks[3] = 0
    toks = [t if (i == 3 or t != 0) else 1 for i, t in enumerate(toks)] + [0]
    want = U.plain_run(cfg, w, toks)
    eng = U.make_engine(folder, dtype, page_tokens=page, max_tokens=1024)
    got = U.run_cuts(eng, "a", toks, [590, 9, 2])                   # the last tokens one by one
    U.assert_close(got, want, dtype)
    got = U.run_cuts(eng, "b", toks, [len(toks)])
    U.assert_close(got, want, dtype)
    # the old position holds half of the last row's weight where it is visible (the other half is the row itself, the same
    # token): with its value turned round the row is another
    m = P.Plain(cfg, w)
    for t in toks[:-1]:
        m.step(t)
    m.values[0][3] = -m.values[0][3]
    moved = U.row_distances(torch.from_numpy(m.step(toks[-1]))[None], want[-1:])
    assert (float(moved) > 0.05) == (window != 300), float(moved)


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
    want, want_other = U.plain_run(cfg, w, toks), U.plain_run(cfg, w, other)
    # (bfloat16: a router that keeps one expert of several turns a close call into another row, and a recurrent state hands
    # it on to every later row)
    times = 2.0 if dtype == "bfloat16" else 1.0
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


def _follows_greedily(cfg, w, prompt, got):
    seq = list(prompt)
    for k, t in enumerate(got):
        lg = U.plain_run(cfg, w, seq)[-1]
        top = torch.topk(lg, 2).values
        if int(lg.argmax()) != t:
            assert float(top[0] - top[1]) < 1e-4 * float(lg.abs().max()), (k, got, int(lg.argmax()))
            return
        seq.append(t)


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
        assert len(got) == 12
        _follows_greedily(cfg, w, p, got)
    assert all(s is not None for s in stats)


def test_command_line_runs_the_design(capsys):
    from fellm_b200 import cli
    folder = U.model_folder("A")
    assert cli.main(["inspect", "--model", folder]) == 0
    out = capsys.readouterr().out
    assert "architecture: Nalizen" in out and "l1.mlp.e3.up" in out and "l0.mix.lower" in out
    assert cli.main(["run", folder, "--prompt", "5 17 3 9 100", "--max-tokens", "6", "--temperature", "0", "--repetition-penalty", "1.0",
                     "--dtype", "float32", "--page-tokens", "16", "-c", "256", "--kv-device-budget", "4194304"]) == 0
    toks = [int(t) for t in capsys.readouterr().out.split()]
    cfg, w = U.plain_model("A")
    assert len(toks) == 6
    _follows_greedily(cfg, w, [5, 17, 3, 9, 100], toks)


def test_bfloat16_generation_runs_through_the_entry_point():
    from fellm_b200.engine import GenParams
    eng = U.make_engine("M", "bfloat16", cuda_graphs=True, n_ubatch=16, n_batch=64)
    out = list(eng.generate(U.tokens("M", 50, 30), GenParams.greedy(20)))
    assert len(out) == 20 and all(0 <= t < U.CFG_M["vocab"] for t in out)


def test_trace_replay_program(tmp_path):
    """bin/trace_run on a written folder: steps of portions beside single tokens, a request that ends and one that takes
    its slot; the logits it writes are the plain implementation's."""
    import subprocess
    import sys
    root = Path(__file__).resolve().parent.parent
    folder = U.model_folder("C")
    cfg, w = U.plain_model("C")
    a, b, c = U.tokens("C", 40, 40), U.tokens("C", 9, 41), U.tokens("C", 30, 42)
    steps = [dict(step=0, entries=[dict(id="a", tokens=a[:33], want=[0, 32]), dict(id="b", tokens=b[:2], want=[])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=a[33:34], want=[0]), dict(id="b", tokens=b[2:], want=[6])], end=["b"]),
             dict(step=2, entries=[dict(id="c", tokens=c, want=[29])], end=[]),
             dict(step=3, entries=[dict(id="a", tokens=a[34:], want=[5])], end=["a", "c"])]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "128"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    wa, wb, wc = U.plain_run(cfg, w, a), U.plain_run(cfg, w, b), U.plain_run(cfg, w, c)
    want = {0: torch.stack([wa[0], wa[32]]), 1: torch.stack([wa[33], wb[8]]), 2: wc[29:30], 3: wa[39:40]}
    for i, wt in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
        assert U.distance(got, wt) < U.LIMIT["float32"], i
