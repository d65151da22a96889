"""Meresun without a GPU: the configuration reader, the model description made from it, the tensors it
asks for, what its layers keep between steps, and the plain implementation's own mechanisms."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import meresun_util as U
import plain_meresun as P
from fellm_b200.cache.manager import CacheManager
from fellm_b200.config.errors import ConfigError
from fellm_b200.config.registry import config_from_dict
from fellm_b200.models.model import build_model
from fellm_b200.parts.base import PagedKV


def _spec(cfg):
    arch, c = config_from_dict(cfg)
    return arch, c, arch.build_spec(c)


def test_config_round_trip_and_registry():
    for name, (cfg, _) in U.CONFIGS.items():
        arch, c, spec = _spec(cfg)
        assert arch.name == "Meresun" and c.to_dict() == cfg, name
        assert spec.vocab_size == cfg["vocab"] and spec.hidden_size == cfg["width"]
        assert all(ls.arrangement == "parallel_gated" and ls.norm2 is None and ls.gate is not None for ls in spec.layers)
    for seed in range(30):
        cfg = U.random_config(seed)
        _, c, _ = _spec(cfg)
        assert c.to_dict() == cfg, seed


@pytest.mark.parametrize("path,value,word", [
    (("width",), None, "width"), (("norm",), {}, "norm.eps"), (("norm", "groups"), 5, "norm.groups"),
    (("layers", 0, "type"), "conv", "layers[0].type"), (("layers", 1, "mixer", "heads"), 0, "heads"),
    (("layers", 1, "mixer", "mask"), {}, "mask.size"), (("layers", 1, "mixer", "kv_rank"), None, "kv_rank"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"), (("layers", 0, "mixer", "rot", "dims"), 10, "rot.dims"),
    (("layers", 0, "mixer", "rot", "scaling", "factor"), 0.0, "rot.scaling"),
    (("layers", 0, "mlp", "kind"), "routed", "mlp.kind"), (("layers", 0, "mlp", "router", "top"), 7, "router.top"),
    (("layers", 0, "mlp", "router", "top"), 5, "router.top"), (("layers", 0, "mlp", "router", "groups", "count"), 4, "router.groups"),
    (("layers", 0, "mlp", "expert"), {}, "expert.ff"), (("layers", 0, "mlp", "expert", "limit"), 0.0, "expert.limit"),
    (("loop", "stop"), 9, "loop"), (("token_side",), {}, "token_side")])
def test_config_errors_name_the_key(path, value, word):
    cfg = copy.deepcopy(U.CFG_A)
    d = cfg
    for k in path[:-1]:
        d = d[k]
    if value is None:
        del d[path[-1]]
    else:
        d[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        _spec(cfg)
    assert word in str(e.value)


def test_what_a_file_leaves_out_does_not_exist():
    cfg = copy.deepcopy(U.CFG_D)
    del cfg["loop"], cfg["token_side"], cfg["embedding"], cfg["norm"]["groups"]
    del cfg["layers"][0]["mixer"]["mask"], cfg["layers"][0]["mixer"]["rot"]
    _, c, spec = _spec(cfg)
    assert c.side_dim == 0 and c.loop is None and c.embedding_scale == 1.0 and c.norm_groups == 1
    assert c.layers[0].mixer.window is None and c.layers[0].mixer.rot_dims == 0
    assert [(r.layer, r.before) for r in spec.schedule] == [(i, None) for i in range(3)] and not spec.connectors
    assert not spec.shared and all(ls.side is None for ls in spec.layers)
    table = build_model(spec, "float32").param_table()
    assert "side.embed" not in table and "l0.side.gate" not in table and "l0.mix.sink" in table


def test_schedule_of_a_loop():
    _, _, spec = _spec(U.CFG_A)                      # layer 0, then layers 1, 2 twice: the second pass re-adds the embedding
    assert [(r.layer, r.before) for r in spec.schedule] == [(0, None), (1, None), (2, None), (1, (0, 1)), (2, None)]
    assert [i for i, _ in P.layer_order(U.CFG_A)] == [r.layer for r in spec.schedule]
    assert [re for _, re in P.layer_order(U.CFG_A)] == [r.before is not None for r in spec.schedule]
    _, _, spec = _spec(U.CFG_B)
    assert [(r.layer, r.before) for r in spec.schedule] == [(i, None) for i in range(4)] and not spec.connectors
    _, _, spec = _spec(U.CFG_C)
    assert [(r.layer, r.before) for r in spec.schedule] == [(0, None), (1, None), (0, (0, 1)), (1, None), (0, (0, 2)), (1, None)]
    _, _, spec = _spec(U.CFG_D)                      # one pass: nothing is re-added
    assert [(r.layer, r.before) for r in spec.schedule] == [(0, None), (1, None), (2, None)]


def test_tensor_names_and_shapes():
    _, _, spec = _spec(U.CFG_A)
    table = build_model(spec, "float32").param_table()
    for n in ("embed", "head", "final.norm", "side.embed", "l0.norm1", "l0.mix.dq", "l0.mix.dq.norm", "l0.mix.uq", "l0.mix.dkv",
              "l0.mix.dkv.norm", "l0.mix.uk", "l0.mix.uv", "l0.mix.sink", "l0.mix.o", "l0.mlp.router", "l0.mlp.correction",
              "l0.mlp.e0.gate", "l0.mlp.e5.down", "l0.rg1", "l0.rg1.b", "l0.rg2", "l0.rg2.b", "l0.side.gate", "l0.side.proj",
              "l0.side.norm", "l1.mlp.up", "l1.mlp.down", "l1.mlp.act", "l2.rg1", "l2.rg1.b"):
        assert n in table, n
    for n in ("l2.rg2", "l2.rg2.b", "l2.mlp.up", "l0.mlp.e6.gate", "l0.norm2", "l1.mlp.router", "l0.mlp.up"):
        assert n not in table, n
    shape = lambda n: tuple(table[n][2].shape)
    assert shape("side.embed") == (211, 3 * 5) and shape("l0.side.gate") == (5, 96) and shape("l0.side.proj") == (96, 5)
    assert shape("l0.mix.dq") == (24, 96) and shape("l0.mix.uq") == (3 * (20 + 8), 24) and shape("l0.mix.dkv") == (40 + 8, 96)
    assert shape("l0.mix.uk") == (3 * 20, 40) and shape("l0.mix.uv") == (3 * 12, 40) and shape("l0.mix.o") == (96, 3 * 12)
    assert shape("l0.mix.sink") == (3,) and shape("l0.mix.dkv.norm") == (40,) and shape("l1.mlp.act") == (4,)
    assert shape("l0.mlp.router") == (6, 96) and shape("l0.mlp.correction") == (6,) and shape("l0.mlp.e1.down") == (96, 40)


def test_one_product_for_everything_that_reads_a_layer_input():
    """After binding, the mixer's down projections, the gates and a dense up of a layer are views of ONE matrix, in
    that order, each part's columns recorded; the gates' bias lies at their rows of the joint bias, zeros elsewhere; a
    layer without a dense feed-forward joins two parts."""
    from fellm_b200.weights.loader import bind_tensors
    from fellm_b200.weights.random_init import random_tensors
    _, _, spec = _spec(U.CFG_A)
    model = build_model(spec, "float32")
    tensors = random_tensors(model, 3)
    bind_tensors(model, tensors, "cpu")
    for i, block in enumerate(model.blocks):
        w, bias, cols = block.joint
        parts = {"mixer": block.mixer, "gate": block.gate, "ffn": block.ffn}
        assert list(cols) == (["mixer", "gate", "ffn"] if i == 1 else ["mixer", "gate"])         # layer 1 is the dense one
        end = 0
        for key, (a, b) in cols.items():
            part = parts[key]
            view = part.w[part.input_rows]
            assert a == end and view.shape[0] == b - a and view.data_ptr() == w[a:b].data_ptr() and torch.equal(view, w[a:b])
            end = b
        assert end == w.shape[0] == bias.numel()
        a, b = cols["gate"]
        assert torch.equal(bias[a:b], block.gate.w["bias"]) and float(bias[:a].abs().sum()) == 0.0 and float(bias[b:].abs().sum()) == 0.0
        assert torch.equal(block.gate.w["weight"][:96].float(), tensors[f"l{i}.rg1"].float())
    assert torch.equal(model.blocks[1].ffn.w["up.weight"].float(), tensors["l1.mlp.up"].float())


def test_cache_needs_and_window_trimming():
    _, _, spec = _spec(U.CFG_A)
    needs = build_model(spec, "float32").cache_needs()
    # one key "head" per token: the latent followed by the rotated key part, read as its own value
    assert needs[0] == PagedKV(1, 40 + 8, 21, None, None, True) and needs[0].value_dim == 0
    assert needs[1] == PagedKV(1, 32 + 16, 50, None, None, True)
    assert needs[2] == PagedKV(1, 56 + 4, 21, None, None, True)
    assert needs[3] == needs[1] and needs[4] == needs[2] and len(needs) == 5          # each pass has its own
    cm = CacheManager([PagedKV(1, 48, 21, None, None, True)], page_tokens=16, max_tokens=64, max_requests=2, n_ctx=512,
                      dtype=torch.float32, device="cpu")
    assert cm.paged[0].pool.shape[-1] == 16 * 48
    cm.add_request("a")
    for _ in range(200):
        cm.reserve("a", 1)
        cm.advance("a", 1)
        cm.audit()
        first = cm.paged[0].first_page[0]
        assert first * 16 <= max(0, cm.length("a") - 21 + 1)          # nothing the next query can see was given back
        assert 4 - cm.free_pages() <= 3


def test_plain_norms_and_activations():
    torch.manual_seed(0)
    f64 = torch.float64
    x = torch.randn(3, 12, dtype=f64) * torch.tensor([1.0] * 4 + [50.0] * 4 + [0.01] * 4, dtype=f64)
    w = torch.randn(12, dtype=f64)
    g = P.grouped_rms_norm(x, w, 1e-6, 3)
    for k in range(3):                      # every part has a root mean square of its own
        part = x[:, 4 * k:4 * k + 4]
        assert torch.allclose(g[:, 4 * k:4 * k + 4], part / torch.sqrt((part ** 2).mean(-1, keepdim=True) + 1e-6) * w[4 * k:4 * k + 4])
    assert torch.allclose(P.grouped_rms_norm(x, w, 1e-6, 1), P.rms_norm(x, w, 1e-6))
    assert not torch.allclose(g, P.rms_norm(x, w, 1e-6))
    # eps is under the root: a zero vector stays zero, a tiny one is damped
    assert torch.equal(P.rms_unit(torch.zeros(1, 4, dtype=f64), 1e-6), torch.zeros(1, 4, dtype=f64))
    assert abs(float(P.rms_unit(torch.full((1, 4), 1e-3, dtype=f64), 1e-6)[0, 0]) - 1e-3 / math.sqrt(2e-6)) < 1e-12
    assert abs(float(P.gelu_tanh(torch.tensor(1.0, dtype=f64))) - 0.8411919906082768) < 1e-12
    # the polynomial activation: each power over its own root mean square, then the four numbers
    z = torch.randn(2, 9, dtype=f64)
    coef = torch.tensor([0.5, -1.5, 2.0, 0.25], dtype=f64)
    want = 0.25 + sum(c * (z ** (k + 1)) / torch.sqrt(((z ** (k + 1)) ** 2).mean(-1, keepdim=True) + 1e-5) for k, c in enumerate(coef[:3]))
    assert torch.allclose(P.poly_norm(z, coef, 1e-5), want)
    # an expert: the gate is clamped from above only, the other branch on both sides, and 1 is added to it
    wg, wu, wd = torch.eye(3, dtype=f64), torch.eye(3, dtype=f64), torch.eye(3, dtype=f64)
    h = torch.tensor([[5.0, -5.0, 0.2]], dtype=f64)
    y = P.clamped_glu_expert(h, wg, wu, wd, 1.0)[0]
    sg = lambda t: 1 / (1 + math.exp(-1.702 * t))
    assert abs(float(y[0]) - 1.0 * sg(1.0) * 2.0) < 1e-12 and abs(float(y[1]) - (-5.0) * sg(-5.0) * 0.0) < 1e-12
    assert abs(float(y[2]) - 0.2 * sg(0.2) * 1.2) < 1e-12


def test_plain_frequencies_and_rotation():
    f64 = torch.float64
    f, mag = P.scaled_frequencies(8, 100.0, None)
    assert mag == 1.0 and f == [100.0 ** (-2.0 * i / 8) for i in range(4)]
    sc = dict(factor=4.0, original=64, fast=8.0, slow=1.0)
    f2, mag2 = P.scaled_frequencies(8, 100.0, sc)
    assert abs(mag2 - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    lo = max(math.floor(8 * math.log(64 / (2 * math.pi * 8.0)) / (2 * math.log(100.0))), 0)
    hi = min(math.ceil(8 * math.log(64 / (2 * math.pi * 1.0)) / (2 * math.log(100.0))), 7)
    assert (lo, hi) == (0, 3)
    for i in range(4):
        r = min(max((i - lo) / (hi - lo), 0.0), 1.0)
        assert abs(f2[i] - (f[i] / 4.0 * r + f[i] * (1 - r))) < 1e-15
    assert f2[0] == f[0] and abs(f2[3] - f[3] / 4.0) < 1e-15
    # hi <= lo (both edges before the first pair): the width of the ramp is 0.001, so pair 0 keeps its frequency and
    # every later pair is divided
    f3, _ = P.scaled_frequencies(6, 10.0, dict(factor=2.0, original=1.0, fast=1.0, slow=1.0))
    assert f3[0] == 1.0 and abs(f3[1] - 10.0 ** (-2.0 / 6) / 2.0) < 1e-15 and abs(f3[2] - 10.0 ** (-4.0 / 6) / 2.0) < 1e-15
    # neighbours are paired; position 0 is multiplied by the magnitude alone
    x = torch.randn(3, 2, 6, dtype=f64)
    r = P.rotate_pairs(x[..., :4], [1.0, 0.5], 1.5)
    assert torch.allclose(r[0], 1.5 * x[0, :, :4])
    assert torch.allclose(r[2, 1, 0], 1.5 * (x[2, 1, 0] * math.cos(2.0) - x[2, 1, 1] * math.sin(2.0)))
    assert torch.allclose(r[2, 1, 3], 1.5 * (x[2, 1, 3] * math.cos(1.0) + x[2, 1, 2] * math.sin(1.0)))
    assert torch.allclose(P.rotate_pairs(x[..., :4], [1.0, 0.5], 1.0, first=5)[0, 0, 1], x[0, 0, 1] * math.cos(5.0) + x[0, 0, 0] * math.sin(5.0))


def test_plain_attention_sink_and_window():
    f64 = torch.float64
    torch.manual_seed(1)
    v = torch.randn(9, 2, 3, dtype=f64)
    zq = torch.zeros(9, 2, 4, dtype=f64)
    k = torch.randn(9, 2, 4, dtype=f64)
    # q = 0 and a sink of 0: every key and the sink weigh the same, so the sum of the window's values over n + 1
    o = P.sink_softmax_attention(zq, k, v, 1.0, 4, torch.zeros(2, dtype=f64))
    assert torch.allclose(o[6, 1], v[3:7, 1].sum(0) / 5) and torch.allclose(o[2, 0], v[:3, 0].sum(0) / 4)
    # a sink far below every score changes nothing, one far above takes everything
    o = P.sink_softmax_attention(zq, k, v, 1.0, None, torch.tensor([-1e3, 1e3], dtype=f64))
    assert torch.allclose(o[5, 0], v[:6, 0].mean(0)) and float(o[5, 1].abs().max()) < 1e-300
    # the sink is not scaled: doubling the scale with q = 0 changes nothing
    a = P.sink_softmax_attention(zq, k, v, 1.0, 3, torch.tensor([0.7, -0.2], dtype=f64))
    b = P.sink_softmax_attention(zq, k, v, 2.0, 3, torch.tensor([0.7, -0.2], dtype=f64))
    assert torch.equal(a, b)
    assert torch.allclose(a[4, 0], v[2:5, 0].sum(0) / (3 + math.exp(0.7)))
    # a window of one: the query's own position and the sink
    o = P.sink_softmax_attention(torch.randn(9, 2, 4, dtype=f64), k, v, 0.0, 1, torch.zeros(2, dtype=f64))
    assert torch.allclose(o, v / 2)


def test_plain_latent_attention_equals_attention_over_the_latent():
    """The mixer's result computed with the query taken into the latent's space (the form that needs no keys or
    values per head) equals the one with every head's keys and values written out."""
    torch.manual_seed(2)
    f64 = torch.float64
    m = U.CFG_A["layers"][1]["mixer"]
    H, dn, dr, dv, rq, rk, d = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"], 96
    W = {"dq": torch.randn(rq, d, dtype=f64) / 8, "dq.norm": torch.rand(rq, dtype=f64) + 0.5, "uq": torch.randn(H * (dn + dr), rq, dtype=f64) / 4,
         "dkv": torch.randn(rk + dr, d, dtype=f64) / 8, "dkv.norm": torch.rand(rk, dtype=f64) + 0.5, "uk": torch.randn(H * dn, rk, dtype=f64) / 4,
         "uv": torch.randn(H * dv, rk, dtype=f64) / 4, "sink": torch.randn(H, dtype=f64), "o": torch.randn(d, H * dv, dtype=f64) / 4}
    T = 70
    h = torch.randn(T, d, dtype=f64)
    want = P.latent_attention_mixer(h, W, "", m, 1e-5)
    cq = P.rms_norm(h @ W["dq"].T, W["dq.norm"], 1e-5)
    q = (cq @ W["uq"].T).view(T, H, dn + dr)
    kv = h @ W["dkv"].T
    c = P.rms_norm(kv[:, :rk], W["dkv.norm"], 1e-5)
    f, mag = P.scaled_frequencies(dr, m["rot"]["base"], m["rot"]["scaling"])
    qa = torch.einsum("thn,hnr->thr", q[..., :dn], W["uk"].view(H, dn, rk))
    qq = torch.cat([qa, P.rotate_pairs(q[..., dn:], f, mag)], -1)
    row = torch.cat([c, P.rotate_pairs(kv[:, None, rk:], f, mag)[:, 0]], -1)[:, None, :].expand(T, H, rk + dr)
    lat = P.sink_softmax_attention(qq, row, c[:, None, :].expand(T, H, rk), m["scale"], m["mask"]["size"], W["sink"])
    got = torch.einsum("thr,hvr->thv", lat, W["uv"].view(H, dv, rk)).reshape(T, H * dv) @ W["o"].T
    assert torch.allclose(got, want, atol=1e-10)


def test_plain_routing():
    f64 = torch.float64
    # scores .9 .1 | .6 .6 | .5 .2: with two best summed the middle group wins; the choice stays inside it
    z = torch.logit(torch.tensor([[0.9, 0.1, 0.6, 0.6, 0.5, 0.2]], dtype=f64))
    zero = torch.zeros(6, dtype=f64)
    idx, w = P.route(z, zero, dict(experts=6, top=2, groups=dict(count=3, keep=1)))
    assert sorted(idx[0].tolist()) == [2, 3] and torch.allclose(w, torch.tensor([[0.5, 0.5]], dtype=f64))
    # without groups the largest scores win; the weights are the scores over their sum
    idx, w = P.route(z, zero, dict(experts=6, top=2))
    assert idx[0, 0] == 0 and idx[0, 1] in (2, 3) and torch.allclose(w, torch.tensor([[0.6, 0.4]], dtype=f64))
    # the correction moves the choice and not the weights; choice scores may all be negative, an expert outside the
    # kept groups is never taken all the same
    corr = torch.tensor([-5.0, -5.0, -5.0, -5.0, -3.0, -3.0], dtype=f64)
    idx, w = P.route(z, corr, dict(experts=6, top=2, groups=dict(count=3, keep=1)))
    assert sorted(idx[0].tolist()) == [4, 5] and torch.allclose(w.sort().values, torch.tensor([[0.2 / 0.7, 0.5 / 0.7]], dtype=f64))
    idx, _ = P.route(z, torch.tensor([0.0, 0.0, -9.0, -9.0, -9.0, 1.0], dtype=f64), dict(experts=6, top=3, groups=dict(count=3, keep=2)))
    assert sorted(idx[0].tolist()) == [0, 1, 5]           # groups 0 and 2 are kept: .9 + .1 and 1.2 - 8.5 beat -8.4 - 8.4
    # groups of one expert: the group's score is its expert's
    idx, _ = P.route(z, zero, dict(experts=6, top=2, groups=dict(count=6, keep=2)))
    assert idx[0, 0] == 0 and idx[0, 1] in (2, 3)


def test_plain_routed_experts_and_side_input():
    torch.manual_seed(3)
    f64 = torch.float64
    d, E = 4, 4
    W = {"router": torch.randn(E, d, dtype=f64), "correction": torch.randn(E, dtype=f64)}
    for e in range(E):
        W.update({f"e{e}.gate": torch.randn(5, d, dtype=f64), f"e{e}.up": torch.randn(5, d, dtype=f64), f"e{e}.down": torch.randn(d, 5, dtype=f64)})
    h = torch.randn(6, d, dtype=f64)
    mlp = dict(expert=dict(ff=5, limit=0.7), router=dict(experts=E, top=E))
    out = P.routed_experts(h, W, "", mlp)
    s = torch.sigmoid(h @ W["router"].T)
    s = s / s.sum(-1, keepdim=True)
    want = sum(s[:, e:e + 1] * P.clamped_glu_expert(h, W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"], 0.7) for e in range(E))
    assert torch.allclose(out, want)
    # the side input: a unit vector (times the norm weight) whatever the table's magnitude; layer i reads its own part
    Wd = {"side.embed": torch.randn(10, 6, dtype=f64), "gate": torch.randn(3, d, dtype=f64), "proj": torch.randn(d, 3, dtype=f64), "norm": torch.ones(d, dtype=f64)}
    x = torch.randn(2, d, dtype=f64)
    y0 = P.token_side_input(x, [4, 7], Wd, "", 0, 3, 0.0)
    assert torch.allclose((y0 ** 2).mean(-1), torch.ones(2, dtype=f64))
    Wd2 = dict(Wd)
    Wd2["side.embed"] = Wd["side.embed"].clone()
    Wd2["side.embed"][:, 3:] *= -7.0
    assert torch.equal(P.token_side_input(x, [4, 7], Wd2, "", 0, 3, 0.0), y0)
    assert torch.allclose(P.token_side_input(x, [4, 7], Wd2, "", 1, 3, 0.0), -P.token_side_input(x, [4, 7], Wd, "", 1, 3, 0.0))


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_written_folder_is_read_back_and_runs_in_the_plain_implementation(name):
    cfg, w = U.plain_model(name)
    assert cfg == U.CONFIGS[name][0]
    lg = U.plain_logits(name, 12, 0)
    assert lg.shape == (12, cfg["vocab"]) and bool(torch.isfinite(lg).all())
    kept = []
    lg2 = P.forward(U.tokens(name, 12, 0)[:7], w, cfg, kept)
    assert torch.allclose(lg[:7], lg2, atol=1e-9)                       # a position depends on the ones before it only
    assert len(kept) == len(P.layer_order(cfg))
