"""Nalizen without a GPU: the configuration reader, the model description made from it, the tensors it asks for, what
its layers keep between steps (a reader of another layer's pages still keeps a row of its own), and the plain
implementation's own mechanisms."""
from __future__ import annotations

import copy
import math

import numpy as np
import pytest

import nalizen_util as U
import plain_nalizen as P
from fellm_b200.cache.manager import CacheManager, PagedView, StateView
from fellm_b200.config.errors import ConfigError
from fellm_b200.config.registry import config_from_dict
from fellm_b200.models.model import build_model
from fellm_b200.parts.base import FixedState, PagedKV


def _spec(cfg):
    arch, c = config_from_dict(cfg)
    return arch, c, arch.build_spec(c)


def test_config_round_trip_and_registry():
    for name, (cfg, _) in U.CONFIGS.items():
        arch, c, spec = _spec(cfg)
        assert arch.name == "Nalizen" and c.to_dict() == cfg, name
        assert spec.vocab_size == cfg["vocab"] and spec.hidden_size == cfg["width"]
        assert all(ls.arrangement == "outnorm" and ls.mixer.kind == "token_shifted" for ls in spec.layers)
        assert all((ls.ffn is None) == (ls.norm2 is None) for ls in spec.layers)
    for seed in range(40):
        cfg = U.random_config(seed)
        _, c, _ = _spec(cfg)
        assert c.to_dict() == cfg, seed


def test_what_a_file_leaves_out_does_not_exist():
    cfg = copy.deepcopy(U.CFG_B)
    del cfg["embedding"], cfg["token_side"]
    m = cfg["layers"][1]["mixer"]
    del m["kv_heads"], m["vdim"]
    _, c, spec = _spec(cfg)
    assert c.embedding_scale == 1.0 and c.side_dim == 0 and not spec.shared and all(ls.side is None for ls in spec.layers)
    assert c.layers[1].mixer.kv_heads == c.layers[1].mixer.heads and c.layers[1].mixer.vdim == c.layers[1].mixer.dim
    assert c.layers[1].mixer.rot_dims == 0 and c.layers[0].mixer.window is None and c.layers[0].mixer.scaling is None


@pytest.mark.parametrize("path,value,word", [
    (("width",), None, "width"), (("norm",), {}, "norm.eps"), (("vocab",), 0, "vocab"),
    (("layers", 0, "type"), "conv", "layers[0].type"), (("layers", 1, "mixer", "heads"), 0, "heads"),
    (("layers", 1, "mixer", "heads"), 5, "kv_heads"), (("layers", 1, "mixer", "mask"), {}, "mask.size"),
    (("layers", 1, "mixer", "scale"), None, "scale"), (("layers", 0, "mixer", "vdim"), None, "vdim"),
    (("layers", 1, "mixer", "rot", "dims"), 7, "rot.dims"), (("layers", 1, "mixer", "rot", "dims"), 26, "rot.dims"),
    (("layers", 1, "mixer", "rot", "scaling", "factor"), 0.0, "rot.scaling"),
    (("layers", 1, "mixer", "rot", "scaling", "low"), None, "low"),
    (("layers", 3, "mixer", "kv_from"), 3, "kv_from"), (("layers", 3, "mixer", "kv_from"), 0, "kv_from"),
    (("layers", 3, "mixer", "kv_from"), 4, "kv_from"), (("layers", 3, "mixer", "dim"), 32, "kv_from"),
    (("layers", 3, "mixer", "rot", "base"), 500.0, "kv_from"),
    (("layers", 0, "mlp", "kind"), "routed", "mlp.kind"), (("layers", 1, "mlp", "router", "top"), 7, "router.top"),
    (("layers", 1, "mlp", "expert"), {}, "expert.ff"), (("token_side",), {}, "token_side")])
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


def test_a_reader_of_a_reader_is_refused():
    cfg = copy.deepcopy(U.CFG_C)
    cfg["layers"][4]["mixer"]["kv_from"] = 2
    with pytest.raises(ConfigError) as e:
        _spec(cfg)
    assert "kv_from" in str(e.value)


def test_tensor_names_and_shapes():
    _, c, spec = _spec(U.CFG_A)
    table = build_model(spec, "bfloat16").param_table()
    shape = {n: d.shape for n, (_, _, d) in table.items()}
    assert shape["embed"] == (211, 96) and shape["side.embed"] == (211, 25) and "head" not in shape
    assert shape["final.norm"] == (96,) and shape["final.norm.b"] == (96,)
    assert shape["l0.mix.q"] == (60, 96) and shape["l0.mix.f"] == (60, 96) and shape["l0.mix.f.b"] == (60,)
    assert shape["l0.mix.lower"] == (60,) and shape["l0.mix.v"] == (36, 96) and shape["l0.mix.norm"] == (12,)
    assert shape["l0.mix.o"] == (96, 36) and shape["l0.shift"] == (96,)
    assert shape["l1.mix.q"] == (144, 96) and shape["l1.mix.k"] == (48, 96) and shape["l1.mix.v"] == (32, 96)
    assert shape["l1.mix.g"] == (96, 96) and shape["l1.mix.o"] == (96, 96)
    assert "l3.mix.k" not in shape and "l3.mix.v" not in shape and shape["l3.mix.q"] == (144, 96)      # reads layer 1's
    assert "l3.norm2" not in shape and "l3.mlp.up" not in shape                                        # no feed-forward
    assert shape["l0.mlp.gate"] == (160, 96) and shape["l0.mlp.down"] == (96, 160)
    assert shape["l1.mlp.router"] == (6, 96) and shape["l1.mlp.router.b"] == (6,)
    assert shape["l1.mlp.e5.up"] == (40, 96) and shape["l1.mlp.e5.down"] == (96, 40) and "l1.mlp.e0.gate" not in shape
    assert shape["l4.side.gate"] == (5, 96) and shape["l4.side.proj"] == (96, 5) and shape["l4.side.norm"] == (96,)


def test_what_the_layers_keep_and_whose_pages_they_read():
    _, c, spec = _spec(U.CFG_A)
    assert [r.cache_of for r in spec.schedule] == [None, None, None, 1, None]
    needs = build_model(spec, "float32").cache_needs()
    row = FixedState((96,))
    assert needs[0] == [row, FixedState((3, 20, 12))]
    # pages are kept for the WIDEST window among the layer and its readers
    assert needs[1] == [row, PagedKV(2, 24, 50, None, 16, False)]
    assert needs[3] == [row]                       # the reader keeps the previous token's row, nothing else
    # a reader with a narrower window leaves the owner's pages alone; no window anywhere: nothing is given back
    _, _, spec_b = _spec(U.CFG_B)
    needs_b = build_model(spec_b, "float32").cache_needs()
    assert needs_b[0][1].window is None and needs_b[1][1] == PagedKV(1, 8, 1, None, 40, False) and needs_b[3] == [FixedState((128,))]
    cache = CacheManager(needs, page_tokens=16, max_tokens=256, max_requests=3, n_ctx=256, dtype=None, device="cpu")
    views = cache.views(None)
    assert isinstance(views[3], list) and len(views[3]) == 1 and isinstance(views[3][0], StateView)
    assert isinstance(views[1][1], PagedView) and views[1][1].window == 50
    # five rows of the previous token are five layers of one state group
    assert sum(1 for g in cache.fixed if g.need == row) == 1 and [len(g.entries) for g in cache.fixed if g.need == row] == [5]
    # the window of 50 gives pages back only when no query of either layer can reach them
    cache.add_request("a")
    cache.reserve("a", 200)
    cache.advance("a", 200)
    assert len(cache.paged[0].held_pages(cache.slot("a"))) == math.ceil(200 / 16) - (200 - 50 + 1) // 16
    cache.audit()


# ----------------------------------------------------------------------------- the plain implementation's own mechanisms

def test_layer_norm_takes_the_variance_of_the_deviations():
    y = np.array([[1000.0, 1001.0, 1002.0, 1003.0]])
    got = P.layer_norm(y, np.full(4, 2.0), np.full(4, 0.5), 0.0)
    assert np.allclose(got, np.array([-1.5, -0.5, 0.5, 1.5]) / math.sqrt(1.25) * 2 + 0.5)


def test_token_shift_starts_from_zeros_and_hands_on_the_unshifted_row():
    s = np.array([0.0, 0.25, 1.0])
    x0, x1 = np.array([4.0, 4.0, 4.0]), np.array([8.0, 8.0, 8.0])
    assert np.allclose(P.token_shift(x0, np.zeros(3), s), [4.0, 3.0, 0.0])
    assert np.allclose(P.token_shift(x1, x0, s), [8.0, 7.0, 4.0])


def test_frequencies_keep_short_waves_and_stretch_long_ones():
    plain = P.rotary_frequencies(16, 10000.0)
    assert np.allclose(plain, [10000.0 ** (-i / 8) for i in range(8)])
    sc = dict(factor=4.0, low=1.0, high=4.0, original=64)
    got = P.rotary_frequencies(16, 10000.0, sc)
    wave = 2 * math.pi / plain
    assert np.allclose(got[wave < 16], plain[wave < 16]) and np.allclose(got[wave > 64], plain[wave > 64] / 4)
    mid = (wave >= 16) & (wave <= 64)
    assert mid.any() and np.all(got[mid] < plain[mid]) and np.all(got[mid] > plain[mid] / 4)
    s = (64 / wave[mid] - 1.0) / 3.0
    assert np.allclose(got[mid], (1 - s) * plain[mid] / 4 + s * plain[mid])


def test_rotation_pairs_the_halves_and_leaves_the_rest():
    x = np.arange(1.0, 9.0)[None, :]
    f = np.array([0.5, 0.25])
    got = P.rotate(x, 3, f)
    for i in range(2):
        c, s = math.cos(3 * f[i]), math.sin(3 * f[i])
        assert np.isclose(got[0, i], x[0, i] * c - x[0, i + 2] * s) and np.isclose(got[0, i + 2], x[0, i + 2] * c + x[0, i] * s)
    assert np.allclose(got[0, 4:], x[0, 4:]) and np.isclose((got ** 2).sum(), (x ** 2).sum())


def test_window_counts_the_query_itself():
    keys = [np.eye(4)[None, j % 4] * 5.0 for j in range(10)]
    vals = [np.full((1, 2), float(j)) for j in range(10)]
    q = np.ones((1, 4))
    out = P.attend(q, keys, vals, 9, 3, 1.0, 1)                 # positions 7, 8, 9: equal scores
    assert np.allclose(out, 8.0)
    assert np.allclose(P.attend(q, keys, vals, 9, 1, 1.0, 1), 9.0) and np.allclose(P.attend(q, keys, vals, 9, None, 1.0, 1), 4.5)


def test_hgrn2_gate_weighs_the_old_and_the_new():
    S = np.zeros((1, 2, 2))
    q, f, v = np.array([[1.0, 2.0]]), np.array([[0.25, 1.0]]), np.array([[4.0, 8.0]])
    S, o = P.hgrn2_step(S, q, f, v)
    assert np.allclose(S[0], [[3.0, 6.0], [0.0, 0.0]]) and np.allclose(o, [[3.0, 6.0]])        # a gate of 1 writes nothing
    S, o = P.hgrn2_step(S, q, np.array([[0.5, 0.0]]), np.array([[2.0, 2.0]]))
    assert np.allclose(S[0], [[2.5, 4.0], [2.0, 2.0]]) and np.allclose(o, [[6.5, 8.0]])


def test_router_softmax_runs_over_the_chosen_logits_alone():
    x = np.array([1.0, 0.0])
    router, b = np.array([[1.0, 0.0], [3.0, 0.0], [2.0, 0.0], [2.0, 0.0]]), np.array([0.0, 0.0, 0.5, 0.0])
    ups = [np.array([[float(e + 1), 0.0]]) for e in range(4)]
    downs = [np.array([[1.0], [-1.0]]) for _ in range(4)]
    got = P.routed_ff(x, router, b, ups, downs, 2)            # experts 1 (logit 3) and 2 (2.5, by its bias)
    w1 = math.exp(3.0) / (math.exp(3.0) + math.exp(2.5))
    want = w1 * 2.0 ** 2 + (1 - w1) * 3.0 ** 2
    assert np.allclose(got, [want, -want])
    assert np.allclose(P.routed_ff(-x, router, b, ups, downs, 4), 0.0)            # relu: nothing passes


def test_plain_model_does_not_depend_on_later_tokens():
    cfg, w = U.plain_model("C")
    toks = U.tokens("C", 30, 1)
    a, b = U.plain_run(cfg, w, toks), U.plain_run(cfg, w, toks[:19])
    assert float((a[:19] - b).abs().max()) == 0.0
