"""HGRN2: linear attention whose forget gate also decides what is written.  Per head, with dk key channels and dv
value channels,

    q = SiLU(W_q h)                                   [dk]
    f = l + (1 - l) sigmoid(W_f h + b_f)              [dk], l a lower bound per channel (a tensor of the layer)
    v = W_v h                                         [dv]
    S <- diag(f) S + (1 - f) v^T;   o = S^T q         (S [dk, dv], zero when a request starts; there is no key)
    o over its root mean square over dv, times a weight [dv] shared by the heads; heads side by side; W_o.

The three input projections are one product with float32 sums and a float32 result; the gate, its sigmoid, the
state and every sum of the recurrence are float32 in both engine dtypes (ops.gated_write_scan: the scan kernel the
other recurrent mixers use, in the form B = f q, G = f, K = 1 - f, c = sum (1 - f) q).  Kept per request: S, float32."""
from __future__ import annotations

import torch

from .. import ops
from ..config.errors import ConfigError
from .base import FixedState, Mixer, ParamDecl, register_part
from .gated_delta import _pad_rows
from .linear import linear, linear_modules


@register_part("mixer", "hgrn2")
class Hgrn2(Mixer):
    can_store = True          # forward(store=True) writes its rows instead of adding them

    def __init__(self, *, dtype: str, size: int, heads: int, key_dim: int, value_dim: int, norm_eps: float):
        super().__init__()
        self.size, self.H, self.dk, self.dv, self.eps = int(size), int(heads), int(key_dim), int(value_dim), float(norm_eps)
        if self.dk > ops.MAX_SCAN_KEY_DIM:
            raise ConfigError(f"hgrn2: key size {self.dk} is above {ops.MAX_SCAN_KEY_DIM}")
        d, n, m = self.size, self.H * self.dk, self.H * self.dv
        self.decls = {"q.weight": ParamDecl((n, d), init=("normal", 0.05)),
                      "f.weight": ParamDecl((n, d), init=("normal", 0.05)),
                      "f.bias": ParamDecl((n,), role="vector", init=("normal", 1.0)),
                      "lower": ParamDecl((n,), role="vector", init=("uniform", 0.0, 0.9)),
                      "v.weight": ParamDecl((m, d), init=("normal", 0.05)),
                      "norm.weight": ParamDecl((self.dv,), role="vector", init=("uniform", 0.5, 1.5)),
                      "o.weight": ParamDecl((d, m))}

    def prepare(self):
        w = self.w
        mats = [w.pop("q.weight"), w.pop("f.weight"), w.pop("v.weight")]
        if any(m.dtype != mats[0].dtype for m in mats):
            mats = [m.float() for m in mats]
        w["qfv.weight"] = _pad_rows(torch.cat(mats, 0))          # q | f | v rows, one product
        w["f.bias"], w["lower"] = w["f.bias"].contiguous(), w["lower"].contiguous()

    def cache_need(self):
        return FixedState((self.H, self.dk, self.dv))

    def forward(self, h, ctx, cache, out, reads_only=False, store=False):
        if reads_only:
            raise ConfigError("an hgrn2 layer cannot run on another layer's state")
        w, n = self.w, self.H * self.dk
        z = linear(h, w["qfv.weight"], out_dtype=torch.float32)
        o = ops.gated_write_scan(z, n, 2 * n, w["lower"], w["f.bias"], cache.states, ctx.item_start, cache.item_slot,
                                 ctx.n_items, self.H, self.dk, self.dv, max_item_rows=ctx.max_item_rows)
        y = ops.head_norm_gate(o, w["norm.weight"], False, None, None, self.eps, self.H, self.dv, h.dtype)
        linear(y, w["o.weight"], out=out, accumulate=not store)
        return out

    def weight_order(self):
        return [self.w["qfv.weight"], self.w["o.weight"]]

    def kernel_modules(self, dtype):
        return linear_modules(dtype) + [("recurrent", None)]
