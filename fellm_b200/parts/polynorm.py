"""Feed-forward with a polynomial activation over unit powers: f = W_down act(W_up h),

    act(z) = a N(z) + b N(z^2) + c N(z^3) + e,      N(v) = v / sqrt(mean(v^2) + eps) over a token's ff values,

powers taken element by element; (a, b, c, e) is a tensor of the layer.  The up product leaves float32 sums, the
powers and their root mean squares are float32 in both engines, and the activation is rounded once, into the down
product's input."""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, ParamDecl, register_part
from .linear import linear, linear_modules


@register_part("feed_forward", "polynorm")
class PolyNormFeedForward(FeedForward):
    def __init__(self, *, dtype: str, size: int, ff: int, eps: float):
        super().__init__()
        self.size, self.ff, self.eps = int(size), int(ff), float(eps)
        self.decls = {"up.weight": ParamDecl((self.ff, self.size)), "down.weight": ParamDecl((self.size, self.ff)),
                      "act": ParamDecl((4,), role="vector", init=("uniform", 0.2, 0.8))}

    def prepare(self):
        self.w["up.weight"] = self.w["up.weight"].contiguous()
        self.w["down.weight"] = self.w["down.weight"].contiguous()

    can_store = True       # forward(store=True) writes the float32 rows `out` instead of adding into them

    input_rows = "up.weight"        # forward(pre=z): the float32 product of the layer's input with these rows, made elsewhere

    def forward(self, hn, ctx, out, store=False, pre=None):
        z = pre if pre is not None else linear(hn, self.w["up.weight"], out_dtype=torch.float32)
        a = ops.poly_norm(z, self.w["act"], self.eps, hn.dtype)
        if store:
            linear(a, self.w["down.weight"], out=out, out_dtype=torch.float32)
        else:
            linear(a, self.w["down.weight"], out=out, accumulate=True)
        return out

    def weight_order(self):
        return [self.w["up.weight"], self.w["down.weight"]]

    def kernel_modules(self, dtype):
        return linear_modules(dtype) + [("elementwise", None)]
