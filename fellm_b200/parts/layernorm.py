"""LayerNorm with weight and bias: y = (x - mean) / sqrt(var + eps) * w + b, var the mean of the squared deviations
from the mean, all in float32.

Beside the plain forward() it offers `add_normed(x, y)`: x += LN(y), for arrangements that norm a sublayer's OUTPUT on
its way into the residual stream (one kernel: the sublayer's float32 rows are read once, the stream is updated in
place, and the new rows can be left in the activation dtype for the sublayer that reads the stream next)."""
from __future__ import annotations

from .. import ops
from .base import Norm, ParamDecl, register_part


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    def __init__(self, *, dtype: str, size: int, eps: float):
        super().__init__()
        self.size, self.eps, self.dtype = int(size), float(eps), dtype
        self.decls = {"weight": ParamDecl((self.size,), role="vector", init=("uniform", 0.5, 1.5)),
                      "bias": ParamDecl((self.size,), role="vector", init=("normal", 0.1))}

    def forward(self, x, out_dtype, rows=None):
        return ops.layernorm(x, self.w["weight"], self.w["bias"], self.eps, out_dtype, rows=rows)

    def add_normed(self, x, y, cast=None):
        """x float32 [T, d] += LN(y); `cast`: a tensor of the activation dtype that also gets the new rows."""
        return ops.add_layernorm(x, y, self.w["weight"], self.w["bias"], self.eps, cast=cast)

    def kernel_modules(self, dtype):
        return [("sublayer", None)]
