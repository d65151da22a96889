"""Gates on what a block's sublayers add to the residual stream: sublayer s's result is multiplied, element by
element, by sigmoid(W_s h + b_s), h being the sublayer's own input.  One part owns the gates of all sublayers of a
block that read the same h (one product for their logits, float32); ops.gated_add applies them on the way into the
stream."""
from __future__ import annotations

import torch

from .. import ops
from ..config.errors import ConfigError
from .base import ParamDecl, ResidualGate, register_part
from .linear import linear, linear_modules


@register_part("gate", "sigmoid")
class SigmoidGates(ResidualGate):
    def __init__(self, *, dtype: str, size: int, sublayers: int):
        """Tensors: <s>.weight [size, size], <s>.bias [size] for s < sublayers."""
        super().__init__()
        self.size, self.n = int(size), int(sublayers)
        if not 1 <= self.n <= 2:
            raise ConfigError(f"sigmoid gates: {self.n} sublayers (1 or 2 are taken)")
        self.decls = {}
        for s in range(self.n):
            self.decls[f"{s}.weight"] = ParamDecl((self.size, self.size))
            self.decls[f"{s}.bias"] = ParamDecl((self.size,), role="vector", init=("normal", 0.5))

    def prepare(self):
        mats = [self.w.pop(f"{s}.weight") for s in range(self.n)]
        dt = mats[0].dtype if all(m.dtype == mats[0].dtype for m in mats) else torch.float32
        self.w["weight"] = torch.cat([m.to(dt) for m in mats], 0).contiguous()           # [n size, size]
        self.w["bias"] = torch.cat([self.w.pop(f"{s}.bias") for s in range(self.n)]).contiguous()

    input_rows, input_bias = "weight", "bias"       # the block may make the logits in a product it shares with its sublayers

    def logits(self, h):
        """h [T, size] -> float32 [T, n size]: sublayer s's logits at columns [s size, (s + 1) size)."""
        return linear(h, self.w["weight"], self.w["bias"], out_dtype=torch.float32)

    def add(self, x, results, zg):
        """x += sum over the sublayers of results[s] * sigmoid(zg[:, s])."""
        return ops.gated_add(x, results, zg)

    def weight_order(self):
        return [self.w["weight"]]

    def kernel_modules(self, dtype):
        return linear_modules(dtype) + [("elementwise", None)]
