"""What a token adds to the residual stream by itself, after a block: with e = table[token, offset : offset + m] (a
slice of a table shared by all layers; a layer owns a slice),

    g = gelu_tanh(W_gate x) * e;    y = W_proj g;    x <- x + y / sqrt(mean(y^2) + eps) * w

gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))); the norm's weight is a plain vector.  One kernel per
step and layer (ops.token_side), float32 sums.  The table belongs to a 'shared' part of the model ('table'), which
this part asks for by its tensor's name.  A block whose
sublayers reach the stream through gates hands their results and the gates' logits on to this part, whose kernel
adds them on its way in (one launch less, and the stream is read once)."""
from __future__ import annotations

import torch

from .. import ops
from ..config.errors import ConfigError
from .base import ParamDecl, Shared, SideInput, register_part


@register_part("shared", "table")
class SharedTable(Shared):
    """A [vocab, width] table that several parts read rows of."""

    def __init__(self, *, dtype: str, vocab: int, width: int):
        super().__init__()
        self.decls = {"weight": ParamDecl((int(vocab), int(width)))}

    def prepare(self):
        self.w["weight"] = self.w["weight"].contiguous()


@register_part("side", "token_gated")
class TokenGatedSide(SideInput):
    def __init__(self, *, dtype: str, size: int, dim: int, offset: int, eps: float, table: str):
        """`table`: the tensor name of the shared table; this layer reads columns [offset, offset + dim) of a token's row.
        Tensors: gate.weight [dim, size], proj.weight [size, dim], norm.weight [size]."""
        super().__init__()
        self.size, self.m, self.offset, self.eps, self.uses_shared = int(size), int(dim), int(offset), float(eps), str(table)
        if self.m < 1 or self.offset < 0:
            raise ConfigError(f"token side input: dim {self.m} must be positive and offset {self.offset} not negative")
        self.decls = {"gate.weight": ParamDecl((self.m, self.size), init=("normal", 0.1)),
                      "proj.weight": ParamDecl((self.size, self.m), init=("normal", 0.1)),
                      "norm.weight": ParamDecl((self.size,), role="vector", init=("uniform", 0.5, 1.5))}
        self.table = None

    def attach(self, shared):
        table = shared.w["weight"]
        if self.offset + self.m > table.shape[1]:
            raise ConfigError(f"token side input: columns {self.offset}..{self.offset + self.m - 1} are outside the "
                              f"shared table's {table.shape[1]}")
        wg, wp = self.w["gate.weight"], self.w["proj.weight"]
        if not (table.dtype == wg.dtype == wp.dtype):                    # a file that stores some of them in 32-bit
            table, wg, wp = table.float(), wg.float(), wp.float()
        self.table, self.w["gate.weight"], self.w["proj.weight"] = table, wg.contiguous(), wp.contiguous()

    takes_gated_add = True        # forward(pending=(results, logits)): the gated sublayers' sum is added in the same launch

    def forward(self, x, ctx, pending=None):
        return ops.token_side(x, ctx.tokens, self.table, self.offset, self.w["gate.weight"], self.w["proj.weight"],
                              self.w["norm.weight"], self.eps, status=ctx.status, pending=pending)

    def kernel_modules(self, dtype):
        return [("elementwise", None)]
