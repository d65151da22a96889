"""Connectors: what rewrites the residual stream between two blocks.

'concat_proj': x <- W [x ; x0] + step[t], with x0 the embedding's output and t the number of the
pass that starts: the entry of a pass of a looped run of layers (the same weights run several
times in a row, each pass with caches of its own).

'add_step': x <- x + step[t]: the same entry without a projection and without the embedding.

'add_embedding': x <- x + x0: the embedding's output added again; it owns no tensor and does nothing before the first
pass."""
from __future__ import annotations

import torch

from .. import ops
from .base import Connector, ParamDecl, register_part
from .linear import linear, linear_modules


@register_part("connector", "concat_proj")
class ConcatProjection(Connector):
    def __init__(self, *, dtype: str, size: int, steps: int):
        super().__init__()
        self.size, self.steps = int(size), int(steps)
        self.decls = {"in.weight": ParamDecl((self.size, 2 * self.size)),
                      "step": ParamDecl((self.steps, self.size), role="vector", init=("normal", 0.05))}

    def forward(self, x, x0, step, act_dtype):
        xc = ops.concat_cast(x, x0, act_dtype)
        ops.residual_written(x)
        return linear(xc, self.w["in.weight"], self.w["step"][step], out=x, out_dtype=torch.float32)

    def weight_order(self):
        return [self.w["in.weight"]]

    def kernel_modules(self, dtype):
        return linear_modules(dtype) + [("elementwise", None)]


@register_part("connector", "add_step")
class AddStep(Connector):
    needs_embedding = False

    def __init__(self, *, dtype: str, size: int, steps: int):
        super().__init__()
        self.size, self.steps = int(size), int(steps)
        self.decls = {"step": ParamDecl((self.steps, self.size), role="vector", init=("normal", 0.05))}

    def forward(self, x, x0, step, act_dtype):
        return ops.add_row_vector(x, self.w["step"][step])

    def kernel_modules(self, dtype):
        return [("elementwise", None)]


@register_part("connector", "add_embedding")
class AddEmbedding(Connector):
    def __init__(self, *, dtype: str, size: int):
        super().__init__()
        self.size = int(size)

    def forward(self, x, x0, step, act_dtype):
        return x if step == 0 else ops.add_rows(x, x0)

    def kernel_modules(self, dtype):
        return [("elementwise", None)]
