"""RMSNorm: y = x * 1/sqrt(mean(x^2) + eps) * w (crates/backend-cpu/src/kernels/norm.rs:6-39).

'rmsnorm_groups': the row in `groups` equal consecutive parts, each divided by its own root mean square, then the
weight over the whole row."""
from __future__ import annotations

import torch

from .. import ops
from ..config.errors import ConfigError
from .base import Norm, ParamDecl, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    def __init__(self, *, dtype: str, size: int, eps: float):
        super().__init__()
        self.size, self.eps, self.dtype = int(size), float(eps), dtype
        self.decls = {"weight": ParamDecl((self.size,), role="vector", init=("ones",))}

    def forward(self, x, out_dtype, rows=None):
        return ops.rmsnorm(x, self.w["weight"], self.eps, out_dtype, rows=rows)

    def reserve(self, device, max_rows, n_ctx):
        if self.w["weight"].dtype == torch.float32 and self.dtype == "bfloat16":
            ops.reserve_norm_handoff(device, self.size)

    def expect(self, x):
        ops.expect_norm(x, self.w["weight"])

    def kernel_modules(self, dtype):
        return [("elementwise", None)]


@register_part("norm", "rmsnorm_groups")
class GroupedRMSNorm(Norm):
    def __init__(self, *, dtype: str, size: int, eps: float, groups: int):
        super().__init__()
        self.size, self.eps, self.groups, self.dtype = int(size), float(eps), int(groups), dtype
        if self.groups < 1 or self.size % self.groups:
            raise ConfigError(f"rmsnorm_groups: {self.groups} groups do not divide a row of {self.size}")
        self.decls = {"weight": ParamDecl((self.size,), role="vector", init=("ones",))}

    def forward(self, x, out_dtype, rows=None):
        return ops.rmsnorm_groups(x, self.w["weight"], self.eps, self.groups, out_dtype, rows=rows)

    def kernel_modules(self, dtype):
        return [("elementwise", None)]
