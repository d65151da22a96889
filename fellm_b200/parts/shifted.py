"""Token shift in front of any mixer: what the mixer reads of token t is

    h_t = x_t + (x_(t-1) - x_t) * s          (s a tensor of the layer, one value a channel; x_(-1) = 0)

where x is the residual stream itself, as it was before the shift.  The previous token's row is kept per request in
float32 (FixedState), beside whatever the inner mixer keeps; the shift is computed in float32 from the float32 stream
and rounded once to the activation dtype.  The part therefore reads the STREAM (`reads_stream`): an arrangement hands
it the float32 rows, not a normed or cast copy.

The row it keeps is the part's own even where the inner mixer reads the cache of another schedule entry
(`private_need`): forward() then gets `cache` = (its own views, the other entry's views)."""
from __future__ import annotations

import torch

from .. import ops
from ..config.errors import ConfigError
from .base import FixedState, Mixer, ParamDecl, build_part, register_part


def _as_list(need):
    return list(need) if isinstance(need, (list, tuple)) else ([] if need is None else [need])


@register_part("mixer", "token_shifted")
class TokenShifted(Mixer):
    reads_stream = True

    def __init__(self, *, dtype: str, size: int, inner):
        """`inner`: a PartSpec of the 'mixer' category.  Own tensor: shift [size]."""
        super().__init__()
        self.size = int(size)
        self.act_dtype = torch.bfloat16 if dtype == "bfloat16" else torch.float32
        self.inner = build_part("mixer", inner, dtype)
        self.decls = {"shift": ParamDecl((self.size,), role="vector", init=("uniform", 0.0, 1.0))}
        need = self.inner.cache_need()
        self._inner_is_list = isinstance(need, (list, tuple))

    @property
    def can_store(self):
        return getattr(self.inner, "can_store", False)

    def children(self):
        return [self.inner]

    def cache_need(self):
        return [FixedState((self.size,))] + _as_list(self.inner.cache_need())

    def private_need(self):
        return [FixedState((self.size,))]

    def forward(self, x, ctx, cache, out, reads_only=False, **kw):
        if x.dtype != torch.float32:
            raise ConfigError("token_shifted reads the float32 residual stream itself")
        if reads_only:
            own, other = cache
            mine, rest = own[0], list(other[1:])
        else:
            mine, rest = cache[0], list(cache[1:])
        h = ops.token_shift(x, self.w["shift"], mine.states, ctx.item_start, mine.item_slot, ctx.n_items,
                            ctx.max_item_rows, self.act_dtype, row_item=ctx.row_item)
        inner_cache = rest if self._inner_is_list else (rest[0] if rest else None)
        return self.inner.forward(h, ctx, inner_cache, out, reads_only=reads_only, **kw)

    def weight_order(self):
        return self.inner.weight_order()

    def kernel_modules(self, dtype):
        return [("recurrent", None)]
