"""Routed experts: a feed-forward made of `experts` small gated feed-forwards of which every token uses `top`.

    z = W_router h, float32;  s = softmax(z) over all experts
    the `top` experts with the largest scores are chosen (ties: the lower expert)
    weights = their scores as they are (renormalize=True: divided by their sum)
    out = sum over the chosen experts, in the order of their scores, of weight * W_down (SiLU(W_gate h) * (W_up h))

With score="sigmoid" the scores are s = sigmoid(z); the choice is made on s + correction (a tensor of the layer), and
with groups=(count, keep, best) only inside the `keep` of `count` equal groups of neighbouring experts whose `best`
largest choice scores sum highest; the weights stay the plain s (renormalize: over their sum).  With
act=("clamped", limit, alpha) an expert computes min(g, limit) sigmoid(alpha min(g, limit)) (clamp(u, -limit, limit) + 1)
in place of SiLU(g) u.

With router_bias=True the logits are z = W_router h + b (b a tensor of the layer).  With renormalize=True the softmax
scores over their sum ARE the softmax over the chosen logits alone.  With plain="relu2" an expert has no gate:
W_down relu(W_up h)^2 (the first grouped product leaves float32 rows, ops.relu2 squares them into the activation dtype).

Experts have no biases.  Nothing goes through the host: the router's choices are sorted by expert on the device
(ops.moe_plan; the router's product and the routing are one launch, ops.moe_router) and two grouped products walk
the sorted rows (tcgen05 for steps of many rows, mma.sync tiles between, a warp a column for a handful of tokens), the first gathering its input rows by token and
applying SiLU(gate) * up in its epilogue, the second leaving float32 rows that ops.moe_combine adds, weighted, into
the residual stream.  A token's result does not depend on what else is in the step.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.errors import ConfigError
from .base import FeedForward, ParamDecl, register_part
from .linear import linear_modules


@register_part("feed_forward", "moe")
class RoutedExperts(FeedForward):
    def __init__(self, *, dtype: str, size: int, ff: int, experts: int, top: int, renormalize: bool = False,
                 score: str = "softmax", correction: bool = False, groups=None, act=None, router_bias: bool = False,
                 plain=None):
        super().__init__()
        self.size, self.ff, self.E, self.top = int(size), int(ff), int(experts), int(top)
        self.renormalize = bool(renormalize)
        if not 1 <= self.top <= min(self.E, ops.MOE_MAX_TOP):
            raise ConfigError(f"moe: top {self.top} must be in 1..{min(self.E, ops.MOE_MAX_TOP)} ({self.E} experts)")
        if score not in ("softmax", "sigmoid"):
            raise ConfigError(f"moe: unknown score {score!r} (softmax, sigmoid)")
        if score == "softmax" and (correction or groups):
            raise ConfigError("moe: a correction of the choice and groups of experts go with sigmoid scores")
        self.score, self.groups = score, None
        if groups:
            count, keep, best = (int(v) for v in groups)
            if count < 1 or self.E % count or not 1 <= keep <= count or best < 1:
                raise ConfigError(f"moe: {count} groups (keep {keep}) do not divide {self.E} experts")
            if self.top > (self.E // count) * keep:
                raise ConfigError(f"moe: top {self.top} is above the {(self.E // count) * keep} experts of {keep} groups")
            self.groups = (count, keep, best)
        self.act = None
        if act:
            kind, limit, alpha = act
            if kind != "clamped" or not float(limit) > 0.0:
                raise ConfigError(f"moe: unknown expert activation {act!r} (('clamped', limit > 0, alpha))")
            self.act = (float(limit), float(alpha))
        if plain not in (None, "relu2"):
            raise ConfigError(f"moe: unknown activation of plain experts {plain!r} (relu2)")
        if plain and act:
            raise ConfigError("moe: plain experts have no gated activation")
        self.plain = plain
        self.decls = {"router.weight": ParamDecl((self.E, self.size), init=("normal", 0.5))}
        if router_bias:
            self.decls["router.bias"] = ParamDecl((self.E,), role="vector", init=("normal", 0.5))
        if correction:
            self.decls["correction"] = ParamDecl((self.E,), role="vector", init=("normal", 0.2))
        for e in range(self.E):
            if not self.plain:
                self.decls[f"e{e}.gate.weight"] = ParamDecl((self.ff, self.size))
            self.decls[f"e{e}.up.weight"] = ParamDecl((self.ff, self.size))
            self.decls[f"e{e}.down.weight"] = ParamDecl((self.size, self.ff))

    def prepare(self):
        w = self.w
        if self.plain:
            ups = [w.pop(f"e{e}.up.weight") for e in range(self.E)]
            downs = [w.pop(f"e{e}.down.weight") for e in range(self.E)]
            dt = ups[0].dtype if all(m.dtype == ups[0].dtype for m in ups + downs) else torch.float32
            self.interleaved = False
            w["up.weight"] = torch.stack([m.to(dt) for m in ups], 0).contiguous()          # [E, ff, d]
            w["down.weight"] = torch.stack([m.to(dt) for m in downs], 0).contiguous()      # [E, d, ff]
            w["router.weight"] = w["router.weight"].contiguous()
            return
        mats = [w.pop(f"e{e}.{n}.weight") for e in range(self.E) for n in ("gate", "up", "down")]
        dt = mats[0].dtype if all(m.dtype == mats[0].dtype for m in mats) else torch.float32
        # on the tensor-core paths an expert's gate and up rows lie in blocks of 8 by turns, as the dense feed-forward's do
        self.interleaved = dt == torch.bfloat16 and mats[0].is_cuda and self.ff % 8 == 0 and self.size % 8 == 0
        if self.interleaved:
            gu = [ops.interleave_gate_up(mats[3 * e], mats[3 * e + 1]) for e in range(self.E)]
        else:
            gu = [torch.cat([mats[3 * e].to(dt), mats[3 * e + 1].to(dt)], 0) for e in range(self.E)]
        w["gate_up.weight"] = torch.stack(gu, 0).contiguous()                                  # [E, 2 ff, d]
        w["down.weight"] = torch.stack([mats[3 * e + 2].to(dt) for e in range(self.E)], 0).contiguous()     # [E, d, ff]
        w["router.weight"] = w["router.weight"].contiguous()

    can_store = True          # forward(store=True) writes its rows instead of adding them

    def forward(self, hn, ctx, out, store=False):
        w = self.w
        idx, score = ops.moe_router(hn, w["router.weight"], self.top, self.renormalize, score=self.score,
                                    correction=w.get("correction"), groups=self.groups, bias=w.get("router.bias"))
        first = w["up.weight"] if self.plain else w["gate_up.weight"]
        if hn.dtype != first.dtype:          # a file that stores some experts in 32-bit under a bfloat16 engine
            hn = hn.to(first.dtype)
        bf = hn.dtype == torch.bfloat16
        k_ok = self.ff % 8 == 0 and self.size % 8 == 0 and hn.stride(0) % 8 == 0
        tile = ops.moe_row_tile(idx.numel(), bf, k_ok and (self.interleaved or bool(self.plain)))
        plan = ops.moe_plan(idx, self.E, tile)
        if self.plain:
            a = ops.relu2(ops.moe_gemm(hn, first, plan, gated=False, gather=True), hn.dtype)
            y = ops.moe_gemm(a, w["down.weight"], plan, gated=False, gather=False)
            ops.moe_combine(out, y, plan, score, store=store)
            return out
        a = ops.moe_gemm(hn, w["gate_up.weight"], plan, gated=True, gather=True, interleaved=self.interleaved, act=self.act)
        y = ops.moe_gemm(a, w["down.weight"], plan, gated=False, gather=False)
        ops.moe_combine(out, y, plan, score, store=store)
        return out

    def weight_order(self):
        return [self.w["router.weight"], self.w["up.weight" if self.plain else "gate_up.weight"], self.w["down.weight"]]

    def kernel_modules(self, dtype):
        return linear_modules(dtype) + [("moe", None)] + ([("sublayer", None)] if self.plain else [])
