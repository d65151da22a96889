"""Latent attention: queries, keys and values go through low-rank latents, and the cache keeps per token only ONE
normed key-value latent (rk elements) and ONE rotated key part (dr elements) shared by all heads.

    cq = RMSNorm(W_dq h) w_q                 q_h = W_uq,h cq = [qn_h (dn) | qr_h (dr)]
    [c' | kr] = W_dkv h                      c = RMSNorm(c') w_c              (kr is not normed)
    kn_j,h = W_uk,h c_j      v_j,h = W_uv,h c_j
    s_ij,h = scale (qn_i,h . kn_j,h + rot_i(qr_i,h) . rot_j(kr_j))
    p = softmax over the keys j the window lets i see, the denominator holding exp(sink_h) once more where the layer has sinks
    out = W_o [sum_j p_ij,h v_j,h]_h

Nothing per head is ever stored: with qa_i,h = W_uk,h^T qn_i,h the unrotated part of the score is qa_i,h . c_j, and
sum_j p_ij v_j,h = W_uv,h sum_j p_ij c_j.  So the attention kernel runs over the cached rows [c_j | rot_j(kr_j)] with
queries [qa_i,h | rot_i(qr_i,h)], one key "head" for all query heads, the keys read as the values and only their
first rk elements read out; a product per head before it (W_uk^T) and one behind it (W_uv) do the rest.  `scale` is
the layer's own and is used as given.  The rotation is the position part's (pairs (2i, 2i+1), scaled frequencies and
a magnitude where the part has them); norms, angles, scores and the softmax are float32 in both engines.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.errors import ConfigError
from .base import Mixer, PagedKV, ParamDecl, build_part, register_part
from .gated_delta import _pad_rows, stack_rows
from .linear import linear, linear_modules


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    def __init__(self, *, dtype: str, size: int, heads: int, dim: int, rot_dim: int, v_dim: int, q_rank: int,
                 kv_rank: int, scale: float, norm_eps: float, position, window=None, sink: bool = False):
        """`dim` / `rot_dim`: the unrotated / rotated elements of a head's query and key; `position`: a PartSpec of the
        'position' category for the rot_dim part (adjacent pairs; it may rotate fewer than rot_dim elements, or none).
        Tensors: dq.weight [q_rank, size], dq.norm [q_rank], uq.weight [heads (dim + rot_dim), q_rank],
        dkv.weight [kv_rank + rot_dim, size], dkv.norm [kv_rank], uk.weight [heads dim, kv_rank],
        uv.weight [heads v_dim, kv_rank], o.weight [size, heads v_dim], sink [heads] (with sink=True)."""
        super().__init__()
        self.size, self.H, self.dn, self.dr, self.dv = int(size), int(heads), int(dim), int(rot_dim), int(v_dim)
        self.rq, self.rk, self.scale, self.eps = int(q_rank), int(kv_rank), float(scale), float(norm_eps)
        self.window = None if window is None else int(window)
        self.sink = bool(sink)
        if min(self.H, self.dn, self.dv, self.rq, self.rk) < 1 or self.dr < 0:
            raise ConfigError("latent_attention: heads, dim, v_dim and the ranks must be positive")
        if self.rk + self.dr > ops.ATTENTION_SIMT_MAX_HD:
            raise ConfigError(f"latent_attention: kv_rank + rot_dim = {self.rk + self.dr} is above the attention kernel's "
                              f"{ops.ATTENTION_SIMT_MAX_HD}")
        if self.window is not None and self.window < 1:
            raise ConfigError(f"latent_attention: window {self.window} must be positive")
        self.position = build_part("position", position, dtype)
        self.n_rot = 0
        if self.position.inv_freq is not None:
            self.n_rot = int(self.position.rot_dim)
            if self.position.pairing != "adjacent" or self.n_rot > self.dr:
                raise ConfigError(f"latent_attention: the rotation pairs neighbours and covers at most rot_dim = {self.dr} "
                                  f"elements (got {self.position.pairing}, {self.n_rot})")
        self.magnitude = float(getattr(self.position, "magnitude", 1.0))
        H, d = self.H, self.size
        self.decls = {"dq.weight": ParamDecl((self.rq, d)), "dq.norm": ParamDecl((self.rq,), role="vector", init=("uniform", 0.5, 1.5)),
                      "uq.weight": ParamDecl((H * (self.dn + self.dr), self.rq), init=("normal", 0.1)),
                      "dkv.weight": ParamDecl((self.rk + self.dr, d)),
                      "dkv.norm": ParamDecl((self.rk,), role="vector", init=("uniform", 0.5, 1.5)),
                      "uk.weight": ParamDecl((H * self.dn, self.rk), init=("normal", 0.1)),
                      "uv.weight": ParamDecl((H * self.dv, self.rk), init=("normal", 0.1)),
                      "o.weight": ParamDecl((d, H * self.dv))}
        if self.sink:
            self.decls["sink"] = ParamDecl((H,), role="vector", init=("normal", 1.0))
        # warps that share a (row, head)'s keys in the attention kernel: by the window alone (the order of a row's sums
        # is then the same in every step)
        self.simt_warps = max(1, min(8, -(-(self.window or (1 << 30)) // 128)))

    def cache_need(self):
        # one key "head" of rk + dr elements per token, read as its own value
        return PagedKV(1, self.rk + self.dr, self.window, None, None, True)

    def prepare(self):
        w = self.w
        H, dn, dr, dv, rq, rk = self.H, self.dn, self.dr, self.dv, self.rq, self.rk
        # both down projections read the same input: one product, rows [query latent | key-value latent | key part]
        w["down.weight"], offs = stack_rows([w.pop("dq.weight"), w.pop("dkv.weight")])
        self.q_off, self.c_off = offs[0], offs[1]
        self.r_off = self.c_off + rk
        w["uq.weight"] = _pad_rows(w["uq.weight"])
        # per head: W_uk,h^T as [rk, dn] rows (qa = W_uk,h^T qn) and W_uv,h [dv, rk]
        uk = w.pop("uk.weight")
        w["ukT.weight"] = uk.view(H, dn, rk).transpose(1, 2).contiguous()
        w["uv.weight"] = w["uv.weight"].view(H, dv, rk).contiguous()
        w["o.weight"] = w["o.weight"].contiguous()
        self.position.to(uk.device)

    can_store = True       # forward(store=True) writes the float32 rows `out` instead of adding into them
    input_rows = "down.weight"      # forward(pre=z): the float32 product of the layer's input with these rows, made elsewhere

    def forward(self, xn, ctx, cache, out, reads_only=False, store=False, pre=None):
        if reads_only:
            raise ConfigError("latent_attention: the layer keeps a cache of its own")
        w = self.w
        H, dn, dr, dv, rq, rk = self.H, self.dn, self.dr, self.dv, self.rq, self.rk
        z = pre if pre is not None else linear(xn, w["down.weight"], out_dtype=torch.float32)
        cq = ops.latent_prep(z, self.q_off, rq, self.c_off, rk, self.r_off, dr, w["dq.norm"], w["dkv.norm"], self.eps,
                             self.position.inv_freq, self.n_rot, self.magnitude, ctx.positions, ctx.row_slot, cache,
                             xn.dtype, status=ctx.status)
        q = linear(cq, w["uq.weight"])
        T = q.shape[0]
        on_mma = ops.latent_attention_takes(q, cache.pool, rk, dr, cache.page_tokens)
        if on_mma and ctx.max_item_rows * H <= ops.LATENT_SINGLE_ROWS and ops.latent_rotate_fusable(q, dn + dr, dn):
            # single tokens: the attention kernel rotates the queries' rotated parts itself, on their way into shared
            # memory (a launch less; for portions the rotation in front is cheaper than the kernel's longer start)
            qa = torch.empty((T, H * rk), dtype=q.dtype, device=q.device)
            ops.head_gemm(q, w["ukT.weight"], qa, a_head=dn + dr, out_head=rk)
            a = ops.latent_attention(qa, H, rk, dr, cache.pool, cache.block_table, ctx.positions, ctx.row_slot, ctx.item_start,
                                     ctx.n_items, ctx.max_item_rows, ctx.max_len, cache.layer, cache.page_tokens, self.scale,
                                     window=self.window, sinks=w.get("sink"),
                                     q_rot=(q, dn + dr, dn, self.position.inv_freq, self.n_rot, self.magnitude))
            return self._read_out(a, T, out, store)
        qa = torch.empty((T, H * (rk + dr)), dtype=q.dtype, device=q.device)
        ops.head_gemm(q, w["ukT.weight"], qa, a_head=dn + dr, out_head=rk + dr)
        ops.latent_rotate_q(q, H, dn, dr, qa, rk, self.position.inv_freq, self.n_rot, self.magnitude, ctx.positions)
        if on_mma:
            a = ops.latent_attention(qa, H, rk, dr, cache.pool, cache.block_table, ctx.positions, ctx.row_slot, ctx.item_start,
                                     ctx.n_items, ctx.max_item_rows, ctx.max_len, cache.layer, cache.page_tokens, self.scale,
                                     window=self.window, sinks=w.get("sink"))
        else:
            # the 32-bit engine, and sizes the tensor-core kernel does not take
            a = ops.paged_attention_general(qa, H, rk + dr, 0, cache.pool, cache.block_table, ctx.positions, ctx.row_slot,
                                            cache.layer, cache.page_tokens, 1, self.scale, window=self.window,
                                            warps=self.simt_warps, sinks=w.get("sink"), out_dim=rk)
        return self._read_out(a, T, out, store)

    def _read_out(self, a, T, out, store):
        """The heads' values out of the latent's read-out, then W_o."""
        w = self.w
        o = torch.empty((T, self.H * self.dv), dtype=a.dtype, device=a.device)
        ops.head_gemm(a, w["uv.weight"], o, a_head=self.rk, out_head=self.dv)
        if store:
            linear(o, w["o.weight"], out=out, out_dtype=torch.float32)
        else:
            linear(o, w["o.weight"], out=out, accumulate=True)
        return out

    def weight_order(self):
        return [self.w["down.weight"], self.w["uq.weight"], self.w["o.weight"]]

    def kernel_modules(self, dtype):
        mods = linear_modules(dtype) + [("latent", None), ("attention_simt", None)]
        if dtype == "bfloat16" and self.rk % 32 == 0 and 32 <= self.rk <= 512 and (self.rk + self.dr) % 16 == 0:
            mods += ops.latent_attention_modules(self.rk, self.dr)
        return mods
