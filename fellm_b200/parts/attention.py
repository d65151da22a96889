"""GQA attention mixer with optional per-head QK RMSNorm and a position encoding, over the
paged cache (crates/fellm-model/src/graph.rs:2014-2246 for one token, 856-1050 for a batch):
q,k,v = W xn; RMSNorm per head on q,k; rotary on q,k; k (normed, rotated) and v written to the
cache; scores scaled by 1/sqrt(hd); kv head g = h // (H/G); causal, optionally windowed; W_o.

Beyond FeLLM's attention the part takes, as parameters: a scale of its own, a soft cap on the scores
(cap * tanh(s / cap)), values of another size than keys (v_dim), blocks of `chunk` positions that a
query does not look out of (counted from position 0 of the sequence), and a gate per head,
sigmoid(W_g h), on the head's output before W_o; biases on the q, k (v) and output projections; values
that are the keys themselves (no W_v, and the cache keeps the keys alone); a bias by distance taken
off the scaled score, slope_h (i - j) with slope_h = 2^(-slope_exp (h + 1) / H); and a query
temperature by position, q times 1 + coef ln(floor((p + 1) / every) + 1).  Any of these but the
biases sends the layer to the general attention kernels (float32 softmax in both engine dtypes);
without them the tensor-core kernels run as before.

Two more, also on the general kernels: `unit_qk_norm`, q and k divided by their root mean square over the head (no
weight) BEHIND the rotation, and `out_gate`, the heads' outputs side by side times sigmoid(W_g h) element by element
(W_g [H v_dim, size], part of the input product) before W_o.  With them the general kernels also take a rotation
(the rows of the input product are rotated and normed where they lie, ops.qk_rotate_norm, and the cache write and
the attention read them from there) and a layer that reads another layer's pages; `cache_window` is then the
window the PAGES are kept for, where other layers with wider windows read them too."""
from __future__ import annotations

import math

import torch

from .. import ops
from ..config.errors import ConfigError
from .base import Mixer, PagedKV, ParamDecl, build_part, register_part
from .linear import linear, linear_modules


@register_part("mixer", "attention")
class Attention(Mixer):
    def __init__(self, *, dtype: str, size: int, heads: int, kv_heads: int, head_dim: int, qk_norm: bool,
                 norm_eps: float, position, window=None, shares_cache: bool = False, scale=None, softcap=None,
                 v_dim=None, chunk=None, head_gate: bool = False, bias: bool = False, values_are_keys: bool = False,
                 slope_exp=None, q_temp=None, unit_qk_norm: bool = False, out_gate: bool = False, cache_window="same"):
        """`position`: a PartSpec of the 'position' category.  `shares_cache`: this layer keeps no
        keys and values (it has no k/v weights) and reads those of the run its schedule entry
        names."""
        super().__init__()
        self.size, self.H, self.G, self.hd = int(size), int(heads), int(kv_heads), int(head_dim)
        if self.H % self.G:
            raise ConfigError(f"attention: {self.H} heads are not a multiple of {self.G} kv heads")
        self.unit_qk_norm, self.out_gate = bool(unit_qk_norm), bool(out_gate)
        self.in_place = self.unit_qk_norm or self.out_gate        # rotation and norm where the product left q and k
        general = bool(softcap or chunk or head_gate or (v_dim is not None and int(v_dim) != self.hd) or bias
                       or values_are_keys or slope_exp or q_temp or self.in_place)
        if general and not 1 <= self.hd <= 256:
            raise ConfigError(f"attention: head_dim {self.hd} must be in 1..256")
        if not general and (self.hd % 16 or not 16 <= self.hd <= 256):       # the tensor-core kernels' sizes
            raise ConfigError(f"attention: head_dim {self.hd} must be a multiple of 16 in 16..256")
        self.qk_norm, self.eps = bool(qk_norm), float(norm_eps)
        self.window = None if window is None else int(window)
        self.cache_window = self.window if cache_window == "same" else (None if cache_window is None else int(cache_window))
        if self.cache_window is not None and (self.window is None or self.cache_window < self.window):
            raise ConfigError(f"attention: pages kept for {self.cache_window} positions do not cover the window {self.window}")
        self.shares_cache = bool(shares_cache)
        self.position = build_part("position", position, dtype)
        # what the kernels need of a position part: inv_freq (float32 [rot_dim/2], or None for no
        # rotation), pairing, rot_dim <= head_dim (the rotated leading elements of a head)
        self.rot_dim = self.hd if self.position.inv_freq is None else int(getattr(self.position, "rot_dim", self.hd))
        if self.position.inv_freq is not None and (self.rot_dim % 2 or not 2 <= self.rot_dim <= self.hd):
            raise ConfigError(f"attention: rotary dimension {self.rot_dim} must be even and within head_dim {self.hd}")
        if self.position.inv_freq is not None and self.position.inv_freq.numel() != self.rot_dim // 2:
            raise ConfigError(f"attention: the position part gives {self.position.inv_freq.numel()} frequencies "
                              f"for a rotary dimension of {self.rot_dim}")
        self.scale = 1.0 / math.sqrt(self.hd) if scale is None else float(scale)      # FeLLM fixes it in code, graph.rs:2379
        self.softcap = None if not softcap else float(softcap)
        self.vd = self.hd if v_dim is None else int(v_dim)
        self.chunk = None if chunk is None else int(chunk)
        self.head_gate = bool(head_gate)
        self.bias, self.values_are_keys = bool(bias), bool(values_are_keys)
        self.slope_exp = None if not slope_exp else float(slope_exp)
        self.q_temp = None
        if q_temp:
            coef, every = q_temp
            if int(every) < 1:
                raise ConfigError(f"attention: the query temperature's step {every} must be positive")
            self.q_temp = (float(coef), int(every))
        if self.values_are_keys and self.vd != self.hd:
            raise ConfigError(f"attention: values that are the keys have the keys' size {self.hd}, not {self.vd}")
        self.general = general
        # warps that share a (row, head)'s keys in the CUDA-core kernel: by the window (or chunk) alone, so that the order
        # of a row's sums is the same in every step
        span = min(x for x in (self.window, None if chunk is None else int(chunk), 1 << 30) if x)
        self.simt_warps = max(1, min(8, -(-span // 128)))
        if self.general:
            if self.qk_norm or ((self.position.inv_freq is not None or self.shares_cache) and not self.in_place):
                raise ConfigError("attention: a soft cap, v_dim, chunk or head gate goes with no weighted QK norm and, without "
                                  "unit_qk_norm or out_gate, with no rotation and a cache of the layer's own")
            if self.in_place and (self.hd > 512 or values_are_keys or head_gate or slope_exp or q_temp or bias):
                raise ConfigError(f"attention: unit_qk_norm and out_gate take heads of up to 512 (got {self.hd}) and go with no "
                                  "bias, head gate, distance slopes, query temperature or values that are keys")
            if self.vd > 256 or self.vd < 1 or (self.chunk is not None and self.chunk < 1):
                raise ConfigError(f"attention: v_dim {self.vd} must be in 1..256 and chunk positive")
        d, H, G, hd = self.size, self.H, self.G, self.hd
        self.decls = {"q_proj.weight": ParamDecl((H * hd, d)), "out_proj.weight": ParamDecl((d, H * self.vd))}
        if not self.shares_cache:
            self.decls["k_proj.weight"] = ParamDecl((G * hd, d))
            if not self.values_are_keys:
                self.decls["v_proj.weight"] = ParamDecl((G * self.vd, d))
        if self.bias:
            rows = {"q_proj": H * hd, "k_proj": G * hd, "v_proj": G * self.vd, "out_proj": d}
            for name, n in rows.items():
                if name + ".weight" in self.decls:
                    self.decls[name + ".bias"] = ParamDecl((n,), role="vector", init=("normal", 0.01))
        if self.head_gate:
            self.decls["gate.weight"] = ParamDecl((H, d), init=("normal", 0.1))
        if self.out_gate:
            self.decls["out_gate.weight"] = ParamDecl((H * self.vd, d), init=("normal", 0.05))
        if self.qk_norm:
            self.decls["q_norm.weight"] = ParamDecl((hd,), role="vector", init=("ones",))
            if not self.shares_cache:
                self.decls["k_norm.weight"] = ParamDecl((hd,), role="vector", init=("ones",))

    takes_lazy_norm = True

    def cache_need(self):
        return PagedKV(self.G, self.hd, self.cache_window, self.chunk, None if self.vd == self.hd else self.vd,
                       self.values_are_keys)

    def prepare(self):
        q = self.w.pop("q_proj.weight")
        if self.shares_cache:
            self.w["qkv.weight"] = q.contiguous()
        else:
            mats = [q, self.w.pop("k_proj.weight")] + ([] if self.values_are_keys else [self.w.pop("v_proj.weight")])
            if any(m.dtype != q.dtype for m in mats):
                mats = [m.float() for m in mats]
            self.w["qkv.weight"] = torch.cat(mats, dim=0).contiguous()      # [(H+2G)*hd, d]; [(H+G)*hd, d] without W_v
        if self.out_gate:
            # the gate's rows ride in the input product, behind q (k, v), from a column that is a multiple of 8
            g, m = self.w.pop("out_gate.weight"), self.w["qkv.weight"]
            if g.dtype != m.dtype:
                g, m = g.float(), m.float()
            from .gated_delta import _pad_rows as pad
            m = pad(m, 8)
            self.gate_off = m.shape[0]
            self.w["qkv.weight"] = torch.cat([m, g], 0).contiguous()
        if self.bias:
            names = ["q_proj.bias"] + ([] if self.shares_cache else ["k_proj.bias"] + ([] if self.values_are_keys else ["v_proj.bias"]))
            self.w["qkv.bias"] = torch.cat([self.w.pop(n) for n in names]).contiguous()
        if self.general:
            from .gated_delta import _pad_rows
            n = self.w["qkv.weight"].shape[0]
            self.w["qkv.weight"] = _pad_rows(self.w["qkv.weight"])
            if self.bias:
                extra = self.w["qkv.weight"].shape[0] - n
                self.w["qkv.bias"] = torch.cat([self.w["qkv.bias"], self.w["qkv.bias"].new_zeros(extra)]).contiguous()
            if self.slope_exp is not None:
                # float64 on the host, rounded once
                self.w["slopes"] = torch.tensor([2.0 ** (-self.slope_exp * (h + 1) / self.H) for h in range(self.H)],
                                                dtype=torch.float64).to(torch.float32).to(q.device)
            if self.head_gate:
                self.w["gate.weight"] = _pad_rows(self.w["gate.weight"])
        self.position.to(q.device)

    def reserve(self, device, max_rows, n_ctx):
        if self.w["qkv.weight"].dtype == torch.bfloat16 and not self.general:
            floats, counters = ops.decode_scratch_need(max_rows, self.H, self.G, self.hd, n_ctx)
            ops.reserve_decode_scratch(device, 1, self.H, self.G, self.hd, 1, floats=floats, counters=counters)

    can_store = property(lambda self: self.general)        # (the general path's forward(store=True) writes its rows)

    def forward(self, xn, ctx, cache, out, reads_only=False, store=False):
        if reads_only != self.shares_cache:
            raise ConfigError("attention: a layer built with shares_cache must run with cache_of, and only it")
        if self.general:
            return self._forward_general(xn, ctx, cache, out, store)
        if store:
            raise ConfigError("attention: only the general kernels' path writes its rows instead of adding them")
        G = 0 if self.shares_cache else self.G
        qkv = linear(xn, self.w["qkv.weight"])
        if (ctx.all_single and not self.shares_cache and qkv.dtype == torch.bfloat16 and self.rot_dim == self.hd
                and ops.decode_fuses_rope(self.H, self.G, self.hd, cache.page_tokens, cache.pool)):
            # a decode step: norm, rotation and the cache write happen inside the attention kernel
            a = ops.attention_decode(None, cache.pool, cache.block_table, ctx.positions, ctx.row_slot, cache.layer,
                                     self.scale, self.window, ctx.max_len,
                                     fuse=(qkv, self.w.get("q_norm.weight"), self.w.get("k_norm.weight"), self.eps,
                                           self.position.inv_freq, self.position.pairing))
            linear(a, self.w["out_proj.weight"], out=out, accumulate=True)
            return out
        q = ops.qk_rope_write(qkv, self.w.get("q_norm.weight"), self.w.get("k_norm.weight"), self.eps,
                              self.position.inv_freq, self.position.pairing, ctx.positions, ctx.row_slot,
                              cache.block_table, cache.pool, cache.layer, cache.page_tokens, self.H, G,
                              self.hd, write_kv=not self.shares_cache, status=ctx.status, rot_dim=self.rot_dim)
        a = ops.paged_attention(q, cache, ctx, self.scale, self.window)
        linear(a, self.w["out_proj.weight"], out=out, accumulate=True)
        return out

    def _forward_general(self, xn, ctx, cache, out, store=False):
        """q, k, v as the product leaves them (rotated and normed in place where the part says so): k and v into the
        pages, then attention over the pages with the part's scale, cap, window, chunk and gate."""
        H, G, hd, vd = self.H, self.G, self.hd, self.vd
        gate = linear(xn, self.w["gate.weight"], out_dtype=torch.float32) if self.head_gate else None
        qkv = linear(xn, self.w["qkv.weight"], self.w.get("qkv.bias"))
        if self.values_are_keys:
            vd = 0              # nothing is kept beside the keys; the read-out has their size
        if self.in_place:
            return self._forward_in_place(qkv, ctx, cache, out, store)
        if ctx.all_single:
            # a decode step: the kernel reads each row's own key and value from the row and writes them into the page itself
            a = ops.paged_attention_general(qkv, H, hd, vd, cache.pool, cache.block_table, ctx.positions, ctx.row_slot,
                                            cache.layer, cache.page_tokens, G, self.scale, window=self.window,
                                            chunk=self.chunk, softcap=self.softcap, gate=gate,
                                            slopes=self.w.get("slopes"), q_temp=self.q_temp, warps=self.simt_warps,
                                            write_new=(H * hd, (H + G) * hd, ctx.status))
            linear(a, self.w["out_proj.weight"], self.w.get("out_proj.bias"), out=out, accumulate=True)
            return out
        ops.kv_write(qkv, H * hd, (H + G) * hd, cache.pool, cache.block_table, ctx.positions, ctx.row_slot, cache.layer,
                     cache.page_tokens, G, hd, vd, status=ctx.status)
        if self._on_tensor_cores(qkv):
            # portions of prompts: the tensor-core kernel (keys and values of one size)
            a = ops.attention_prefill_general(qkv, H, cache.pool, cache.block_table, ctx.positions, ctx.row_slot,
                                              ctx.item_start, ctx.n_items, ctx.max_item_rows, cache.layer, self.scale,
                                              window=self.window, chunk=self.chunk, softcap=self.softcap, gate=gate,
                                              slopes=self.w.get("slopes"), q_temp=self.q_temp,
                                              values_are_keys=(G, cache.page_tokens, hd) if self.values_are_keys else None)
        else:
            a = ops.paged_attention_general(qkv, H, hd, vd, cache.pool, cache.block_table, ctx.positions, ctx.row_slot,
                                            cache.layer, cache.page_tokens, G, self.scale, window=self.window,
                                            chunk=self.chunk, softcap=self.softcap, gate=gate,
                                            slopes=self.w.get("slopes"), q_temp=self.q_temp, warps=self.simt_warps)
        linear(a, self.w["out_proj.weight"], self.w.get("out_proj.bias"), out=out, accumulate=True)
        return out

    def _forward_in_place(self, qkv, ctx, cache, out, store):
        H, hd, vd = self.H, self.hd, self.vd
        G = 0 if self.shares_cache else self.G              # heads of k (and v) in the rows of this layer's product
        if self.position.inv_freq is not None or self.unit_qk_norm:
            ops.qk_rotate_norm(qkv, H, G, H * hd, hd, self.rot_dim, self.position.inv_freq, self.position.pairing,
                               ctx.positions, self.eps, unit_norm=self.unit_qk_norm)
        kw = dict(window=self.window, chunk=self.chunk, softcap=self.softcap, warps=self.simt_warps)
        if ctx.all_single:
            write = None if self.shares_cache else (H * hd, (H + G) * hd, ctx.status)
            a = ops.paged_attention_general(qkv, H, hd, vd, cache.pool, cache.block_table, ctx.positions, ctx.row_slot,
                                            cache.layer, cache.page_tokens, self.G, self.scale, write_new=write, **kw)
        else:
            if not self.shares_cache:
                ops.kv_write(qkv, H * hd, (H + G) * hd, cache.pool, cache.block_table, ctx.positions, ctx.row_slot,
                             cache.layer, cache.page_tokens, G, hd, vd, status=ctx.status)
            if self._on_tensor_cores(qkv):
                a = ops.attention_prefill_general(qkv, H, cache.pool, cache.block_table, ctx.positions, ctx.row_slot,
                                                  ctx.item_start, ctx.n_items, ctx.max_item_rows, cache.layer, self.scale,
                                                  window=self.window, chunk=self.chunk, softcap=self.softcap)
            else:
                a = ops.paged_attention_general(qkv, H, hd, vd, cache.pool, cache.block_table, ctx.positions,
                                                ctx.row_slot, cache.layer, cache.page_tokens, self.G, self.scale, **kw)
        if self.out_gate:
            ops.gate_mul(a, qkv[:, self.gate_off:self.gate_off + H * vd])
        linear(a, self.w["out_proj.weight"], self.w.get("out_proj.bias"), out=out, accumulate=not store)
        return out

    def _on_tensor_cores(self, qkv) -> bool:
        return (qkv.dtype == torch.bfloat16 and self.vd == self.hd and self.hd % 16 == 0 and self.hd <= 256
                and self.H // self.G <= 64 and ops.GENERAL_ATTENTION_MMA)

    def weight_order(self):
        return [self.w["qkv.weight"], self.w["out_proj.weight"]]

    def kernel_modules(self, dtype):
        if self.general:
            mma = dtype == "bfloat16" and self.vd == self.hd and self.hd % 16 == 0 and self.H // self.G <= 64
            extra = ([("qk_rope_write", None)] if self.in_place else []) + ([("sublayer", None)] if self.out_gate else [])
            return linear_modules(dtype) + [("attention_simt", None)] + ([("attention_mma", {"HD": self.hd})] if mma else []) + extra
        return linear_modules(dtype) + [("qk_rope_write", None)] + ops.attention_modules(dtype, self.hd)
