"""Python faces of the CUDA launchers in fellm_b200/csrc: they check devices, dtypes, shapes and
the sizes a kernel takes, pass raw pointers and the current stream, and turn a launcher's return
code into a KernelError.  There is no CPU path and no library fallback behind any of them.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .config.errors import KernelError
from .csrc import jit

_c_int, _c_ll, _c_f, _c_p = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p
_fns = {}


def _fn(module: str, name: str, argtypes, defines=None):
    # (the cache key is made without the jit's own key: that one reads the environment, and this
    # function runs once per kernel launch)
    key = (module, name, tuple(defines.items()) if defines else None)
    f = _fns.get(key)
    if f is None:
        lib = jit.load_module(module, defines)
        try:
            f = getattr(lib, name)
        except AttributeError:
            raise KernelError(f"kernel library {module} has no entry point {name}") from None
        f.argtypes = list(argtypes)
        f.restype = _c_int
        _fns[key] = f
    return f


try:
    _raw_stream = torch._C._cuda_getCurrentRawStream          # the handle without building a Stream object
except AttributeError:                                         # pragma: no cover
    _raw_stream = None


def _stream() -> int:
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


_launches = 0


def launch_count() -> int:
    """Launcher calls so far (each is one kernel launch of this package, or a refusal)."""
    return _launches


def _check(code: int, what: str):
    global _launches
    _launches += 1
    if code == 0:
        return
    if code == -1:
        raise KernelError(f"{what}: a size the kernel does not take")
    if code == -2:
        raise KernelError(f"{what}: bad arguments (null pointer or mismatched dtypes)")
    raise KernelError(f"{what}: CUDA error {code}")


def _dev(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("fellm_b200 kernels run on CUDA tensors only (there is no CPU path)")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _is_bf16(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise KernelError(f"dtype {t.dtype} is not one the kernels take (bfloat16 or float32)")


def _i32(t, name):
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")


# ------------------------------------------------------------------------------ elementwise

def embed_rows(tokens, table, out, status=None, scale: float = 1.0):
    """out[t, :] = float32(table[tokens[t], :]) * scale.  A token outside the table writes zeros and sets
    status to 1 (the host checks ids first; the kernel never reads out of bounds)."""
    _dev(tokens, table, out)
    _i32(tokens, "tokens")
    T, d = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous()
    assert table.shape[1] == d and tokens.numel() == T
    f = _fn("elementwise", "fellm_embed_rows", [_c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_p, _c_f, _c_p])
    _check(f(_p(tokens), _p(table), _is_bf16(table), _p(out), T, d, table.shape[0], _p(status), float(scale), _stream()),
           "embed_rows")
    return out


def add_row_vector(x, v):
    """x float32 [T, d] += v float32 [d], every row."""
    _dev(x, v)
    assert x.dtype == torch.float32 and v.dtype == torch.float32 and x.is_contiguous() and v.is_contiguous()
    T, d = x.shape
    assert v.numel() == d
    residual_written(x)
    f = _fn("elementwise", "fellm_add_row_vector", [_c_p, _c_p, _c_int, _c_int, _c_p])
    _check(f(_p(x), _p(v), T, d, _stream()), "add_row_vector")
    return x


def scale_softcap(z, scale: float = 1.0, cap=None):
    """z float32, in place: z * scale, then cap * tanh(. / cap) where a cap is given."""
    _dev(z)
    assert z.dtype == torch.float32 and z.is_contiguous()
    f = _fn("elementwise", "fellm_scale_softcap", [_c_p, ctypes.c_longlong, _c_f, _c_f, _c_p])
    _check(f(_p(z), z.numel(), float(scale), float(cap or 0.0), _stream()), "scale_softcap")
    return z


def rmsnorm(x, w, eps: float, out_dtype, rows=None, out=None):
    """x float32 [T, d], w float32 [d] -> [T or len(rows), d] in out_dtype."""
    _dev(x, w, rows)
    assert x.dtype == torch.float32 and w.dtype == torch.float32 and x.is_contiguous()
    d = x.shape[-1]
    assert w.numel() == d
    n = x.shape[0] if rows is None else rows.numel()
    if rows is not None:
        _i32(rows, "rows")
    if out is None:
        out = torch.empty((n, d), dtype=out_dtype, device=x.device)
    f = _fn("elementwise", "fellm_rmsnorm", [_c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_f, _c_p])
    _check(f(_p(x), _p(w), _p(out), _is_bf16(out), _p(rows), n, d, float(eps), _stream()), "rmsnorm")
    return out


# ------------------------------------------------------------------------------ norms on a sublayer's output

def layernorm(x, w, b, eps: float, out_dtype, rows=None, out=None):
    """x float32 [T, d] -> (x - mean) / sqrt(var + eps) * w + b, [T or len(rows), d] in out_dtype (var: the mean of the
    squared deviations; w, b float32 [d])."""
    _dev(x, w, b, rows)
    assert x.dtype == torch.float32 and w.dtype == torch.float32 and b.dtype == torch.float32 and x.is_contiguous()
    d = x.shape[-1]
    assert w.numel() == d and b.numel() == d
    n = x.shape[0] if rows is None else rows.numel()
    if rows is not None:
        _i32(rows, "rows")
    if out is None:
        out = torch.empty((n, d), dtype=out_dtype, device=x.device)
    f = _fn("sublayer", "fellm_layernorm", [_c_p, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_f, _c_p])
    _check(f(_p(x), _p(w), _p(b), _p(out), _is_bf16(out), _p(rows), n, d, float(eps), _stream()), "layernorm")
    return out


def add_layernorm(x, y, w, b, eps: float, cast=None):
    """x float32 [T, d] += LN(y) (y float32 [T, d], weight and bias float32 [d]).  cast [T, d] (bfloat16 or float32):
    also receives the new rows of x in its dtype."""
    _dev(x, y, w, b, cast)
    T, d = x.shape
    assert x.dtype == torch.float32 and y.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and y.shape == x.shape
    assert w.dtype == torch.float32 and b.dtype == torch.float32 and w.numel() == d and b.numel() == d
    if cast is not None:
        assert cast.is_contiguous() and cast.shape == x.shape
    residual_written(x)
    f = _fn("sublayer", "fellm_add_layernorm", [_c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_f, _c_p])
    _check(f(_p(x), _p(y), _p(w), _p(b), _p(cast), _is_bf16(cast) if cast is not None else 0, T, d, float(eps), _stream()),
           "add_layernorm")
    return x


def cast_rows(x, out_dtype, out=None):
    """float32 rows in the activation dtype (the tensor itself where that is float32)."""
    if out_dtype == torch.float32:
        return x
    _dev(x)
    assert x.dtype == torch.float32 and x.is_contiguous() and out_dtype == torch.bfloat16
    if out is None:
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    f = _fn("sublayer", "fellm_cast_rows", [_c_p, _c_p, _c_ll, _c_p])
    _check(f(_p(x), _p(out), x.numel(), _stream()), "cast_rows")
    return out


GLU_ACTS = {"silu": 0, "gelu_tanh": 1}


def act_mul(gu, act: str, out=None):
    """gu [T, >= 2F] (gate | up, row stride free) -> [T, F] = act(gate) * up; act 'silu' or 'gelu_tanh'
    (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))))."""
    _dev(gu)
    assert gu.stride(1) == 1 and gu.shape[1] % 2 == 0
    if act not in GLU_ACTS:
        raise KernelError(f"act_mul: unknown activation {act!r}")
    T, F = gu.shape[0], gu.shape[1] // 2
    if out is None:
        out = torch.empty((T, F), dtype=gu.dtype, device=gu.device)
    f = _fn("sublayer", "fellm_act_mul", [_c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_p(gu), gu.stride(0), _p(out), _is_bf16(gu), T, F, GLU_ACTS[act], _stream()), "act_mul")
    return out


def gate_mul(a, g):
    """a [T, N] *= sigmoid(g) in place, g [T, N] of a's dtype (row stride free)."""
    _dev(a, g)
    assert a.is_contiguous() and g.stride(1) == 1 and g.dtype == a.dtype and g.shape == a.shape
    f = _fn("sublayer", "fellm_gate_mul", [_c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_p(a), _p(g), g.stride(0), _is_bf16(a), a.shape[0], a.shape[1], _stream()), "gate_mul")
    return a


def relu2(z, out_dtype, out=None):
    """float32 z -> max(z, 0)^2 in out_dtype."""
    _dev(z)
    assert z.dtype == torch.float32 and z.is_contiguous()
    if out is None:
        out = torch.empty(z.shape, dtype=out_dtype, device=z.device)
    f = _fn("sublayer", "fellm_relu2", [_c_p, _c_p, _c_int, _c_ll, _c_p])
    _check(f(_p(z), _p(out), _is_bf16(out), z.numel(), _stream()), "relu2")
    return out


def silu_mul(gu, out=None):
    """gu [T, 2F] (gate | up) -> [T, F] = silu(gate) * up."""
    _dev(gu)
    assert gu.is_contiguous() and gu.shape[1] % 2 == 0
    T, F = gu.shape[0], gu.shape[1] // 2
    if out is None:
        out = torch.empty((T, F), dtype=gu.dtype, device=gu.device)
    f = _fn("elementwise", "fellm_silu_mul", [_c_p, _c_p, _c_int, _c_int, _c_int, _c_p])
    _check(f(_p(gu), _p(out), _is_bf16(gu), T, F, _stream()), "silu_mul")
    return out


def dyt_norm(x, w, b, alpha: float, out_dtype, rows=None, out=None):
    """Dynamic Tanh: x float32 [T, d] -> tanh(alpha x) * w + b, [T or len(rows), d] in out_dtype."""
    _dev(x, w, b, rows)
    assert x.dtype == torch.float32 and w.dtype == torch.float32 and b.dtype == torch.float32 and x.is_contiguous()
    d = x.shape[-1]
    assert w.numel() == d and b.numel() == d
    n = x.shape[0] if rows is None else rows.numel()
    if rows is not None:
        _i32(rows, "rows")
    if out is None:
        out = torch.empty((n, d), dtype=out_dtype, device=x.device)
    f = _fn("elementwise", "fellm_dyt_norm", [_c_p, _c_p, _c_p, _c_f, _c_p, _c_int, _c_p, _c_int, _c_int, _c_p])
    _check(f(_p(x), _p(w), _p(b), float(alpha), _p(out), _is_bf16(out), _p(rows), n, d, _stream()), "dyt_norm")
    return out


def concat_cast(a, b, out_dtype, out=None):
    """a, b float32 [T, d] -> [T, 2d] = [a | b] in out_dtype."""
    _dev(a, b)
    assert a.dtype == torch.float32 and b.dtype == torch.float32 and a.is_contiguous() and b.is_contiguous() and a.shape == b.shape
    T, d = a.shape
    if out is None:
        out = torch.empty((T, 2 * d), dtype=out_dtype, device=a.device)
    f = _fn("elementwise", "fellm_concat_cast", [_c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_p])
    _check(f(_p(a), _p(b), _p(out), _is_bf16(out), T, d, _stream()), "concat_cast")
    return out


def rmsnorm_groups(x, w, eps: float, groups: int, out_dtype, rows=None, out=None):
    """RMSNorm in `groups` equal consecutive parts of the row, each over its own root mean square, then the weight:
    x float32 [T, d], w float32 [d] -> [T or len(rows), d] in out_dtype."""
    _dev(x, w, rows)
    assert x.dtype == torch.float32 and w.dtype == torch.float32 and x.is_contiguous()
    d = x.shape[-1]
    assert w.numel() == d
    if groups < 1 or d % groups:
        raise KernelError(f"rmsnorm_groups: {groups} groups do not divide a row of {d}")
    n = x.shape[0] if rows is None else rows.numel()
    if rows is not None:
        _i32(rows, "rows")
    if out is None:
        out = torch.empty((n, d), dtype=out_dtype, device=x.device)
    f = _fn("elementwise", "fellm_rmsnorm_groups", [_c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_f, _c_p])
    _check(f(_p(x), _p(w), _p(out), _is_bf16(out), _p(rows), n, d, int(groups), float(eps), _stream()), "rmsnorm_groups")
    return out


def poly_norm(z, coef, eps: float, out_dtype, out=None):
    """z float32 [T, F] (columns of a wider matrix are fine), coef float32 [4] = (a, b, c, e) -> a N(z) + b N(z^2) + c N(z^3) + e in out_dtype, powers
    element by element, N = over the row's root mean square (eps under the root)."""
    _dev(z, coef)
    assert z.dtype == torch.float32 and z.stride(1) == 1 and coef.dtype == torch.float32 and coef.numel() == 4
    T, F = z.shape
    if out is None:
        out = torch.empty((T, F), dtype=out_dtype, device=z.device)
    f = _fn("elementwise", "fellm_poly_norm", [_c_p, _c_int, _c_p, _c_p, _c_int, _c_int, _c_int, _c_f, _c_p])
    _check(f(_p(z), max(z.stride(0), F), _p(coef), _p(out), _is_bf16(out), T, F, float(eps), _stream()), "poly_norm")
    return out


def gated_add(x, ys, zg):
    """x float32 [T, d] += sum over the sublayers s of ys[s] * sigmoid(zg[:, s * d : (s + 1) * d]); ys: one or two
    float32 [T, d]; zg float32 [T, >= len(ys) * d]: the gates' logits."""
    _dev(x, zg, *ys)
    T, d = x.shape
    assert 1 <= len(ys) <= 2 and x.dtype == torch.float32 and x.is_contiguous() and zg.dtype == torch.float32
    assert zg.stride(1) == 1 and zg.shape[1] >= len(ys) * d
    for y in ys:
        assert y.dtype == torch.float32 and y.is_contiguous() and y.shape == x.shape
    residual_written(x)
    f = _fn("elementwise", "fellm_gated_add", [_c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_p])
    _check(f(_p(x), _p(ys[0]), _p(ys[1]) if len(ys) > 1 else None, _p(zg), zg.stride(0), T, d, _stream()), "gated_add")
    return x


def token_side(x, tokens, table, offset: int, w_gate, w_proj, norm_w, eps: float, status=None, pending=None):
    """What a token adds to the stream by itself: e = table[token, offset : offset + m]; g = gelu_tanh(W_gate x) * e;
    y = W_proj g; x += y / sqrt(mean(y^2) + eps) * norm_w.  x float32 [T, d] in place; W_gate [m, d], W_proj [d, m],
    table [vocab, >= offset + m] of one dtype; float32 sums.  pending = (ys, zg): what gated_add(x, ys, zg) would add is
    added first (in the same launch where the kernel can), and the side input is computed from that sum."""
    _dev(x, tokens, table, w_gate, w_proj, norm_w)
    _i32(tokens, "tokens")
    T, d = x.shape
    m = w_gate.shape[0]
    assert x.dtype == torch.float32 and x.is_contiguous() and norm_w.dtype == torch.float32 and norm_w.numel() == d
    assert w_gate.shape == (m, d) and w_proj.shape == (d, m) and w_gate.is_contiguous() and w_proj.is_contiguous()
    assert table.dtype == w_gate.dtype == w_proj.dtype and table.stride(1) == 1 and 0 <= offset and offset + m <= table.shape[1]
    residual_written(x)
    if (TOKEN_SIDE_MMA and _is_bf16(w_gate) and d % 64 == 0 and 64 <= d <= 2048 and m % 16 == 0 and 16 <= m <= 512
            and w_gate.data_ptr() % 4 == 0 and w_proj.data_ptr() % 4 == 0):
        # bfloat16 tables: 16 rows a block on tensor cores
        f = _fn("elementwise", "fellm_token_side_mma", [_c_p, _c_p, _c_p, _c_p, _c_int, _c_p, _c_p, _c_int, _c_int, _c_int, _c_p, _c_p,
                                                        _c_p, _c_int, _c_int, _c_int, _c_f, _c_p, _c_p])
        y0 = y1 = zg = None
        if pending is not None:
            ys, zg = pending
            _dev(zg, *ys)
            assert 1 <= len(ys) <= 2 and zg.dtype == torch.float32 and zg.stride(1) == 1 and zg.shape[1] >= len(ys) * d
            for y in ys:
                assert y.dtype == torch.float32 and y.is_contiguous() and y.shape == x.shape
            y0, y1 = ys[0], (ys[1] if len(ys) > 1 else None)
        _check(f(_p(x), _p(y0), _p(y1), _p(zg), zg.stride(0) if zg is not None else 0, _p(tokens), _p(table), table.stride(0),
                 int(offset), table.shape[0], _p(w_gate), _p(w_proj), _p(norm_w), T, d, m, float(eps), _p(status), _stream()),
               "token_side (tensor cores)")
        return x
    if pending is not None:
        gated_add(x, pending[0], pending[1])
    f = _fn("elementwise", "fellm_token_side", [_c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_p, _c_p, _c_int, _c_p, _c_int, _c_int,
                                                _c_int, _c_f, _c_p, _c_p])
    _check(f(_p(x), _p(tokens), _p(table), table.stride(0), int(offset), table.shape[0], _p(w_gate), _p(w_proj), _is_bf16(w_gate),
             _p(norm_w), T, d, m, float(eps), _p(status), _stream()), "token_side")
    return x


def add_rows(x, y):
    """x float32 += y float32 of the same shape."""
    _dev(x, y)
    assert x.dtype == torch.float32 and y.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and x.shape == y.shape
    residual_written(x)
    f = _fn("elementwise", "fellm_add_rows", [_c_p, _c_p, _c_ll, _c_p])
    _check(f(_p(x), _p(y), x.numel(), _stream()), "add_rows")
    return x


# ------------------------------------------------------------------------------ matrix products

def gemm_simt(a, w, bias=None, out=None, out_dtype=None, accumulate=False):
    """out[M, N] = a[M, K] @ w[N, K]^T (+ bias[N]) with float32 FMA on CUDA cores; with
    accumulate=True, out (float32) += that.  Any mix of bfloat16/float32 a and w."""
    _dev(a, w, bias, out)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm: a is [{M},{K}] but w is {list(w.shape)}")
    assert a.stride(1) == 1 and w.stride(1) == 1
    if out is None:
        assert not accumulate
        out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
    assert out.stride(1) == 1 and out.shape == (M, N)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    if _is_bf16(out) and not _is_bf16(a):
        raise KernelError("gemm_simt: float32 activations do not round down to a bfloat16 result")
    if accumulate:
        residual_written(out)
    f = _fn("gemm_simt", "fellm_gemm_simt",
            [_c_p, _c_int, _c_p, _c_int, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_p])
    _check(f(_p(a), _is_bf16(a), _p(w), _is_bf16(w), _p(bias), _p(out), _is_bf16(out), M, N, K,
             a.stride(0), w.stride(0), out.stride(0), int(accumulate), _stream()), "gemm_simt")
    return out


def head_gemm(a, w, out, *, a_head: int, out_head: int):
    """One product per head in one launch: out[t, h * out_head + n] = sum_k a[t, h * a_head + k] w[h, n, k]
    for h < H, n < N, k < K (w [H, N, K] contiguous; a and out are row-major with the heads side by side in a row,
    a head's block starting every a_head / out_head columns and possibly wider than K / N).  All bfloat16, with
    blocks that start on 16 bytes: tensor cores (mma.sync tiles, float32 sums); else float32 FMA, any mix of
    bfloat16 / float32.  A row's result does not depend on the batch."""
    _dev(a, w, out)
    H, N, K = w.shape
    T = a.shape[0]
    assert w.is_contiguous() and a.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == T
    assert a.shape[1] >= (H - 1) * a_head + K and out.shape[1] >= (H - 1) * out_head + N
    if _is_bf16(out) and not _is_bf16(a):
        raise KernelError("head_gemm: float32 activations do not round down to a bfloat16 result")
    if (_is_bf16(a) and _is_bf16(w) and _is_bf16(out) and K % 8 == 0 and a_head % 8 == 0 and a.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and HEAD_GEMM_MMA):
        f = _fn("gemm_tiled", "fellm_gemm_tiled_batched", [_c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                                           _c_ll, _c_ll, _c_ll, _c_p])
        _check(f(_p(a), _p(w), _p(out), H, T, N, K, a.stride(0), K, out.stride(0), int(a_head), N * K, int(out_head), _stream()),
               "head_gemm (tensor cores)")
        return out
    f = _fn("gemm_simt", "fellm_gemm_simt_batched", [_c_p, _c_int, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                                     _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_p])
    _check(f(_p(a), _is_bf16(a), _p(w), _is_bf16(w), _p(out), _is_bf16(out), H, T, N, K, a.stride(0), K, out.stride(0),
             int(a_head), N * K, int(out_head), _stream()), "head_gemm")
    return out


TOKEN_SIDE_MMA = os.environ.get("FELLM_B200_TOKEN_SIDE_MMA", "1") != "0"
HEAD_GEMM_MMA = os.environ.get("FELLM_B200_HEAD_GEMM_MMA", "1") != "0"


# ------------------------------------------------------------------------------ short convolution

MAX_CONV_TAPS = 8


def shortconv(bcx, w, conv_bias, state, item_slot, item_start, row_item, n_items, all_single, out=None,
              blocked=False):
    """bcx [T, 3d] (B | C | X; blocked: [B16 | C16 | X16] per 16 channels, see block_bcx_rows), w
    float32 [d, Lc], state float32 [slots, Lc-1, d] (a view of one layer's slots; slot stride may
    be larger than (Lc-1)*d).  Returns y [T, d] = C * conv(B*X) and advances each item's state slot."""
    _dev(bcx, w, conv_bias, state, item_slot, item_start, row_item)
    T = bcx.shape[0]
    d, Lc = w.shape
    if not 2 <= Lc <= MAX_CONV_TAPS:
        raise KernelError(f"shortconv: conv_L_cache {Lc} is outside the kernel's range 2..{MAX_CONV_TAPS}")
    assert bcx.shape[1] == 3 * d and bcx.is_contiguous() and w.dtype == torch.float32 and w.is_contiguous()
    assert state.dtype == torch.float32 and state.shape[1:] == (Lc - 1, d)
    assert state.stride(1) == d and state.stride(2) == 1
    for t, nm in ((item_slot, "item_slot"), (item_start, "item_start"), (row_item, "row_item")):
        _i32(t, nm)
    if out is None:
        out = torch.empty((T, d), dtype=bcx.dtype, device=bcx.device)
    f = _fn("shortconv", "fellm_shortconv",
            [_c_p, _c_int, _c_p, _c_p, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_p])
    _check(f(_p(bcx), _is_bf16(bcx), _p(w), _p(conv_bias), _p(state), state.stride(0), _p(item_slot),
             _p(item_start), _p(row_item), _p(out), T, n_items, d, Lc, int(all_single), int(blocked), _stream()),
           "shortconv")
    return out


def block_bcx_rows(w):
    """Rows (or entries) [B | C | X] of a ShortConv input projection, d each, reordered into blocks
    of 16 channels: 16 B rows, 16 C rows, 16 X rows.  d must be a multiple of 16."""
    d = w.shape[0] // 3
    assert w.shape[0] == 3 * d and d % 16 == 0
    rest = w.shape[1:]
    return w.reshape(3, d // 16, 16, *rest).transpose(0, 1).reshape(3 * d, *rest).contiguous()


_conv_takes_cache = {}


def conv_product_takes(M: int, N: int, K: int, taps: int) -> bool:
    """Whether gemm_bf16_conv runs a product of these sizes: decode steps of up to 16 requests on the weight-streaming
    kernel (K of 1024..1280 in whole chunks), of 17..64 requests on the tcgen05 product of few rows (channels a multiple
    of 32, up to 4 taps; the kernel itself takes up to 128 rows)."""
    key = (M, N, K, taps)
    hit = _conv_takes_cache.get(key)
    if hit is None:
        if M <= 16:
            f = _fn("gemm_skinny", "fellm_gemm_skinny_conv_takes", [_c_int, _c_int, _c_int, _c_int])
            hit = bool(f(M, N, K, taps))
        else:
            f = _fn("gemm_umma", "fellm_gemm_umma_swap_conv_takes", [_c_int, _c_int, _c_int, _c_int])
            # measured on B200: a step of 32 rows at width 1024 0.629 -> 0.604 ms, of 64 rows 0.849 -> 0.842 ms, but at
            # width 2048 (64 rows) 1.298 -> 1.318 ms: tiles of 96 rows cost the wider product more than the launch saves;
            # at 96 and 128 rows the two ways lie within 2% of each other (width 1024: 1.061 / 1.065 and 1.283 / 1.271
            # ms; width 1536: 1.289 / 1.264 and 1.580 / 1.543 ms), so the kernel of its own stays there
            hit = bool(_swap_rows(M, N) and FUSE_SWAP_CONV and M <= SWAP_CONV_MAX_ROWS and K <= SWAP_CONV_MAX_K and f(M, N, K, taps))
        _conv_takes_cache[key] = hit
    return hit


def gemm_bf16_conv(x, w_blocked, bias, conv_w, conv_bias, state, row_slot, *, norm=None, out=None, row_scale=None):
    """A decode step's ShortConv input product and gated convolution in one launch: every row of x
    is one token of its own request (row_slot[i] = its state slot).  x bfloat16 [M, K], or with
    norm=(weight, eps) the float32 residual rows to be RMS-normed on the way in, or with
    row_scale=(ssq, parts, eps) the pre-weighted input of a handed-on norm; w_blocked [3d, K]
    and bias in block_bcx_rows order.  Returns y bfloat16 [M, d]; the states move on by one token."""
    _dev(x, w_blocked, bias, conv_w, conv_bias, state, row_slot)
    M, K = x.shape
    N = w_blocked.shape[0]
    d, taps = conv_w.shape
    assert N == 3 * d and w_blocked.dtype == torch.bfloat16 and w_blocked.stride(1) == 1 and x.stride(1) == 1
    assert conv_w.dtype == torch.float32 and conv_w.is_contiguous()
    assert state.dtype == torch.float32 and state.shape[1:] == (taps - 1, d) and state.stride(1) == d and state.stride(2) == 1
    _i32(row_slot, "row_slot")
    if out is None:
        out = torch.empty((M, d), dtype=torch.bfloat16, device=x.device)
    assert out.dtype == torch.bfloat16 and out.stride(1) == 1
    if M > 16:
        # 17..64 requests: the tcgen05 product of few rows, the convolution in its owners' epilogue
        if norm is not None or x.dtype != torch.bfloat16:
            raise KernelError("gemm_bf16_conv: more than 16 rows take bfloat16 rows (normed before, or a handed-on norm's)")
        if not conv_product_takes(M, N, K, taps):
            raise KernelError(f"gemm_bf16_conv does not take a product of {M} x {N} x {K} with {taps} taps")
        if row_scale is not None:
            _announce_row_scale(row_scale, M, N, K, own_plan=True)
        f = _fn("gemm_umma", "fellm_gemm_umma_swap_conv",
                [_c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_ll, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p])
        _check(f(_p(x), _p(w_blocked), _p(bias), _p(conv_w), _p(conv_bias), _p(state), state.stride(0), _p(row_slot), taps,
                 _p(out), M, N, K, x.stride(0), w_blocked.stride(0), out.stride(0), _p(umma_status(x.device)), _stream()),
               "gemm_umma_swap_conv")
        return out
    _announce_next("gemm_skinny", w_blocked, M)
    if row_scale is not None:
        assert norm is None
        _announce_row_scale(row_scale, M, N, K, own_plan=True)
    f = _fn("gemm_skinny", "fellm_gemm_skinny_conv",
            [_c_p, _c_p, _c_p, _c_f, _c_p, _c_p, _c_p, _c_p, _c_p, _c_ll, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_p])
    if norm is not None:
        assert x.dtype == torch.float32 and norm[0].dtype == torch.float32
        code = f(None, _p(x), _p(norm[0]), float(norm[1]), _p(w_blocked), _p(bias), _p(conv_w), _p(conv_bias), _p(state),
                 state.stride(0), _p(row_slot), taps, _p(out), M, N, K, x.stride(0), w_blocked.stride(0), out.stride(0),
                 _stream())
    else:
        assert x.dtype == torch.bfloat16
        code = f(_p(x), None, None, 0.0, _p(w_blocked), _p(bias), _p(conv_w), _p(conv_bias), _p(state),
                 state.stride(0), _p(row_slot), taps, _p(out), M, N, K, x.stride(0), w_blocked.stride(0), out.stride(0),
                 _stream())
    _check(code, "gemm_skinny_conv")
    return out


# ------------------------------------------------------------------------------ recurrent mixers

MAX_SCAN_KEY_DIM = 1024          # 32 lanes x 32 rows of a column


def _state_args(state):
    assert state.dtype == torch.float32 and state[0].is_contiguous()
    return _p(state), state.stride(0)


def causal_conv_act(x, taps, state, item_start, item_slot, n_items, max_item_rows, act="silu", out=None):
    """x [T, C] (row stride free) -> act(causal conv over time per channel), taps float32 [C, L] (last column: the
    current token); state float32 [slots, L-1, C]: the inputs before each portion, moved on by the call.
    max_item_rows: the longest portion of the step (the grid covers that many rows of every item)."""
    _dev(x, taps, state, item_start, item_slot)
    T, C = x.shape
    L = taps.shape[1]
    if not 1 <= L <= MAX_CONV_TAPS:
        raise KernelError(f"causal_conv_act: {L} taps are outside the kernel's range 1..{MAX_CONV_TAPS}")
    assert x.stride(1) == 1 and taps.dtype == torch.float32 and taps.is_contiguous() and taps.shape[0] == C
    assert state.shape[1:] == (max(L - 1, 0), C) or L == 1
    _i32(item_start, "item_start"), _i32(item_slot, "item_slot")
    if out is None:
        out = torch.empty((T, C), dtype=x.dtype, device=x.device)
    sp, ss = _state_args(state)
    f = _fn("recurrent", "fellm_causal_conv_act",
            [_c_p, _c_int, _c_int, _c_p, _c_int, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_p(x), _is_bf16(x), x.stride(0), _p(taps), L, sp, ss, _p(item_start), _p(item_slot), _p(out), out.stride(0),
             n_items, C, {"none": 0, "silu": 1}[act], int(max_item_rows), _stream()), "causal_conv_act")
    return out


def token_shift_mix(h, mu, state, item_start, item_slot, n_items, max_item_rows, out=None):
    """h [T, d], mu float32 [S, d] -> [S, T, d]: h + (h_prev - h) * mu_s, h_prev the row before (the slot's state
    float32 [slots, d] before a portion's first row; the state then takes the portion's last row)."""
    _dev(h, mu, state, item_start, item_slot)
    T, d = h.shape
    S = mu.shape[0]
    assert h.is_contiguous() and mu.dtype == torch.float32 and mu.is_contiguous() and mu.shape[1] == d
    assert state.shape[1:] == (d,)
    _i32(item_start, "item_start"), _i32(item_slot, "item_slot")
    if out is None:
        out = torch.empty((S, T, d), dtype=h.dtype, device=h.device)
    sp, ss = _state_args(state)
    f = _fn("recurrent", "fellm_token_shift_mix",
            [_c_p, _c_int, _c_p, _c_int, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_p(h), _is_bf16(h), _p(mu), S, sp, ss, _p(item_start), _p(item_slot), _p(out), T, n_items, d,
             int(max_item_rows), _stream()), "token_shift_mix")
    return out


def token_shift(x, mu, state, item_start, item_slot, n_items, max_item_rows, out_dtype, out=None, row_item=None):
    """x float32 [T, d] -> x + (x_prev - x) * mu in out_dtype, x_prev the row before (the slot's float32 state [slots, d]
    before a portion's first row; the state then takes the portion's last row of x as it is).  row_item int32 [T] (each
    row's item): lets widths of a multiple of 4 run with 16-byte loads, a thread four channels of a row."""
    _dev(x, mu, state, item_start, item_slot, row_item)
    if row_item is not None:
        _i32(row_item, "row_item")
        assert row_item.numel() >= x.shape[0]
    T, d = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and mu.dtype == torch.float32 and mu.numel() == d and mu.is_contiguous()
    assert state.shape[1:] == (d,)
    _i32(item_start, "item_start"), _i32(item_slot, "item_slot")
    if out is None:
        out = torch.empty((T, d), dtype=out_dtype, device=x.device)
    sp, ss = _state_args(state)
    f = _fn("recurrent", "fellm_token_shift", [_c_p, _c_p, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_p(x), _p(mu), sp, ss, _p(item_start), _p(item_slot), _p(row_item), _p(out), _is_bf16(out), T, n_items, d,
             int(max_item_rows), _stream()), "token_shift")
    return out


GATED_WRITE_BLOCK = int(os.environ.get("FELLM_B200_GATED_WRITE_BLOCK", 0))            # tokens of a block (0, the default: the plain scan; measured no faster)
GATED_WRITE_BLOCK_MIN_ROWS = int(os.environ.get("FELLM_B200_GATED_WRITE_BLOCK_MIN_ROWS", 256))     # shorter portions: the plain scan
GATED_WRITE_PREP_MIN_ROWS = int(os.environ.get("FELLM_B200_GATED_WRITE_PREP_MIN_ROWS", 16))       # a step's longest portion from which the gates are prepared in front


def gated_write_scan(z, f_off, v_off, lower, bias, state, item_start, item_slot, n_items, H, dk, dv, out=None,
                     max_item_rows=0, block=None, prepared=None):
    """Per head S = diag(f) S + (1 - f) v^T, o = S^T q, with q = SiLU(q raw) and f = lower + (1 - lower) sigmoid(f raw +
    bias).  z float32 [T, >= v_off + H*dv]: q raw at column 0 (H x dk), f raw at f_off, v at v_off (H x dv); lower, bias
    float32 [H*dk]; state float32 [slots, H, dk, dv] (the scan kernel's own layout).  Returns float32 [T, H*dv].
    block (default: GATED_WRITE_BLOCK where the step's longest portion has GATED_WRITE_BLOCK_MIN_ROWS rows or more, else 0):
    the portions run in blocks of that many tokens side by side, every block twice (from zeros, then from the state in
    front of it), a walk over the blocks' states between the two; equal to the plain scan up to float32 rounding.
    prepared (default: where the longest portion has GATED_WRITE_PREP_MIN_ROWS rows or more): a kernel in front computes the
    gates once a token and head IN PLACE (z's q and f columns then hold f q and f) and the scan's producers only copy;
    the same numbers as the one-launch form, which single tokens keep."""
    _dev(z, lower, bias, state, item_start, item_slot)
    T = z.shape[0]
    if dk > MAX_SCAN_KEY_DIM:
        raise KernelError(f"gated_write_scan: key size {dk} is above the kernel's {MAX_SCAN_KEY_DIM}")
    assert z.dtype == torch.float32 and z.stride(1) == 1 and z.shape[1] >= v_off + H * dv
    for v in (lower, bias):
        assert v.dtype == torch.float32 and v.numel() == H * dk and v.is_contiguous()
    assert state.shape[1:] == (H, dk, dv)
    _i32(item_start, "item_start"), _i32(item_slot, "item_slot")
    if out is None:
        out = torch.empty((T, H * dv), dtype=torch.float32, device=z.device)
    sp, ss = _state_args(state)
    if block is None:
        block = GATED_WRITE_BLOCK if max_item_rows >= max(GATED_WRITE_BLOCK_MIN_ROWS, 2) else 0
    scratch = None
    if block and max_item_rows > block:
        scratch = torch.empty(n_items * (-(-max_item_rows // block)) * H * (dk * dv + dk), dtype=torch.float32, device=z.device)
    if prepared is None:
        prepared = max_item_rows >= GATED_WRITE_PREP_MIN_ROWS
    prep = torch.empty((T, H), dtype=torch.float32, device=z.device) if prepared else None
    f = _fn("recurrent", "fellm_gated_write_scan",
            [_c_p, _c_int, _c_int, _c_int, _c_p, _c_p, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_p, _c_p, _c_int, _c_p])
    _check(f(_p(z), z.stride(0), int(f_off), int(v_off), _p(lower), _p(bias), sp, ss, _p(item_start), _p(item_slot), _p(out),
             n_items, H, dk, dv, int(max_item_rows), int(block or 0), _p(scratch), _p(prep), T, _stream()), "gated_write_scan")
    return out


_LR_IN = {"none": 0, "tanh": 1}
_LR_OUT = {"none": 0, "exp_neg_exp": 1, "decay_softplus": 2}


def lowrank_expand(z, w2, bias=None, *, f_in="none", f_out="none", rate=None, per=1, out=None):
    """out[t, n] = f_out(bias[n] + sum_r w2[n, r] f_in(z[t, r])) in float32.  z float32 [T, R] (row stride free),
    w2 [N, R] bfloat16 or float32.  f_out 'exp_neg_exp': exp(-exp(v)); 'decay_softplus': exp(-exp(rate[n // per]) *
    softplus(v))."""
    _dev(z, w2, bias, rate)
    T, R = z.shape
    N = w2.shape[0]
    assert z.dtype == torch.float32 and z.stride(1) == 1 and w2.is_contiguous() and w2.shape[1] == R
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    if rate is not None:
        assert rate.dtype == torch.float32 and rate.numel() * per == N
    if out is None:
        out = torch.empty((T, N), dtype=torch.float32, device=z.device)
    f = _fn("recurrent", "fellm_lowrank_expand",
            [_c_p, _c_int, _c_p, _c_int, _c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_p(z), z.stride(0), _p(w2), _is_bf16(w2), _p(bias), _p(rate), int(per), _p(out), T, N, R, _LR_IN[f_in],
             _LR_OUT[f_out], _stream()), "lowrank_expand")
    return out


def delta_scan(qkv, k_off, v_off, small, b_off, a_off, A_log, dt_bias, gch, state, item_start, item_slot, n_items,
               H, G, dk, dv, out=None, max_item_rows=0):
    """The gated delta rule over the step's portions.  qkv [T, *]: q (G x dk) at column 0, k at k_off, v (H x dv) at
    v_off, after convolution and SiLU; small float32 [T, *]: beta's logit at b_off + h and, for a decay per head,
    its logit at a_off + h (A_log, dt_bias [H]); gch float32 [T, H*dk]: the decay per head and key channel itself
    (then A_log and dt_bias are not read).  state float32 [slots, H, dk, dv] (the kernel's own: it keeps each
    head's matrix column by column there).  Returns o float32 [T, H*dv].
    max_item_rows: the longest portion of the step, if known (sizes the staging buffers; no result depends on it)."""
    _dev(qkv, small, A_log, dt_bias, gch, state, item_start, item_slot)
    T = qkv.shape[0]
    if dk > MAX_SCAN_KEY_DIM:
        raise KernelError(f"delta_scan: key size {dk} is above the kernel's {MAX_SCAN_KEY_DIM}")
    assert qkv.stride(1) == 1 and small.dtype == torch.float32 and small.stride(1) == 1
    assert state.shape[1:] == (H, dk, dv)
    if gch is not None:
        assert gch.dtype == torch.float32 and gch.is_contiguous() and gch.shape == (T, H * dk)
    if out is None:
        out = torch.empty((T, H * dv), dtype=torch.float32, device=qkv.device)
    sp, ss = _state_args(state)
    f = _fn("recurrent", "fellm_delta_scan",
            [_c_p, _c_int, _c_int, _c_int, _c_int, _c_p, _c_int, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_ll, _c_p, _c_p,
             _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_p(qkv), _is_bf16(qkv), qkv.stride(0), k_off, v_off, _p(small), small.stride(0), b_off, a_off, _p(A_log),
             _p(dt_bias), _p(gch), sp, ss, _p(item_start), _p(item_slot), _p(out), n_items, H, G, dk, dv,
             int(max_item_rows), _stream()),
           "delta_scan")
    return out


def decay_bonus_scan(r, k, v, w, u, state, item_start, item_slot, n_items, H, dk, out=None, max_item_rows=0):
    """o_t = (S + diag(u) k_t v_t^T)^T r_t; S = diag(w_t) S + k_t v_t^T per head.  r, k, v [T, H*dk] (one row stride),
    w float32 [T, H*dk], u float32 [H, dk], state float32 [slots, H, dk, dk].  Returns o float32 [T, H*dk]."""
    _dev(r, k, v, w, u, state, item_start, item_slot)
    T = r.shape[0]
    if dk > MAX_SCAN_KEY_DIM:
        raise KernelError(f"decay_bonus_scan: key size {dk} is above the kernel's {MAX_SCAN_KEY_DIM}")
    assert r.dtype == k.dtype == v.dtype and r.stride(0) == k.stride(0) == v.stride(0) and r.stride(1) == 1
    assert w.dtype == torch.float32 and w.is_contiguous() and u.dtype == torch.float32 and u.is_contiguous()
    assert state.shape[1:] == (H, dk, dk)
    if out is None:
        out = torch.empty((T, H * dk), dtype=torch.float32, device=r.device)
    sp, ss = _state_args(state)
    f = _fn("recurrent", "fellm_decay_bonus_scan",
            [_c_p, _c_p, _c_p, _c_int, _c_int, _c_p, _c_p, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_p(r), _p(k), _p(v), _is_bf16(r), r.stride(0), _p(w), _p(u), sp, ss, _p(item_start), _p(item_slot), _p(out),
             n_items, H, dk, int(max_item_rows), _stream()), "decay_bonus_scan")
    return out


def retention_scan(qkv, k_off, v_off, positions, inv_freq, rot_dim, decay, kscale, state, item_start, item_slot, n_items,
                   H, dk, dv, out=None, max_item_rows=0):
    """Retention over portions: per head S = decay[h] S + k v^T, o = S^T q, with q and k rotated by position (the first
    rot_dim elements of a head, element i paired with i + rot_dim/2, inv_freq float32 [rot_dim/2]) and k times kscale
    after the rotation.  qkv [T, >= v_off + H*dv]: q at column 0 (H x dk), k at k_off, v at v_off (H x dv).
    state float32 [slots, ..., H, dk, dv] (a slot's states lie slot_stride apart).  Returns float32 [T, H*dv]."""
    _dev(qkv, positions, inv_freq, decay, state, item_start, item_slot)
    T = qkv.shape[0]
    assert qkv.stride(1) == 1 and decay.dtype == torch.float32 and decay.numel() == H and decay.is_contiguous()
    assert rot_dim % 2 == 0 and 0 <= rot_dim <= dk
    if rot_dim:
        assert inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dim // 2 and inv_freq.is_contiguous()
    _i32(positions, "positions"), _i32(item_start, "item_start"), _i32(item_slot, "item_slot")
    if dk > MAX_SCAN_KEY_DIM:
        raise KernelError(f"retention_scan: key size {dk} is above {MAX_SCAN_KEY_DIM}")
    if out is None:
        out = torch.empty((T, H * dv), dtype=torch.float32, device=qkv.device)
    st, stride = _state_args(state)
    f = _fn("recurrent", "fellm_retention_scan",
            [_c_p, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p, _c_int, _c_p, _c_f, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_int,
             _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_p(qkv), _is_bf16(qkv), qkv.stride(0), k_off, v_off, _p(positions), _p(inv_freq) if rot_dim else None,
             rot_dim, _p(decay), float(kscale), st, stride, _p(item_start), _p(item_slot), _p(out), n_items, H, dk, dv,
             int(max_item_rows), _stream()), "retention_scan")
    return out


RETENTION_CHUNKED = os.environ.get("FELLM_B200_RETENTION_CHUNKED", "1") != "0"
RETENTION_CHUNK_MIN_ROWS = int(os.environ.get("FELLM_B200_RETENTION_CHUNK_MIN_ROWS", 128))     # shorter portions: the scan (0.25 us a token)


def retention_chunked(p, k_off, v_off, positions, inv_freq, rot_dim, decay, kscale, state, item_start, item_slot, n_items,
                      max_item_rows, H, dk, dv, out=None):
    """Retention over portions in blocks of 64 tokens (float32 arithmetic; the blocks of a prompt run side by side and
    only the states in front of the blocks are walked in order).  Arguments as retention_scan's, p float32; the sums run
    in another order than the scan's (equal up to float32 rounding)."""
    _dev(p, positions, inv_freq, decay, state, item_start, item_slot)
    T = p.shape[0]
    assert p.dtype == torch.float32 and p.stride(1) == 1 and decay.dtype == torch.float32 and decay.numel() == H
    assert rot_dim % 2 == 0 and 0 <= rot_dim <= dk
    if rot_dim:
        assert inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dim // 2 and inv_freq.is_contiguous()
    _i32(positions, "positions"), _i32(item_start, "item_start"), _i32(item_slot, "item_slot")
    if out is None:
        out = torch.empty((T, H * dv), dtype=torch.float32, device=p.device)
    blocks = -(-max_item_rows // 64)
    scratch = torch.empty(2 * T * H * dk + n_items * blocks * H * dk * dv, dtype=torch.float32, device=p.device)
    st, stride = _state_args(state)
    f = _fn("retention_chunk", "fellm_retention_chunked",
            [_c_p, _c_int, _c_int, _c_int, _c_p, _c_p, _c_int, _c_p, _c_f, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_p(p), p.stride(0), k_off, v_off, _p(positions), _p(inv_freq) if rot_dim else None, rot_dim, _p(decay),
             float(kscale), st, stride, _p(item_start), _p(item_slot), _p(out), _p(scratch), T, n_items, int(max_item_rows),
             H, dk, dv, _stream()), "retention_chunked")
    return out


_GATE_ACT = {None: 0, "silu": 1, "sigmoid": 2}


def head_norm_gate(o, w, per_head: bool, gate, gate_act, eps: float, H: int, dv: int, out_dtype, out=None):
    """o float32 [T, H*dv] -> per head o / rms(o) * w * act(gate) in out_dtype.  w float32 [dv] (shared by the heads) or
    [H*dv] (per_head); gate [T, H*dv] (row stride free), any engine dtype; gate_act 'silu' | 'sigmoid' | None."""
    _dev(o, w, gate)
    T = o.shape[0]
    assert o.dtype == torch.float32 and o.is_contiguous()
    if w is not None:                    # None: the unit norm alone
        assert w.dtype == torch.float32 and w.numel() == (H * dv if per_head else dv)
    if gate_act is not None:
        assert gate is not None and gate.stride(1) == 1 and gate.shape == (T, H * dv)
    if out is None:
        out = torch.empty((T, H * dv), dtype=out_dtype, device=o.device)
    f = _fn("recurrent", "fellm_head_norm_gate",
            [_c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int, _c_f, _c_p])
    _check(f(_p(o), _p(w), int(per_head), _p(gate), _is_bf16(gate) if gate is not None else 0,
             gate.stride(0) if gate is not None else 0, _GATE_ACT[gate_act], _p(out), _is_bf16(out), T, H, dv, float(eps),
             _stream()), "head_norm_gate")
    return out


def branch_combine(x, branches, weights, eps: float):
    """x float32 [T, d] += mean over b of branches[b] / rms(branches[b]) * weights[b] (all float32)."""
    _dev(x, *branches, *weights)
    T, d = x.shape
    n = len(branches)
    for o, w in zip(branches, weights):
        assert o.dtype == torch.float32 and o.is_contiguous() and o.shape == (T, d) and w.dtype == torch.float32 and w.numel() == d
    residual_written(x)
    arr = ctypes.c_void_p * n
    f = _fn("recurrent", "fellm_branch_combine", [_c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_f, _c_p])
    _check(f(arr(*[o.data_ptr() for o in branches]), arr(*[w.data_ptr() for w in weights]), n, _p(x), T, d, float(eps),
             _stream()), "branch_combine")
    return x



# ------------------------------------------------------------------------------ routed experts

MOE_ROW_TILE = 64            # rows of a tile of the grouped products on CUDA cores and mma.sync
MOE_UMMA_ROW_TILE = 128      # ... of the tcgen05 grouped product
MOE_PLAN_TILE = 1024
MOE_MAX_TOP = 16
MOE_MMA = os.environ.get("FELLM_B200_MOE_MMA", "1") != "0"
MOE_UMMA = os.environ.get("FELLM_B200_MOE_UMMA", "1") != "0"
MOE_UMMA_MIN_PAIRS = int(os.environ.get("FELLM_B200_MOE_UMMA_MIN_PAIRS", 256))     # fewer (token, choice) pairs: mma.sync tiles of 64 rows
MOE_FEW_PAIRS = int(os.environ.get("FELLM_B200_MOE_FEW_PAIRS", 64))                # up to this many: a warp a column (weight streaming)


def moe_route(logits, E: int, top: int, renormalize: bool = False):
    """logits float32 [T, >= E] -> (idx int32 [T, top], w float32 [T, top]): the `top` experts with the largest
    softmax scores over all E (ties: the lower expert) and those scores as they are, or renormalised to sum 1."""
    _dev(logits)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    if not 1 <= top <= min(E, MOE_MAX_TOP):
        raise KernelError(f"moe_route: top {top} must be in 1..{min(E, MOE_MAX_TOP)}")
    T = logits.shape[0]
    idx = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    f = _fn("moe", "fellm_moe_route", [_c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p, _c_p])
    _check(f(_p(logits), logits.stride(0), T, E, top, int(renormalize), _p(idx), _p(w), _stream()), "moe_route")
    return idx, w


def moe_router(h, w_router, top: int, renormalize: bool = False, *, score: str = "softmax", correction=None,
               groups=None, bias=None):
    """The router's product and the routing in one launch: z = h W_router^T in float32 (h [T, K] and W_router [E, K]
    bfloat16 or float32), then as moe_route.  score = "sigmoid": the scores are sigmoid(z); the choice looks at
    score + correction (float32 [E]) and, with groups = (count, keep, best), only inside the `keep` of `count` equal
    groups of neighbouring experts whose `best` largest choice scores sum highest; the weights are the plain scores
    (renormalize: over their sum + 1e-20).  bias float32 [E]: added to z first.  Softmax scores renormalised over the
    chosen are the softmax over the chosen logits alone.  Returns (idx int32 [T, top], w float32 [T, top])."""
    _dev(h, w_router, correction, bias)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == w_router.shape[0] and bias.is_contiguous()
    assert h.stride(1) == 1 and w_router.is_contiguous() and h.shape[1] == w_router.shape[1]
    T, K = h.shape
    E = w_router.shape[0]
    if not 1 <= top <= min(E, MOE_MAX_TOP):
        raise KernelError(f"moe_router: top {top} must be in 1..{min(E, MOE_MAX_TOP)}")
    if score not in ("softmax", "sigmoid"):
        raise KernelError(f"moe_router: unknown score {score!r}")
    if score == "softmax" and (correction is not None or groups):
        raise KernelError("moe_router: a correction and groups go with sigmoid scores")
    n_groups, keep, best = groups if groups else (1, 1, 1)
    if correction is not None:
        assert correction.dtype == torch.float32 and correction.numel() == E and correction.is_contiguous()
    idx = torch.empty((T, top), dtype=torch.int32, device=h.device)
    w = torch.empty((T, top), dtype=torch.float32, device=h.device)
    f = _fn("moe", "fellm_moe_router", [_c_p, _c_int, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p,
                                        _c_int, _c_p, _c_int, _c_int, _c_int, _c_p, _c_p])
    _check(f(_p(h), _is_bf16(h), h.stride(0), _p(w_router), _is_bf16(w_router), T, K, E, top, int(renormalize), _p(idx),
             _p(w), int(score == "sigmoid"), _p(correction), int(n_groups), int(keep), int(best), _p(bias), _stream()),
           "moe_router")
    return idx, w


class MoePlan:
    """The (token, choice) pairs of a step sorted by expert: sorted[place] = pair, place_of[pair] = place, and the
    table of row tiles (expert, first row, rows <= row_tile) with their count on the device; max_tiles bounds it on
    the host."""
    __slots__ = ("sorted", "place_of", "table", "n_tiles", "max_tiles", "pairs", "top", "row_tile")


def moe_row_tile(pairs: int, bf16: bool, K_ok: bool) -> int:
    """Rows of a tile for a step of this many pairs: 128 where the tcgen05 grouped product takes the step."""
    return MOE_UMMA_ROW_TILE if (bf16 and K_ok and MOE_UMMA and USE_UMMA and pairs >= MOE_UMMA_MIN_PAIRS) else MOE_ROW_TILE


def moe_plan(idx, E: int, row_tile: int = MOE_ROW_TILE) -> MoePlan:
    _dev(idx)
    _i32(idx, "idx")
    assert idx.is_contiguous()
    T, top = idx.shape
    P = T * top
    tiles = -(-P // MOE_PLAN_TILE)
    plan = MoePlan()
    plan.pairs, plan.top, plan.row_tile = P, top, row_tile
    plan.max_tiles = min(P, E) + P // row_tile
    ints = torch.empty(2 * tiles * E + P + 2 * P + 3 * plan.max_tiles + 1, dtype=torch.int32, device=idx.device)
    at = 2 * tiles * E + P
    scratch = ints[:at]
    plan.sorted, plan.place_of = ints[at:at + P], ints[at + P:at + 2 * P]
    plan.table = ints[at + 2 * P:at + 2 * P + 3 * plan.max_tiles]
    plan.n_tiles = ints[at + 2 * P + 3 * plan.max_tiles:]
    f = _fn("moe", "fellm_moe_plan", [_c_p, _c_int, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p])
    _check(f(_p(idx), P, E, row_tile, _p(scratch), _p(plan.sorted), _p(plan.place_of), _p(plan.table),
             _p(plan.n_tiles), _stream()), "moe_plan")
    return plan


def moe_gemm(a, w, plan: MoePlan, *, gated: bool, gather: bool, interleaved: bool = False, act=None):
    """Grouped product over a plan's row tiles.  w [E, (2 if gated else 1) * N, K]; gather: row r of the result
    reads a[token of the pair sorted r] (a [T, K]); else a [P, K] is in sorted order.  gated: SiLU(gate) * up in
    a's dtype (w's rows: gate rows then up rows, or, interleaved, blocks of 8 gate and 8 up rows by turns); else
    float32.  act = (limit, alpha): the gated activation is the clamped form min(g, limit) sigmoid(alpha min(g, limit))
    (clamp(u, -limit, limit) + 1) instead.  Returns [P, N] in sorted order.
    bfloat16: tcgen05 (tiles of 128 rows, the plan made for them), a warp a column for a handful of pairs, mma.sync
    tiles of 64 rows between; float32, or sizes those do not take: float32 FMA."""
    _dev(a, w)
    assert a.stride(1) == 1 and w.is_contiguous() and a.dtype == w.dtype
    E, n_rows, K = w.shape
    N = n_rows // 2 if gated else n_rows
    assert a.shape[1] == K
    P = plan.pairs
    out = torch.empty((P, N), dtype=a.dtype if gated else torch.float32, device=a.device)
    act_limit, act_alpha = (float(act[0]), float(act[1])) if act else (0.0, 1.0)
    if act and not act_limit > 0.0:
        raise KernelError("moe_gemm: the clamped activation needs a positive limit")
    bf = a.dtype == torch.bfloat16
    if (bf and plan.row_tile == MOE_UMMA_ROW_TILE and K % 8 == 0 and (not gated or (interleaved and N % 8 == 0))
            and w.data_ptr() % 16 == 0):
        if gather:
            rows = torch.empty((P, K), dtype=a.dtype, device=a.device)
            f = _fn("moe", "fellm_moe_gather", [_c_p, _c_int, _c_p, _c_int, _c_p, _c_int, _c_int, _c_p])
            _check(f(_p(a), a.stride(0), _p(plan.sorted), plan.top, _p(rows), P, K, _stream()), "moe_gather")
            a = rows
        assert a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
        f = _fn("gemm_umma", "fellm_gemm_umma_grouped", [_c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                                         _c_p, _c_p, _c_int, _c_p, _c_f, _c_f, _c_p])
        _check(f(_p(a), _p(w), _p(out), _EPI_SWIGLU if gated else _EPI_F32, P, n_rows, K, E, a.stride(0), out.stride(0),
                 _p(plan.table), _p(plan.n_tiles), plan.max_tiles, _p(umma_status(a.device)), act_limit, act_alpha, _stream()),
               "gemm_umma_grouped")
        return out
    if plan.row_tile != MOE_ROW_TILE:
        raise KernelError(f"moe_gemm: a plan of {plan.row_tile}-row tiles needs the tcgen05 grouped product (bfloat16, K % 8 == 0)")
    f = _fn("moe", "fellm_moe_gemm", [_c_p, _c_int, _c_int, _c_p, _c_int, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int,
                                      _c_int, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_f, _c_f, _c_p])
    _check(f(_p(a), _is_bf16(a), a.stride(0), _p(plan.sorted) if gather else None, plan.top, _p(w), _is_bf16(w), _p(out),
             _is_bf16(out), N, N, K, int(gated), _p(plan.table), _p(plan.n_tiles), plan.max_tiles, int(MOE_MMA),
             int(interleaved), int(P <= MOE_FEW_PAIRS), act_limit, act_alpha, _stream()), "moe_gemm")
    return out


def moe_combine(x, y, plan: MoePlan, w, store: bool = False):
    """x float32 [T, d] += sum over a token's choices c, in order, of w[t, c] * y[place of (t, c)] (store: x = the sum)."""
    _dev(x, y, w)
    T, d = x.shape
    assert x.dtype == torch.float32 and y.dtype == torch.float32 and w.dtype == torch.float32
    assert x.is_contiguous() and y.is_contiguous() and w.is_contiguous() and y.shape == (plan.pairs, d)
    residual_written(x)
    f = _fn("moe", "fellm_moe_combine", [_c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_p(x), _p(y), _p(plan.place_of), _p(w), T, plan.top, d, int(store), _stream()), "moe_combine")
    return x


# ------------------------------------------------------------------------------ attention

PAIRINGS = {"adjacent": 0, "split_half": 1}


def qk_rope_write(qkv, q_w, k_w, eps, inv_freq, pairing, positions, row_slot, block_table, pool, layer,
                  page_tokens, H, G, hd, write_kv=True, status=None, q_out=None, rot_dim=None):
    """qkv [T, (H+2G)*hd] -> q_out [T, H, hd] (per-head RMSNorm, rotary), and k (normed, rotated)
    and v written to pool[page, layer, 0/1, g, slot, :].  q_w/k_w None: no QK norm; inv_freq None:
    no rotation; rot_dim (default hd): the first rot_dim elements of a head are rotated, with
    inv_freq [rot_dim/2].  pool: [pages, layers, 2, G, page_tokens, hd]; block_table [slots, width] is indexed
    by row_slot[t], the slot of the request row t belongs to."""
    _dev(qkv, q_w, k_w, inv_freq, positions, row_slot, block_table, pool)
    T = qkv.shape[0]
    if hd % 2:
        raise KernelError(f"attention: head_dim {hd} must be even")
    assert qkv.is_contiguous() and qkv.shape[1] == (H + 2 * G) * hd
    if write_kv:
        assert pool.is_contiguous() and pool.dtype == qkv.dtype
        assert pool.shape[2:] == (2, G, page_tokens, hd), (pool.shape, G, page_tokens, hd)
        _i32(block_table, "block_table")
    _i32(positions, "positions"), _i32(row_slot, "row_slot")
    if q_out is None:
        q_out = torch.empty((T, H, hd), dtype=qkv.dtype, device=qkv.device)
    rot_dim = hd if rot_dim is None else int(rot_dim)
    if inv_freq is not None:
        if rot_dim % 2 or not 2 <= rot_dim <= hd:
            raise KernelError(f"rotary dimension {rot_dim} must be even and within the head size {hd}")
        if inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dim // 2:
            raise KernelError(f"inv_freq must hold {rot_dim // 2} float32 values, got {inv_freq.numel()}")
    f = _fn("qk_rope_write", "fellm_qk_rope_write",
            [_c_p, _c_int, _c_p, _c_p, _c_f, _c_p, _c_int, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_int,
             _c_int, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p])
    _check(f(_p(qkv), _is_bf16(qkv), _p(q_w), _p(k_w), float(eps), _p(inv_freq), PAIRINGS[pairing],
             _p(positions), _p(row_slot), _p(block_table) if write_kv else None,
             block_table.shape[1] if write_kv else 0, _p(pool) if write_kv else None,
             _is_bf16(pool) if write_kv else _is_bf16(qkv), layer, pool.shape[1] if write_kv else 1,
             page_tokens, _p(q_out), T, H, G, hd, rot_dim, int(write_kv), _p(status), _stream()), "qk_rope_write")
    return q_out


def qk_rotate_norm(qkv, n_q, n_k, k_off, hd, rot_dim, inv_freq, pairing, positions, eps, unit_norm=True):
    """In place on the rows of qkv [T, *]: the n_q heads at column 0 and the n_k heads at column k_off (hd each) are rotated
    by position on their first rot_dim elements (inv_freq float32 [rot_dim/2], or None for no rotation) and then, with
    unit_norm, divided by their root mean square over hd (eps inside the root; no weight)."""
    _dev(qkv, inv_freq, positions)
    assert qkv.stride(1) == 1
    _i32(positions, "positions")
    rot_dim = 0 if inv_freq is None else int(rot_dim)
    if hd > 512 or rot_dim % 2 or not 0 <= rot_dim <= hd:
        raise KernelError(f"qk_rotate_norm: head size {hd} (at most 512) / rotated part {rot_dim} (even, within the head)")
    if inv_freq is not None:
        assert inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dim // 2 and inv_freq.is_contiguous()
    assert qkv.shape[1] >= max(n_q * hd, k_off + n_k * hd if n_k else 0)
    f = _fn("qk_rope_write", "fellm_qk_rotate_norm",
            [_c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p, _c_int, _c_p, _c_f, _c_int, _c_p])
    _check(f(_p(qkv), _is_bf16(qkv), qkv.stride(0), qkv.shape[0], int(n_q), int(n_k), int(k_off), int(hd), rot_dim,
             _p(inv_freq), PAIRINGS[pairing], _p(positions), float(eps), int(unit_norm), _stream()), "qk_rotate_norm")
    return qkv


def paged_attention_simt(q, pool, block_table, positions, row_slot, layer, scale, window=None, out=None):
    """q [T, H, hd]; pool [pages, layers, 2, G, page_tokens, hd].  Row t attends to the cache
    positions 0..positions[t] (or the last `window` of them) of its item.  Returns [T, H*hd]."""
    _dev(q, pool, block_table, positions, row_slot)
    T, H, hd = q.shape
    G, page_tokens = pool.shape[3], pool.shape[4]
    if hd > 256:
        raise KernelError(f"attention: head_dim {hd} is above the kernel's maximum 256")
    if H % G:
        raise KernelError(f"attention: {H} heads are not a multiple of {G} kv heads")
    assert q.is_contiguous() and pool.is_contiguous() and pool.shape[5] == hd
    _i32(block_table, "block_table"), _i32(positions, "positions"), _i32(row_slot, "row_slot")
    if out is None:
        out = torch.empty((T, H * hd), dtype=q.dtype, device=q.device)
    f = _fn("attention_simt", "fellm_paged_attention_simt",
            [_c_p, _c_int, _c_p, _c_int, _c_p, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_f, _c_int, _c_p])
    _check(f(_p(q), _is_bf16(q), _p(pool), _is_bf16(pool), _p(block_table), block_table.shape[1],
             _p(positions), _p(row_slot), _p(out), T, H, G, hd, page_tokens, layer, pool.shape[1],
             float(scale), int(window or 0), _stream()), "paged_attention_simt")
    return out


def kv_write(src, k_off, v_off, pool, block_table, positions, row_slot, layer, page_tokens, G, hd, vd, status=None):
    """The step's keys (G x hd at column k_off of src's rows) and values (G x vd at v_off) into their pages, as they
    are.  pool [pages, layers, ...]: a page-layer record is K [G][page_tokens][hd] then V [G][page_tokens][vd]."""
    _dev(src, pool, block_table, positions, row_slot)
    T = src.shape[0]
    assert src.stride(1) == 1 and pool.is_contiguous() and pool.dtype == src.dtype
    assert pool[0, 0].numel() == G * page_tokens * (hd + vd)
    _i32(block_table, "block_table"), _i32(positions, "positions"), _i32(row_slot, "row_slot")
    f = _fn("attention_simt", "fellm_kv_write",
            [_c_p, _c_int, _c_int, _c_int, _c_int, _c_p, _c_int, _c_p, _c_int, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_p, _c_p])
    _check(f(_p(src), _is_bf16(src), src.stride(0), k_off, v_off, _p(pool), _is_bf16(pool), _p(block_table),
             block_table.shape[1], _p(positions), _p(row_slot), T, G, hd, vd, page_tokens, layer, pool.shape[1],
             _p(status), _stream()), "kv_write")


ATTENTION_SIMT_MAX_HD = 1024       # the CUDA-core attention kernel's largest key (and value) size


def paged_attention_general(q, H, hd, vd, pool, block_table, positions, row_slot, layer, page_tokens, G, scale, *,
                            window=None, chunk=None, softcap=None, gate=None, slopes=None, q_temp=None, warps=1, write_new=None,
                            sinks=None, out_dim=None, out=None):
    """Attention on CUDA cores with float32 arithmetic for every form the part describes: q read in place from rows
    [T, >= H*hd] (heads at column 0), values of size vd, scores soft-capped (softcap * tanh(s / softcap)), keys limited
    to the last `window` positions and to the query's own block of `chunk` positions, and gate float32 [T, >= H]
    whose sigmoid scales each head's output.  slopes float32 [H]: slopes[h] * (query position - key position) is
    taken off the scaled score.  q_temp = (coef, every): the query at position p is multiplied by
    1 + coef ln(floor((p + 1) / every) + 1).  vd == 0: the values are the keys (a page-layer record holds keys alone).
    warps (1..8): how many warps share a (row, head)'s key tiles; a constant of the layer, since it sets the order of the sums.
    write_new = (k_off, v_off, status): a decode step (every row its request's only one): the rows' own keys and values,
    at those columns of q's rows, are read from there and written into their pages by this kernel (no kv_write in front).
    sinks float32 [H]: exp(sinks[h]) joins head h's softmax denominator (no key, no value, not scaled).  out_dim (with
    vd == 0): only the first out_dim elements of a key are read out as its value.
    Returns [T, H*vd] (H*hd, or H*out_dim, when the values are the keys) in q's dtype."""
    _dev(q, pool, block_table, positions, row_slot, gate, slopes, sinks)
    if sinks is not None:
        assert sinks.dtype == torch.float32 and sinks.numel() == H and sinks.is_contiguous()
    od = int(out_dim or 0)
    if od and (vd or od > hd):
        raise KernelError(f"attention: a read-out of {od} elements needs values that are keys of at least that size")
    T = q.shape[0]
    if slopes is not None:
        assert slopes.dtype == torch.float32 and slopes.numel() == H and slopes.is_contiguous()
    if hd > ATTENTION_SIMT_MAX_HD or vd > ATTENTION_SIMT_MAX_HD:
        raise KernelError(f"attention: head sizes {hd} / {vd} are above the kernel's maximum {ATTENTION_SIMT_MAX_HD}")
    if H % G:
        raise KernelError(f"attention: {H} heads are not a multiple of {G} kv heads")
    assert q.stride(1) == 1 and pool.is_contiguous() and pool[0, 0].numel() == G * page_tokens * (hd + vd)
    _i32(block_table, "block_table"), _i32(positions, "positions"), _i32(row_slot, "row_slot")
    if gate is not None:
        assert gate.dtype == torch.float32 and gate.stride(1) == 1
    if out is None:
        out = torch.empty((T, H * (vd or od or hd)), dtype=q.dtype, device=q.device)
    qt_coef, qt_every = q_temp if q_temp else (0.0, 0)
    f = _fn("attention_simt", "fellm_paged_attention_general",
            [_c_p, _c_int, _c_p, _c_int, _c_p, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_int, _c_f, _c_int, _c_p, _c_int, _c_p, _c_f, _c_int, _c_int, _c_int,
             _c_int, _c_p, _c_p, _c_int, _c_p])
    nk, nv, status = write_new if write_new else (-1, -1, None)
    _check(f(_p(q), _is_bf16(q), _p(pool), _is_bf16(pool), _p(block_table), block_table.shape[1],
             _p(positions), _p(row_slot), _p(out), T, H, G, hd, page_tokens, layer, pool.shape[1],
             float(scale), int(window or 0), vd, q.stride(0), float(softcap or 0.0), int(chunk or 0), _p(gate),
             gate.stride(0) if gate is not None else 0, _p(slopes), float(qt_coef), int(qt_every), int(warps), int(nk), int(nv),
             _p(status), _p(sinks), od, _stream()), "paged_attention_general")
    return out


def latent_prep(z, q_off, rq, c_off, rk, r_off, dr, wq, wc, eps, freq, n_rot, mag, positions, row_slot, cache, out_dtype,
                status=None):
    """A latent-attention layer's down projections z float32 [T, >= ...] -> the normed query latent [T, rq] in out_dtype
    (returned), and into the token's cache row the normed key-value latent (rk) followed by the rotated key part (dr;
    pairs (2i, 2i+1) of its first n_rot elements, angle = position * freq[i], cos and sin times mag).  cache: a
    PagedView whose page-layer record is [page_tokens][rk + dr]."""
    _dev(z, wq, wc, freq, positions, row_slot, cache.pool, cache.block_table)
    assert z.dtype == torch.float32 and z.stride(1) == 1 and wq.dtype == torch.float32 and wc.dtype == torch.float32
    assert wq.numel() == rq and wc.numel() == rk
    pool = cache.pool
    assert pool.is_contiguous() and pool[0, 0].numel() == cache.page_tokens * (rk + dr)
    _i32(positions, "positions"), _i32(row_slot, "row_slot"), _i32(cache.block_table, "block_table")
    T = z.shape[0]
    cq = torch.empty((T, rq), dtype=out_dtype, device=z.device)
    if _is_bf16(cq) != _is_bf16(pool):
        raise KernelError("latent_prep: the cache and the activations are of one dtype")
    f = _fn("latent", "fellm_latent_prep", [_c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p, _c_f, _c_p,
                                            _c_int, _c_f, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int, _c_p,
                                            _c_int, _c_p, _c_p])
    _check(f(_p(z), z.stride(0), q_off, rq, c_off, rk, r_off, dr, _p(wq), _p(wc), float(eps), _p(freq), int(n_rot), float(mag),
             _p(positions), _p(row_slot), _p(cache.block_table), cache.block_table.shape[1], _p(pool), _is_bf16(pool),
             cache.page_tokens, cache.layer, pool.shape[1], _p(cq), T, _p(status), _stream()), "latent_prep")
    return cq


def latent_rotate_q(q, H, dn, dr, q_abs, rk, freq, n_rot, mag, positions):
    """The rotated part of every head's query (dr elements behind the dn unrotated ones of q [T, H * (dn + dr)]), rotated
    by the row's position, into elements [rk, rk + dr) of the head's row of q_abs [T, H * (rk + dr)]."""
    _dev(q, q_abs, freq, positions)
    assert q.stride(1) == 1 and q_abs.is_contiguous() and q.dtype == q_abs.dtype
    assert q.shape[1] >= H * (dn + dr) and q_abs.shape[1] == H * (rk + dr)
    _i32(positions, "positions")
    f = _fn("latent", "fellm_latent_rotate_q", [_c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p, _c_int, _c_p, _c_int, _c_f, _c_p,
                                                _c_int, _c_p])
    _check(f(_p(q), _is_bf16(q), q.stride(0), H, dn, dr, _p(q_abs), rk, _p(freq), int(n_rot), float(mag), _p(positions),
             q.shape[0], _stream()), "latent_rotate_q")
    return q_abs


LATENT_ATTENTION_MMA = os.environ.get("FELLM_B200_LATENT_ATTENTION_MMA", "1") != "0"
LATENT_SINGLE_ROWS = 32        # up to this many (token, head) rows an item: the kernel's form for single tokens
LATENT_MAX_SPLITS = 16


def latent_attention_takes(q_abs, pool, rk: int, dr: int, page_tokens: int) -> bool:
    """Whether the tensor-core kernel takes a latent-attention layer of these sizes: bfloat16 queries and cache, a
    latent of a multiple of 32 up to 512, rows of a multiple of 16 elements, pages of a multiple of 64 tokens."""
    return (LATENT_ATTENTION_MMA and q_abs.dtype == torch.bfloat16 and pool.dtype == torch.bfloat16 and rk % 32 == 0
            and 32 <= rk <= 512 and dr >= 0 and (rk + dr) % 16 == 0 and page_tokens % 64 == 0)


def latent_rotate_fusable(q, q_head: int, off: int) -> bool:
    """Whether latent_attention can read the queries' rotated parts from q itself (16-byte chunks)."""
    return q.dtype == torch.bfloat16 and q.stride(1) == 1 and q.stride(0) % 8 == 0 and q_head % 8 == 0 and off % 8 == 0 and q.data_ptr() % 16 == 0


def latent_attention_modules(rk: int, dr: int):
    return [("latent_attention_mma", {"LAT_RK": rk, "LAT_DR": dr})]


def latent_attention(q_abs, H, rk, dr, pool, block_table, positions, row_slot, item_start, n_items, max_item_rows, max_len,
                     layer, page_tokens, scale, *, window=None, sinks=None, out=None, q_rot=None):
    """Latent attention on tensor cores (bfloat16): q_abs [T, H * (rk + dr)] contiguous, the queries taken into the
    cache rows' space; pool's page-layer record is [page_tokens][rk + dr]; rows of item i are
    item_start[i]..item_start[i + 1] with consecutive positions.  A key's value is the first rk elements of its row.
    sinks float32 [H]: exp(sinks[h]) joins head h's denominator.  max_len: the longest context of the step (it only
    sizes the split of a single token's key walk).  q_rot = (q, q_head, off, freq, n_rot, mag): q_abs is [T, H * rk], and
    head h's rotated part is read from columns [h q_head + off, + dr) of q [T, >= H q_head] and rotated by the row's
    position inside the kernel (pairs (2i, 2i + 1) of its first n_rot elements, angle = position * freq[i], cos and sin
    times mag); see latent_rotate_fusable.  Returns [T, H * rk]."""
    _dev(q_abs, pool, block_table, positions, row_slot, item_start, sinks)
    T = q_abs.shape[0]
    assert latent_attention_takes(q_abs, pool, rk, dr, page_tokens)
    qsrc, ldq, q_head, q_off, freq, n_rot, mag = None, 0, 0, 0, None, 0, 1.0
    if q_rot is not None and dr:
        qsrc, q_head, q_off, freq, n_rot, mag = q_rot
        _dev(qsrc, freq)
        assert latent_rotate_fusable(qsrc, q_head, q_off) and qsrc.shape[0] == T and qsrc.shape[1] >= (H - 1) * q_head + q_off + dr
        ldq = qsrc.stride(0)
    width = rk if (q_rot is not None) else rk + dr
    assert q_abs.is_contiguous() and q_abs.shape[1] == H * width and pool.is_contiguous()
    assert pool[0, 0].numel() == page_tokens * (rk + dr)
    _i32(block_table, "block_table"), _i32(positions, "positions"), _i32(row_slot, "row_slot"), _i32(item_start, "item_start")
    if sinks is not None:
        assert sinks.dtype == torch.float32 and sinks.numel() == H and sinks.is_contiguous()
    if out is None:
        out = torch.empty((T, H * rk), dtype=torch.bfloat16, device=q_abs.device)
    variant = 1 if max_item_rows * H <= LATENT_SINGLE_ROWS else 0
    n_splits, scratch = 1, None
    if variant == 1:
        # few CTAs walk many keys: split the walk so that the SMs have work (a constant of the step's shape)
        kt = 64 if rk % 64 == 0 else 32
        longest = -(-int(max_len) // 1024) * 1024          # (a captured step serves contexts up to the next multiple of 1,024)
        span = min(int(window), longest) if window else longest
        tiles = span // kt + 2
        ctas = n_items * (-(-max_item_rows * H // 16))
        n_splits = max(1, min(tiles // 2, 148 // max(ctas, 1), LATENT_MAX_SPLITS))
        if n_splits > 1:
            scratch = torch.empty((T * H * n_splits * (rk + 2),), dtype=torch.float32, device=q_abs.device)
    f = _fn("latent_attention_mma", "fellm_latent_attention_mma",
            [_c_p, _c_p, _c_p, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_f, _c_int, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_p, _c_int, _c_f, _c_p], defines={"LAT_RK": rk, "LAT_DR": dr})
    _check(f(_p(q_abs), _p(pool), _p(block_table), block_table.shape[1], _p(positions), _p(row_slot), _p(item_start),
             int(n_items), int(max_item_rows), T, _p(out), _p(scratch), n_splits, H, page_tokens, layer, pool.shape[1],
             float(scale), int(window or 0), _p(sinks), variant, _p(qsrc), ldq, int(q_head), int(q_off), _p(freq), int(n_rot), float(mag),
             _stream()), "latent_attention")
    return out


# ------------------------------------------------------------------------------ tensor-core products

_EPI_STORE, _EPI_ACC, _EPI_SWIGLU, _EPI_F32 = 0, 1, 2, 3
SKINNY_MAX_ROWS = 32      # measured on B200 (350M shapes): above 32 rows the tcgen05 product wins on every shape
_GEMM_ARGS = [_c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p]
_SKINNY_ARGS = [_c_p, _c_p, _c_p, _c_f, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p]
NORM_FUSE_MAX_ROWS = 16


def fast_gemm_modules():
    return [("gemm_skinny", None), ("gemm_tiled", None), ("gemm_umma", None)]


_umma_status = {}
USE_UMMA = os.environ.get("FELLM_B200_UMMA", "1") != "0"
USE_UMMA_SWAP = os.environ.get("FELLM_B200_UMMA_SWAP", "1") != "0"
FUSE_SWAP_CONV = os.environ.get("FELLM_B200_FUSE_SWAP_CONV", "1") != "0"     # the convolution in that product's epilogue (17..64 rows)
SWAP_CONV_MAX_K = int(os.environ.get("FELLM_B200_SWAP_CONV_MAX_K", 1536))
SWAP_CONV_MAX_ROWS = int(os.environ.get("FELLM_B200_SWAP_CONV_MAX_ROWS", 64))
SWAP_MIN_ROWS = int(os.environ.get("FELLM_B200_SWAP_MIN_ROWS", 17))     # fewer rows: the weight-streaming kernel (norm and convolution fused)
SWAP_MAX_ROWS = int(os.environ.get("FELLM_B200_SWAP_MAX_ROWS", 128))     # more rows: the persistent tcgen05 product (width 1024, 128 rows: 1.68 ms a step there, 1.28 here)
SWAP_MAX_N = 16384                                                       # wider (the vocabulary head): the persistent tcgen05 product


def umma_status(device) -> torch.Tensor:
    """Device int32 the tcgen05 product sets when one of its bounded waits ran out (101 TMA
    producer, 102 MMA issuer, 103 epilogue); zero otherwise."""
    key = torch.device(device).index or 0
    t = _umma_status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _umma_status[key] = t
    return t


def check_umma_status(device):
    """Reads the status word (synchronises)."""
    t = _umma_status.get(torch.device(device).index or 0)
    if t is not None:
        code = int(t.item())
        if code:
            t.zero_()
            if code == 302:
                raise KernelError("decode attention: a row's position has no cache page mapped")
            what = ("the TMA decode attention" if code == 301 else
                    "the tcgen05 prefill attention" if 311 <= code <= 317 else
                    "the tcgen05 product of few rows" if 111 <= code <= 113 else
                    "the tcgen05 product on CTA pairs" if 121 <= code <= 124 else
                    "the tcgen05 product with K over two CTAs" if 131 <= code <= 134 else "the tcgen05 product")
            raise KernelError(f"{what} gave up waiting on a barrier (role {code})")


def fast_gemm_takes(x, w) -> bool:
    """The tensor-core kernels read 16-byte vectors along K."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1)


def norm_fusable(x_f32, w, norm_w) -> bool:
    """Whether RMSNorm of the float32 rows x can run inside the product with w (few rows, the whole
    K range in one CTA's shared memory)."""
    M, K = x_f32.shape
    return (M <= NORM_FUSE_MAX_ROWS and w.dtype == torch.bfloat16 and x_f32.dtype == torch.float32
            and norm_w.dtype == torch.float32 and K % 8 == 0 and K <= 8192 and w.stride(0) % 8 == 0
            and x_f32.stride(1) == 1 and x_f32.stride(0) % 4 == 0 and w.stride(1) == 1
            and not _wide_on_umma(M, w.shape[0], K))


WIDE_GENERAL_N = int(os.environ.get("FELLM_B200_WIDE_GENERAL_N", 32768))


def _wide_on_umma(M: int, N: int, K: int) -> bool:
    """A very wide product (a vocabulary head) of 9..16 rows that the single-shot weight-streaming kernel does not
    take (K = 1536: six slices, no power of two of K warps) runs on the persistent tcgen05 product behind an
    RMSNorm kernel of its own: the general weight-streaming kernel with two row tiles is bound by its instructions
    there (measured on B200, [65536 x 1536]: 83 us at 16 rows, 32 us at 8, 31 us of bytes)."""
    return (USE_UMMA and 8 < M <= 16 and N >= WIDE_GENERAL_N and K % 8 == 0
            and not _single_shot(M, N, K, False) and not _single_shot(M, N, K, True))


_single_shot_cache = {}

# The matrix each bfloat16 product's successor reads, by the data pointer of the product's own matrix:
# a product's launch tells its kernel, whose CTAs ask the L2 for it before they wait for the kernel in
# front of them.  Filled by register_weight_chain(); empty: nobody prefetches.
_next_weight = {}
WEIGHT_PREFETCH = os.environ.get("FELLM_B200_WEIGHT_PREFETCH", "1") != "0"
PREFETCH_MAX_BYTES = int(os.environ.get("FELLM_B200_WEIGHT_PREFETCH_MAX_MB", 48)) << 20     # well inside the L2's 126 MB


def register_weight_chain(weights):
    """weights: the bfloat16 matrices of a decode step in the order its products read them (the last
    is followed by the first: the next step).  Replaces what was registered before for these matrices."""
    ws = [w for w in weights if w is not None and w.dtype == torch.bfloat16 and w.is_cuda and w.is_contiguous()]
    for w, nxt in zip(ws, ws[1:] + ws[:1]):
        _next_weight[w.data_ptr()] = (nxt.data_ptr(), min(nxt.numel() * 2, PREFETCH_MAX_BYTES))


PREFETCH_MAX_ROWS = 16     # measured on B200: 2% off a step of 1 or 8 rows, 1-6% ON a step of 64 (its products are short of bandwidth, not of latency)


def _announce_next(module: str, w, rows: int):
    """Tells the module's next launch which matrix comes after w."""
    if WEIGHT_PREFETCH and _next_weight and rows <= PREFETCH_MAX_ROWS:
        nxt = _next_weight.get(w.data_ptr())
        if nxt is not None:
            _fn(module, "fellm_next_weights", [_c_p, _c_ll])(nxt[0], nxt[1])


def _single_shot(M: int, N: int, K: int, norm: bool) -> bool:
    key = (M, N, K, norm)
    hit = _single_shot_cache.get(key)
    if hit is None:
        f = _fn("gemm_skinny", "fellm_gemm_skinny_single_shot", [_c_int, _c_int, _c_int, _c_int])
        hit = _single_shot_cache[key] = bool(f(M, N, K, int(norm)))
    return hit


# ---- an RMSNorm handed on from the product that writes the residual stream to the product that reads it
#
# In a decode step of up to 16 rows every product is a few microseconds long, and a product that first has
# to norm float32 rows (read them, sum the squares, scale, round) spends a third of that before its first
# MMA.  So the product that ADDS into the residual stream can do the norm's work for its successor: beside
# x += ..., it leaves xg = bfloat16(x * g) (g: the next norm's weights) and the sums of x^2 of every 16
# columns.  The successor stages xg like any bfloat16 input and multiplies its finished sums by the rows'
# factors 1 / sqrt(sum x^2 / K + eps): RMSNorm(x) W^T with the factor taken out of the product.
#
# Who writes and who reads is settled by the caller: expect_norm(x, g) says "the next product that adds
# into x is followed by an RMSNorm with weights g"; norm_handoff(x, g) gives the reader what was left, if
# it is still good (same tensor, same weights, nothing written to x since).
NORM_HANDOFF = os.environ.get("FELLM_B200_NORM_HANDOFF", "1") != "0"
HANDOFF_MAX_ROWS = 128       # up to 16 rows: the weight-streaming kernel on both sides; 17..128: the tcgen05 product of few rows
_handoff_bufs = {}          # device -> (xg bfloat16 [16 * width], ssq float32 [16 * width / 16], width)
_handoff_retired = []
_expected_norm = None       # (data_ptr of x, norm weights)
_handoff = None             # NormHandoff: what the last such product left


class NormHandoff:
    __slots__ = ("x_ptr", "version", "rows", "norm_ptr", "xg", "ssq", "parts")


def reserve_norm_handoff(device, width: int):
    """Room for handed-on norms of rows up to `width` wide (called before the first step, so that nothing
    is allocated under a captured graph).  Without it no norm is handed on."""
    device = torch.device(device)
    if device.type != "cuda" or width % 16 or width > 2048:        # the kernel takes up to 128 parts of 16 columns
        return
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    have = _handoff_bufs.get(device)
    if have is None or have[2] < width:
        if have is not None:
            _handoff_retired.append(have)      # graphs captured with the old buffers may still be replayed
        _handoff_bufs[device] = (torch.zeros(HANDOFF_MAX_ROWS * width, dtype=torch.bfloat16, device=device),
                                 torch.zeros(HANDOFF_MAX_ROWS * width // 16, dtype=torch.float32, device=device), width)
        forget_norm_handoff()


def forget_norm_handoff():
    global _expected_norm, _handoff
    _expected_norm = _handoff = None


def expect_norm(x, norm_w):
    """The next product that adds into x (float32 [rows, d]) is followed by RMSNorm with norm_w [d]."""
    global _expected_norm
    _expected_norm = None
    if (NORM_HANDOFF and x.is_cuda and x.dtype == torch.float32 and x.shape[0] <= HANDOFF_MAX_ROWS
            and norm_w.dtype == torch.float32 and norm_w.numel() == x.shape[1] and norm_w.is_contiguous()):
        bufs = _handoff_bufs.get(x.device)
        if bufs is not None and bufs[2] >= x.shape[1]:
            _expected_norm = (x.data_ptr(), norm_w)


def residual_written(out):
    """Every kernel call that adds into a float32 tensor says so: what was handed on for it is stale.
    Returns the norm expected after this write (expect_norm), if one was announced for this tensor."""
    global _handoff, _expected_norm
    if _handoff is not None and _handoff.x_ptr == out.data_ptr():
        _handoff = None
    exp, _expected_norm = _expected_norm, None          # an expectation is for the very next write
    return exp if (exp is not None and exp[0] == out.data_ptr()) else None


def norm_handoff(x, norm_w):
    """What the last product that added into x left for RMSNorm(x, norm_w), or None."""
    h = _handoff
    if (h is None or h.x_ptr != x.data_ptr() or h.version != x._version or h.rows != x.shape[0]
            or h.norm_ptr != norm_w.data_ptr()):
        return None
    return h


def _swap_rows(M: int, N: int) -> bool:
    """Whether gemm_bf16 gives a product of M rows and N columns to the tcgen05 product of few rows."""
    return USE_UMMA and USE_UMMA_SWAP and max(SWAP_MIN_ROWS, 17) <= M <= SWAP_MAX_ROWS and N <= SWAP_MAX_N


def row_scale_takes(M: int, N: int, K: int) -> bool:
    """Whether a product of these sizes can take a handed-on norm's input: up to 16 rows the single-shot
    weight-streaming kernel, 17..128 rows the tcgen05 product of few rows."""
    if K % 8:
        return False
    if M <= 16:
        return _single_shot(M, N, K, False)
    return _swap_rows(M, N)


def _announce_handoff(exp, out, M: int, N: int, K: int, norm_fused: bool):
    """Before an accumulate product of the weight-streaming kernel: if its successor's norm is known (exp)
    and the kernel can do it, tell the kernel and note what it leaves."""
    global _handoff
    if exp is None or M > HANDOFF_MAX_ROWS or not out.is_contiguous() or norm_fused:
        return
    if M <= 16:
        if N % 16 or not _single_shot(M, N, K, False):
            return
        module, per_part = "gemm_skinny", 16
    else:
        if N % 128 or not _swap_rows(M, N):
            return
        module, per_part = "gemm_umma", 128
    xg, ssq, width = _handoff_bufs[out.device]
    _handoff = None                      # the buffers are about to be rewritten
    f = _fn(module, f"fellm_{module}_next_norm", [_c_p, _c_p, _c_int, _c_p])
    f(_p(exp[1]), _p(xg), N, _p(ssq))
    h = NormHandoff()
    h.x_ptr, h.version, h.rows, h.norm_ptr = out.data_ptr(), out._version, M, exp[1].data_ptr()
    h.xg, h.ssq, h.parts = xg[:M * N].view(M, N), ssq, N // per_part
    return h


def _announce_row_scale(row_scale, M: int, N: int, K: int, own_plan: bool = False):
    ssq, parts, eps = row_scale
    if not own_plan and not row_scale_takes(M, N, K):
        raise KernelError(f"a product of {M} x {N} x {K} does not take a handed-on norm")
    assert ssq.dtype == torch.float32 and ssq.numel() >= M * parts
    module = "gemm_skinny" if M <= 16 else "gemm_umma"
    _fn(module, f"fellm_{module}_row_scale", [_c_p, _c_int, _c_f])(_p(ssq), int(parts), float(eps))


def gemm_bf16(x, w, bias=None, *, out=None, out_dtype=None, accumulate=False, swiglu=False, norm=None, row_scale=None):
    """out = x[M,K] @ w[N,K]^T (+bias) on tensor cores, bfloat16 in, float32 sums.
    accumulate: out (float32 [M,N]) += ; swiglu: w's rows are interleaved in blocks of 8 gate / 8 up
    and out is bfloat16 [M, N/2] = silu(gate)*up; out_dtype float32: float32 store.
    norm=(weight float32 [K], eps): x is the float32 residual stream and is RMS-normed on its way
    into the product (see norm_fusable).
    row_scale=(ssq, parts, eps): x is the pre-weighted input of a handed-on norm (norm_handoff)."""
    global _handoff
    _dev(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm: x is [{M},{K}] but w is {list(w.shape)}")
    if norm is not None:
        if not norm_fusable(x, w, norm[0]):
            raise KernelError("gemm_bf16: this product cannot take a fused RMSNorm")
    elif not fast_gemm_takes(x, w):
        raise KernelError(f"gemm_bf16: K={K} and the row strides must be multiples of 8 bfloat16 elements")
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    if accumulate:
        epi = _EPI_ACC
        assert out is not None and out.dtype == torch.float32 and out.shape == (M, N)
    elif swiglu:
        epi = _EPI_SWIGLU
        if N % 16:
            raise KernelError(f"gemm_bf16: the gate/up matrix needs a multiple of 16 rows, got {N}")
        if out is None:
            out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
        assert out.dtype == torch.bfloat16 and out.shape == (M, N // 2)
    elif (out_dtype or (out.dtype if out is not None else torch.bfloat16)) == torch.float32:
        epi = _EPI_F32
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    else:
        epi = _EPI_STORE
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        assert out.dtype == torch.bfloat16
    assert out.stride(1) == 1
    if M == 0:
        return out
    umma_ok = (USE_UMMA and norm is None and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
               and (epi != _EPI_SWIGLU or out.stride(0) % 8 == 0))
    # few rows: the weight-streaming kernel; up to 64 rows: it too where its single-shot form takes the
    # product (all of W requested at once by every SM), else up to 32 rows except for very wide products
    # (measured at 64 rows: 14 us against 26 us for [1024, 4608], 8 against 9-11 for K = 1024, but 13
    # against 11 for the 9216 rows of gate/up, which stays with tcgen05 beyond 32 rows)
    expected = residual_written(out) if accumulate else None
    if umma_ok and USE_UMMA_SWAP and SWAP_MIN_ROWS <= M <= SWAP_MAX_ROWS and N <= SWAP_MAX_N and (row_scale is None or M > 16):
        # a decode step of 17..128 rows: tcgen05 with the weights as the MMA's 128 rows
        _announce_next("gemm_umma", w, M)
        if row_scale is not None:
            _announce_row_scale(row_scale, M, N, K)
        left = _announce_handoff(expected, out, M, N, K, False) if M > 16 else None
        gemm_umma_swap(x, w, bias, out=out, epi=epi, written=True)
        if left is not None:
            _handoff = left
        return out
    skinny = M <= 64 and ((M <= 16 and not (umma_ok and _wide_on_umma(M, N, K))) or not umma_ok
                          or (_single_shot(M, N, K, norm is not None) and (M <= 32 or N < 8192))
                          or (M <= SKINNY_MAX_ROWS and N < 8192))
    if row_scale is not None and (not skinny or M > 16):
        raise KernelError(f"a product of {M} x {N} x {K} does not take a handed-on norm")
    if skinny:
        _announce_next("gemm_skinny", w, M)
        if row_scale is not None:
            _announce_row_scale(row_scale, M, N, K)
        left = _announce_handoff(expected, out, M, N, K, norm is not None) if M <= 16 else None
        f = _fn("gemm_skinny", "fellm_gemm_skinny", _SKINNY_ARGS)
        if norm is not None:
            code = f(None, _p(x), _p(norm[0]), float(norm[1]), _p(w), _p(bias), _p(out), epi, M, N, K, x.stride(0),
                     w.stride(0), out.stride(0), _stream())
        else:
            code = f(_p(x), None, None, 0.0, _p(w), _p(bias), _p(out), epi, M, N, K, x.stride(0), w.stride(0),
                     out.stride(0), _stream())
        _check(code, "gemm_skinny")
        if left is not None:
            _handoff = left
    elif umma_ok:
        f = _fn("gemm_umma", "fellm_gemm_umma", _GEMM_ARGS[:-1] + [_c_p, _c_p])
        _check(f(_p(x), _p(w), _p(bias), _p(out), epi, M, N, K, x.stride(0), w.stride(0), out.stride(0),
                 _p(umma_status(x.device)), _stream()), "gemm_umma")
    else:
        f = _fn("gemm_tiled", "fellm_gemm_tiled", _GEMM_ARGS)
        _check(f(_p(x), _p(w), _p(bias), _p(out), epi, M, N, K, x.stride(0), w.stride(0), out.stride(0), _stream()),
               "gemm_tiled")
    return out


_argmax_scratch_cache = {}
FUSED_ARGMAX = os.environ.get("FELLM_B200_FUSED_ARGMAX", "1") != "0"


def head_argmax_scratch(M: int, N: int, K: int, norm: bool) -> int:
    """8-byte keys gemm_bf16_argmax needs for a product of these sizes; 0: it does not take it (more than
    16 rows, or sizes the single-shot product leaves to the general kernel)."""
    key = (M, N, K, norm)
    hit = _argmax_scratch_cache.get(key)
    if hit is None:
        f = _fn("gemm_skinny", "fellm_gemm_skinny_argmax_scratch", [_c_int, _c_int, _c_int, _c_int])
        f.restype = _c_ll
        hit = _argmax_scratch_cache[key] = int(f(M, N, K, int(norm)))
    return hit


def gemm_bf16_argmax(x, w, bias, keys, out_tokens, *, norm=None, row_scale=None):
    """out_tokens[m] = argmax_n (x W^T + bias)[m, n], ties to the lower n, without storing the [M, N]
    logits: the vocabulary head of a greedy decode step of up to 16 rows.  x bfloat16 [M, K], or with
    norm=(weight, eps) the float32 residual rows, or with row_scale=(ssq, parts, eps) the pre-weighted input
    of a handed-on norm; keys: int64 scratch of head_argmax_scratch() entries; out_tokens int32 [>= M]."""
    _dev(x, w, bias, keys, out_tokens)
    M, K = x.shape
    N = w.shape[0]
    need = head_argmax_scratch(M, N, K, norm is not None)
    if not need or w.dtype != torch.bfloat16 or w.stride(1) != 1 or x.stride(1) != 1:
        raise KernelError(f"gemm_bf16_argmax does not take a product of {M} x {N} x {K}")
    assert keys.dtype == torch.int64 and keys.numel() >= need and out_tokens.dtype == torch.int32 and out_tokens.numel() >= M
    _announce_next("gemm_skinny", w, M)
    if row_scale is not None:
        assert norm is None
        _announce_row_scale(row_scale, M, N, K)
    f = _fn("gemm_skinny", "fellm_gemm_skinny_argmax",
            [_c_p, _c_p, _c_p, _c_f, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p])
    if norm is not None:
        assert x.dtype == torch.float32 and norm[0].dtype == torch.float32
        code = f(None, _p(x), _p(norm[0]), float(norm[1]), _p(w), _p(bias), _p(keys), _p(out_tokens), M, N, K,
                 x.stride(0), w.stride(0), _stream())
    else:
        assert x.dtype == torch.bfloat16
        code = f(_p(x), None, None, 0.0, _p(w), _p(bias), _p(keys), _p(out_tokens), M, N, K, x.stride(0), w.stride(0),
                 _stream())
    _check(code, "gemm_skinny_argmax")
    global _launches
    _launches += 1                      # the product and the pick of the best key
    return out_tokens


def gemm_umma_swap(x, w, bias=None, *, out, epi: int, written: bool = False):
    """The tcgen05 product for up to 128 rows (weights as the MMA's rows, K split over a cluster),
    callable by itself.  epi: 0 store bfloat16, 1 add into float32, 2 SiLU(gate)*up, 3 store float32."""
    M, K = x.shape
    if epi == _EPI_ACC and not written:
        residual_written(out)
    f = _fn("gemm_umma", "fellm_gemm_umma_swap", _GEMM_ARGS[:-1] + [_c_p, _c_p])
    _check(f(_p(x), _p(w), _p(bias), _p(out), epi, M, w.shape[0], K, x.stride(0), w.stride(0), out.stride(0),
             _p(umma_status(x.device)), _stream()), "gemm_umma_swap")
    return out


def gemm_tiled(x, w, bias=None, *, out, epi: int):
    """The mma.sync product, callable by itself (tests compare the tcgen05 product with it)."""
    M, K = x.shape
    if epi == _EPI_ACC:
        residual_written(out)
    f = _fn("gemm_tiled", "fellm_gemm_tiled", _GEMM_ARGS)
    _check(f(_p(x), _p(w), _p(bias), _p(out), epi, M, w.shape[0], K, x.stride(0), w.stride(0), out.stride(0), _stream()),
           "gemm_tiled")
    return out


def interleave_gate_up(gate, up):
    """[F,K] gate and up -> [2F,K] with rows in blocks of 16: 8 gate rows, then the 8 up rows of the
    same features (what the SiLU(gate)*up epilogues expect).  F must be a multiple of 8."""
    F, K = gate.shape
    assert F % 8 == 0 and up.shape == gate.shape
    return torch.stack([gate.reshape(F // 8, 8, K), up.reshape(F // 8, 8, K)], dim=1).reshape(2 * F, K).contiguous()


# ------------------------------------------------------------------------------ attention dispatch

_decode_scratch = {}
_decode_scratch_retired = []      # replaced buffers stay alive: a CUDA graph captured earlier still names them


def decode_scratch_need(max_rows: int, heads: int, kv_heads: int, head_dim: int, n_ctx: int):
    """(floats, counters) the split-KV decode kernel can ask for with up to max_rows rows and
    contexts up to n_ctx: the largest over every row count of what attention_decode reserves."""
    floats = 0
    for rows in range(1, max(max_rows, 1) + 1):
        for bucket in range(1024, max(n_ctx, 1) + 1024, 1024):       # the split is chosen per 1024 of context
            _, max_splits = decode_split(bucket, rows, kv_heads)
            floats = max(floats, rows * heads * max_splits * (head_dim + 2))
    return floats, max(max_rows, 1) * kv_heads


def reserve_decode_scratch(device, rows: int, heads: int, kv_heads: int, head_dim: int, max_splits: int, *,
                           floats: int = 0, counters: int = 0):
    """Scratch of the split-KV decode kernel: partial results of every (row, head, key range) and
    one counter per (row, kv head).  An engine sizes it once, before its first step, for the
    largest step it can run (floats=, counters= from decode_scratch_need); a later call that needs
    more (kernels called by hand at other sizes) gets a new buffer, never during a graph capture,
    and the old one is kept alive for the graphs that were captured with it."""
    need = max(rows * heads * max_splits * (head_dim + 2), floats, 1 << 21)     # at least 8 MB: growth is rare
    need_c = max(rows * kv_heads, counters, 1 << 16)
    device = torch.device(device)
    cur = _decode_scratch.get(device)
    if cur is None or cur[0].numel() < need or cur[1].numel() < need_c:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("decode attention scratch must be reserved before graph capture")
        if cur is not None:
            _decode_scratch_retired.append(cur)
        scratch = torch.empty(max(need, cur[0].numel() if cur else 0), dtype=torch.float32, device=device)
        counters_t = torch.zeros(max(need_c, cur[1].numel() if cur else 0), dtype=torch.int32, device=device)
        _decode_scratch[device] = (scratch, counters_t)
    return _decode_scratch[device]


# CTAs the split of decode attention aims at: one wave of the TMA kernel (three CTAs of 68 KB to an
# SM).  Measured on B200, 16 layers of width 1024, context 2048 (4000): batch 8 379 (411) us a step
# with 444, 387 (438) with 592, 399 (417) with 300; batch 32 764 with 444, 822 with 592.
DECODE_TARGET_CTAS = int(os.environ.get("FELLM_B200_DECODE_TARGET", 0))     # 0: three CTAs for every SM of the device
BIG_BATCH_SPLITS = int(os.environ.get("FELLM_B200_DECODE_BIG_SPLITS", 2))
DECODE_STAGES = int(os.environ.get("FELLM_B200_DECODE_STAGES", 0))           # 0: by the step's size (decode_stages)
_sm_count = {}


def sm_count(device=None) -> int:
    """SMs of the device (of a B200, 148, where no GPU is present: the planners are checked on CPU too)."""
    if not torch.cuda.is_available():
        return 148
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    n = _sm_count.get(idx)
    if n is None:
        n = _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


def decode_target_ctas() -> int:
    return DECODE_TARGET_CTAS or 3 * sm_count()


SPLIT_WHOLE_ROUNDS = os.environ.get("FELLM_B200_SPLIT_ROUNDS", "1") != "0"
DECODE_MAX_RANGES = int(os.environ.get("FELLM_B200_DECODE_MAX_RANGES", 8))        # of contexts up to 8 x 512 keys (0: no limit)
USE_TMA_DECODE = os.environ.get("FELLM_B200_TMA_DECODE", "1") != "0"
FUSE_DECODE_ROPE = os.environ.get("FELLM_B200_FUSE_ROPE", "1") != "0"
USE_TMA_PREFILL = os.environ.get("FELLM_B200_TMA_PREFILL", "1") != "0"
USE_UMMA_PREFILL = os.environ.get("FELLM_B200_UMMA_ATTN", "1") != "0"
GENERAL_ATTENTION_MMA = os.environ.get("FELLM_B200_GENERAL_ATTN_MMA", "1") != "0"     # capped / chunked / gated prefill on tensor cores
UMMA_PREFILL_MIN_ROWS = int(os.environ.get("FELLM_B200_UMMA_ATTN_MIN_ROWS", 1))    # (token, head) rows of the longest item


def decode_stages(rows: int, kv_heads: int) -> int:
    """Half pages a warp of the TMA decode kernel keeps in flight: 4 (a CTA to an SM) for the few CTAs of a
    step of one or two requests, which then ask for most of their keys at once, else 2 (three CTAs to an SM).
    Measured on B200 (16 layers of width 1024, context 2048): batch 1 0.332 ms a step with 4 against 0.356
    with 2; batch 8 0.400 against 0.396; batch 64 1.22 against 0.92."""
    if DECODE_STAGES:
        return DECODE_STAGES
    return 4 if rows * kv_heads <= 16 else 2


def decode_split(max_len: int, rows: int, kv_heads: int, target: int = 0):
    """(split_len, max_splits): key ranges of a multiple of 64 keys, enough of them to fill the
    machine (at most 8, one cluster, while a range then stays within 512 keys).  max_len is
    rounded up to 1024 so that the choice (and a captured graph) holds while contexts grow."""
    bucket = -(-max(max_len, 1) // 1024) * 1024
    items = max(rows * kv_heads, 1)
    if not target:
        target = decode_target_ctas() // 3 if decode_stages(rows, kv_heads) == 4 else decode_target_ctas()
    want = max(1, target // items)
    if DECODE_MAX_RANGES and bucket <= DECODE_MAX_RANGES * 512:
        # up to 8 ranges are one cluster and merge through its shared memory: worth more than further ranges while a
        # range stays within two pages a warp (measured on B200, context 2,050..2,250: batch 1 0.316 -> 0.310 ms a step
        # with 8 ranges instead of 16, batch 4 0.3415 -> 0.340 with 6 instead of 12)
        want = min(want, DECODE_MAX_RANGES)
    if items > target:
        want = BIG_BATCH_SPLITS      # more than a wave even unsplit: halves, so that the last wave is a short one
    split_len = max(64, -(-(-(-bucket // want)) // 64) * 64)
    if split_len > 256 and SPLIT_WHOLE_ROUNDS:
        split_len = -(-split_len // 256) * 256      # whole rounds of the kernel's four warps, a page each
    return split_len, -(-bucket // split_len)


def _mma_checks(q, pool, what):
    T, H, hd = q.shape
    if q.dtype != torch.bfloat16 or pool.dtype != torch.bfloat16:
        raise KernelError(f"{what} takes bfloat16 queries and cache")
    if hd % 16 or not 16 <= hd <= 256:
        raise KernelError(f"{what}: head_dim {hd} must be a multiple of 16 in 16..256")
    G = pool.shape[3]
    if H % G:
        raise KernelError(f"{what}: {H} heads are not a multiple of {G} kv heads")
    assert q.is_contiguous() and pool.is_contiguous() and pool.shape[5] == hd
    return T, H, G, hd, pool.shape[4]


def decode_fuses_rope(H: int, G: int, hd: int, page_tokens: int, pool) -> bool:
    """Whether attention_decode can take the QKV product's output itself (fuse=...): the TMA kernel's sizes."""
    return (USE_TMA_DECODE and FUSE_DECODE_ROPE and hd == 64 and page_tokens == 64 and G > 0 and H % G == 0
            and H // G <= 16 and pool.numel() // hd < 2 ** 31)


def attention_decode(q, pool, block_table, positions, row_slot, layer, scale, window, max_len, out=None, fuse=None):
    """One query row per request (bfloat16): split-KV decode attention on tensor cores.
    q [T, H, hd] -> [T, H*hd].  The kernel library is compiled for this head size.
    fuse=(qkv [T, (H+2G)*hd], q_w, k_w, eps, inv_freq, pairing) with q=None (see decode_fuses_rope):
    the kernel norms and rotates q and k itself and writes k and v into the cache."""
    if fuse is not None:
        qkv = fuse[0]
        G, hd, page_tokens = pool.shape[3], pool.shape[5], pool.shape[4]
        T = qkv.shape[0]
        H = qkv.shape[1] // hd - 2 * G
        assert q is None and qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and decode_fuses_rope(H, G, hd, page_tokens, pool)
        _dev(qkv, pool, block_table, positions, row_slot, fuse[1], fuse[2], fuse[4])
        assert pool.dtype == torch.bfloat16 and pool.is_contiguous()
    else:
        _dev(q, pool, block_table, positions, row_slot)
        T, H, G, hd, page_tokens = _mma_checks(q, pool, "attention_decode")
    split_len, max_splits = decode_split(max_len, T, G)
    scratch, counters = reserve_decode_scratch(pool.device, T, H, G, hd, max_splits)
    if out is None:
        out = torch.empty((T, H * hd), dtype=torch.bfloat16, device=pool.device)
    if fuse is not None or (USE_TMA_DECODE and hd == 64 and page_tokens == 64 and H // G <= 16 and pool.numel() // hd < 2 ** 31):
        # pages of 64 tokens at head size 64: whole tiles by TMA
        f = _fn("attention_mma", "fellm_attn_decode_tma",
                [_c_p, _c_p, ctypes.c_longlong, _c_p, _c_int, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int,
                 _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_f, _c_p, _c_int,
                 _c_int, _c_p], defines={"HD": hd})
        if fuse is not None:
            qkv, q_w, k_w, eps, inv_freq, pairing = fuse
            extra = (_p(qkv), _p(q_w), _p(k_w), float(eps), _p(inv_freq), PAIRINGS[pairing])
        else:
            extra = (None, None, None, 0.0, None, 0)
        _check(f(_p(q), _p(pool), pool.shape[0], _p(block_table), block_table.shape[1], _p(positions), _p(row_slot),
                 _p(out), _p(scratch), _p(counters), T, H, G, hd, page_tokens, layer, pool.shape[1], float(scale),
                 int(window or 0), split_len, max_splits, _p(umma_status(pool.device)), *extra, decode_stages(T, G),
                 _stream()), "attention_decode (TMA)")
        return out
    f = _fn("attention_mma", "fellm_attn_decode_mma",
            [_c_p, _c_p, _c_p, _c_int, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_f, _c_int, _c_int, _c_int, _c_p], defines={"HD": hd})
    _check(f(_p(q), _p(pool), _p(block_table), block_table.shape[1], _p(positions), _p(row_slot), _p(out),
             _p(scratch), _p(counters), T, H, G, hd, page_tokens, layer, pool.shape[1], float(scale),
             int(window or 0), split_len, max_splits, _stream()), "attention_decode")
    return out


def attention_prefill(q, pool, block_table, positions, row_slot, item_start, n_items, max_item_rows, layer, scale,
                      window, out=None):
    """Portions of prompts (items of any length, one token included) on tensor cores (bfloat16).
    Rows of item i are item_start[i]..item_start[i+1] with consecutive positions."""
    _dev(q, pool, block_table, positions, row_slot, item_start)
    T, H, G, hd, page_tokens = _mma_checks(q, pool, "attention_prefill")
    if H // G > 64:
        raise KernelError(f"attention_prefill: {H // G} heads per kv head exceed the kernel's 64")
    _i32(item_start, "item_start")
    if out is None:
        out = torch.empty((T, H * hd), dtype=q.dtype, device=q.device)
    if (USE_UMMA_PREFILL and hd == 64 and page_tokens == 64 and not window and pool.numel() // hd < 2 ** 31
            and 128 % (H // G) == 0 and max_item_rows * (H // G) >= UMMA_PREFILL_MIN_ROWS):
        # tcgen05: 128 (token, head) rows a CTA, S and P V in tensor memory
        f = _fn("attention_umma", "fellm_attn_prefill_umma",
                [_c_p, _c_p, ctypes.c_longlong, _c_p, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_p, _c_int, _c_int, _c_int,
                 _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_p, _c_p])
        _check(f(_p(q), _p(pool), pool.shape[0], _p(block_table), block_table.shape[1], _p(positions), _p(row_slot),
                 _p(item_start), n_items, max_item_rows, _p(out), T, H, G, hd, page_tokens, layer, pool.shape[1],
                 float(scale), 0, _p(umma_status(q.device)), _stream()), "attention_prefill (tcgen05)")
        return out
    if USE_TMA_PREFILL and hd == 64 and page_tokens == 64 and not window and pool.numel() // hd < 2 ** 31:
        # a key tile is a page: K and V by bulk tensor copies
        f = _fn("attention_mma", "fellm_attn_prefill_tma",
                [_c_p, _c_p, ctypes.c_longlong, _c_p, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_p, _c_int, _c_int, _c_int,
                 _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_p, _c_p], defines={"HD": hd})
        _check(f(_p(q), _p(pool), pool.shape[0], _p(block_table), block_table.shape[1], _p(positions), _p(row_slot),
                 _p(item_start), n_items, max_item_rows, _p(out), T, H, G, hd, page_tokens, layer, pool.shape[1],
                 float(scale), 0, _p(umma_status(q.device)), _stream()), "attention_prefill (TMA)")
        return out
    f = _fn("attention_mma", "fellm_attn_prefill_mma",
            [_c_p, _c_p, _c_p, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_f, _c_int, _c_p], defines={"HD": hd})
    _check(f(_p(q), _p(pool), _p(block_table), block_table.shape[1], _p(positions), _p(row_slot), _p(item_start),
             n_items, max_item_rows, _p(out), T, H, G, hd, page_tokens, layer, pool.shape[1], float(scale),
             int(window or 0), _stream()), "attention_prefill")
    return out


def attention_prefill_general(qkv, H, pool, block_table, positions, row_slot, item_start, n_items, max_item_rows, layer,
                              scale, *, window=None, chunk=None, softcap=None, gate=None, slopes=None, q_temp=None,
                              values_are_keys=None, out=None):
    """Portions of prompts on tensor cores (bfloat16; keys and values of one size, the one the library is compiled
    for) with the part's soft cap, chunks and gate: q is read in place from rows [T, >= H*hd] (heads at column 0),
    gate float32 [T, >= H].  pool [pages, layers, 2, G, page_tokens, hd].  slopes float32 [H] and q_temp = (coef,
    every) as in paged_attention_general.  values_are_keys = (G, page_tokens, hd): the pool is [pages, layers,
    G * page_tokens * hd], keys alone, read as the values too."""
    _dev(qkv, pool, block_table, positions, row_slot, item_start, gate, slopes)
    T = qkv.shape[0]
    if values_are_keys:
        G, page_tokens, hd = values_are_keys
        assert pool.dim() == 3 and pool.shape[2] == G * page_tokens * hd
    else:
        G, page_tokens, hd = pool.shape[3], pool.shape[4], pool.shape[5]
    if slopes is not None:
        assert slopes.dtype == torch.float32 and slopes.numel() == H and slopes.is_contiguous()
    qt_coef, qt_every = q_temp if q_temp else (0.0, 0)
    if qkv.dtype != torch.bfloat16 or pool.dtype != torch.bfloat16 or hd % 16 or not 16 <= hd <= 256 or H % G or H // G > 64:
        raise KernelError("attention_prefill_general takes bfloat16, head sizes of a multiple of 16 in 16..256, up to 64 heads a kv head")
    assert qkv.stride(1) == 1 and qkv.stride(0) % 2 == 0 and pool.is_contiguous()
    _i32(block_table, "block_table"), _i32(positions, "positions"), _i32(row_slot, "row_slot"), _i32(item_start, "item_start")
    if gate is not None:
        assert gate.dtype == torch.float32 and gate.stride(1) == 1
    if out is None:
        out = torch.empty((T, H * hd), dtype=torch.bfloat16, device=qkv.device)
    f = _fn("attention_mma", "fellm_attn_prefill_mma_biased",
            [_c_p, _c_int, _c_p, _c_p, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_f, _c_int, _c_int, _c_f, _c_p, _c_int, _c_p, _c_f, _c_int, _c_int, _c_p], defines={"HD": hd})
    _check(f(_p(qkv), qkv.stride(0), _p(pool), _p(block_table), block_table.shape[1], _p(positions), _p(row_slot),
             _p(item_start), n_items, max_item_rows, _p(out), T, H, G, hd, page_tokens, layer, pool.shape[1], float(scale),
             int(window or 0), int(chunk or 0), float(softcap or 0.0), _p(gate), gate.stride(0) if gate is not None else 0,
             _p(slopes), float(qt_coef), int(qt_every), int(bool(values_are_keys)), _stream()), "attention_prefill_general")
    return out


def attention_modules(dtype: str, head_dim: int):
    mods = [("attention_simt", None)]
    if dtype == "bfloat16":
        mods.append(("attention_mma", {"HD": head_dim}))
        if head_dim == 64 and USE_UMMA_PREFILL:
            mods.append(("attention_umma", None))
    return mods


def paged_attention(q, cache, ctx, scale, window=None):
    """Attention of the step's rows over their items' cache pages; picks the kernel: the float32
    engine runs on CUDA cores; bfloat16 on tensor cores, split over the keys when every item
    brings one token."""
    if q.dtype == torch.bfloat16:
        if ctx.all_single:
            return attention_decode(q, cache.pool, cache.block_table, ctx.positions, ctx.row_slot, cache.layer,
                                    scale, window, ctx.max_len)
        return attention_prefill(q, cache.pool, cache.block_table, ctx.positions, ctx.row_slot, ctx.item_start,
                                 ctx.n_items, ctx.max_item_rows, cache.layer, scale, window)
    return paged_attention_simt(q, cache.pool, cache.block_table, ctx.positions, ctx.row_slot, cache.layer,
                                scale, window)


# ------------------------------------------------------------------------------ sampling

def sample_params_size() -> int:
    f = _fn("sampling", "fellm_sample_params_size", [])
    return int(f())


def sample(logits, params_dev, counts, bias_tok, bias_val, out_tokens, out_probs=None, update_counts=True):
    """One block per row of float32 logits [B, V]; params_dev: B packed records (see
    fellm_b200/sampling/sampler.py).  counts [slots, V] int32 or None."""
    _dev(logits, params_dev, counts, bias_tok, bias_val, out_tokens, out_probs)
    B, V = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous() and out_tokens.dtype == torch.int32
    if counts is not None:
        assert counts.dtype == torch.int32 and counts.shape[1] == V and counts.is_contiguous()
    f = _fn("sampling", "fellm_sample", [_c_p, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_p])
    _check(f(_p(logits), B, V, _p(params_dev), _p(counts), _p(bias_tok), _p(bias_val), _p(out_tokens),
             _p(out_probs), int(update_counts), _stream()), "sample")
    return out_tokens


def argmax_rows(logits, pval, pidx, out_tokens):
    """Greedy tokens of float32 logits [B, V], ties to the lower id; pval/pidx: scratch [B*64]."""
    _dev(logits, pval, pidx, out_tokens)
    B, V = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous() and pval.numel() >= B * 64 and pidx.numel() >= B * 64
    f = _fn("sampling", "fellm_argmax_rows", [_c_p, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p])
    _check(f(_p(logits), B, V, _p(pval), _p(pidx), _p(out_tokens), _stream()), "argmax_rows")
    return out_tokens


def count_tokens(counts, slots, tokens):
    _dev(counts, slots, tokens)
    _i32(slots, "slots"), _i32(tokens, "tokens")
    f = _fn("sampling", "fellm_count_tokens", [_c_p, _c_int, _c_p, _c_p, _c_int, _c_p])
    _check(f(_p(counts), counts.shape[1], _p(slots), _p(tokens), tokens.numel(), _stream()), "count_tokens")
