"""Launcher of the few-token fused product (csrc/gemv_fused.cu): a weight-streaming matrix product
for up to `MAX_TOKENS` rows that can take its input straight from the residual stream (RMSNorm
computed in the kernel) and finish its output itself (residual add, SwiGLU, or rotation plus the
cache write), so that a decode step launches five kernels a layer instead of nine.

`BARE_CUDA_B200_GEMV_MAX_TOKENS=0` switches the path off (every product then goes to the tcgen05
kernel)."""

from __future__ import annotations

import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Dict, Optional, Tuple

import torch

from . import build
from .lib import DT_BF16, DT_F32, AddTo, LazyNorm, Partials, Prenormed, RotateAndCache, _check, _ptr, sm_count

PRO_BF16, PRO_NORM, PRO_PRENORMED = 0, 1, 2
SQ_SLOTS = 32
EPI_STORE, EPI_ADD, EPI_SWIGLU, EPI_ROPE = 0, 1, 2, 3
MAX_TOKENS = int(os.environ.get("BARE_CUDA_B200_GEMV_MAX_TOKENS", "24"))     # measured: 24 rows still gain, 32 lose
_lib = None
_smem: Dict[Tuple[int, int], int] = {}


def lib():
    global _lib
    if _lib is None:
        l = build.load_library("gemv_fused.cu")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_gemv_fused_smem.argtypes = [I, I]
        l.llm_gemv_fused_smem.restype = L
        l.llm_gemv_fused.argtypes = [P, I, I, I, I, I, P, L, P, I, F, P, P, I, L, I, I, P, P, P, L, I, I, I, I,
                                     P, P, P, I, I, P, I, L, P, L, P, I, P, I, P, P]
        l.llm_gemv_fused.restype = c_int
        _lib = l
    return _lib


def supports(weight: torch.Tensor) -> bool:
    n, k = weight.shape
    return (MAX_TOKENS > 0 and weight.dtype == torch.bfloat16 and weight.is_cuda and weight.is_contiguous()
            and k % 32 == 0 and weight.data_ptr() % 16 == 0)


def smem_bytes(tokens: int, k: int) -> int:
    key = (-(-tokens // 8), k)
    if key not in _smem:
        _smem[key] = int(lib().llm_gemv_fused_smem(tokens, k))
    return _smem[key]


def takes(rows: int, k: int) -> bool:
    """Whether the kernel runs `rows` tokens against an inner dimension k (x must fit in shared memory)."""
    return 0 < rows <= MAX_TOKENS and smem_bytes(rows, k) > 0


def run(ctx, weight: torch.Tensor, x, rows: int, out_dtype: torch.dtype, buffer: str, swiglu: bool,
        epilogue) -> Optional[Partials]:
    """x[:rows] @ weight^T with the input and output forms the kernel fuses.  `x` is a bfloat16
    matrix or a `LazyNorm`; `epilogue` None, `AddTo` or `RotateAndCache`.  Returns the result, or
    None when the epilogue consumed it."""
    n, k = weight.shape
    sq_in, sq_items, sq_stride = None, 0, 0
    if isinstance(x, LazyNorm) and x.prenormed is not None:
        pre = x.prenormed
        pro, xt, x_stride, sq_in, sq_items, sq_stride = PRO_PRENORMED, pre.x, pre.x.stride(0), pre.sq, pre.items, pre.sq.stride(0)
        norm_w, eps, row_index, norm_code = None, x.eps, x.row_index, DT_F32
    elif isinstance(x, LazyNorm):
        pro, xt, x_stride = PRO_NORM, x.residual, x.residual.stride(0)
        norm_w, eps, row_index = x.weight, x.eps, x.row_index
        norm_code = DT_BF16 if norm_w.dtype == torch.bfloat16 else DT_F32
    else:
        pro, xt, x_stride, norm_w, eps, row_index, norm_code = PRO_BF16, x, x.stride(0), None, 0.0, None, DT_F32
    cache = None
    up_offset = q_heads = write_cache = 0
    positions = row_seq = inv_freq = None
    pre_x = pre_w = pre_sq = None
    if swiglu:
        epi, n_out, up_offset = EPI_SWIGLU, n // 2, n // 2
        out = ctx.ws.get(buffer, (rows, n_out), out_dtype)
    elif isinstance(epilogue, AddTo):
        epi, n_out, out = EPI_ADD, n, epilogue.residual
        if epilogue.then_norm is not None:
            pre_w = epilogue.then_norm.tensors["weight"]
            pre_x = ctx.ws.get("prenormed.x", (rows, n), torch.bfloat16, max_rows=MAX_TOKENS)
            pre_sq = ctx.ws.get("prenormed.sq", (-(-n // 16), SQ_SLOTS), torch.float32, max_rows=-(-n // 16))
    elif (isinstance(epilogue, RotateAndCache) and epilogue.cache.head_dim % 16 == 0
          and epilogue.cache.dtype == torch.bfloat16 and epilogue.q_out.dtype == torch.bfloat16):
        epi, n_out, out, cache = EPI_ROPE, n, epilogue.q_out, epilogue.cache
        positions, row_seq, inv_freq = epilogue.positions, epilogue.row_seq, epilogue.inv_freq
        q_heads, write_cache = epilogue.q_heads, 1 if epilogue.write_cache else 0
    else:
        epi, n_out = EPI_STORE, n
        out = ctx.ws.get(buffer, (rows, n), out_dtype)
    from . import gemm
    _check(lib().llm_gemv_fused(
        weight.data_ptr(), n, k, rows, pro, epi, xt.data_ptr(), x_stride, _ptr(norm_w), norm_code, eps,
        _ptr(row_index), out.data_ptr(), DT_BF16 if out.dtype == torch.bfloat16 else DT_F32, out.stride(0), n_out,
        up_offset, cache.k_ptr if cache else 0, cache.v_ptr if cache else 0,
        cache.block_table.data_ptr() if cache else 0, cache.page_stride if cache else 0,
        cache.table_stride if cache else 0, cache.page_tokens if cache else 1, cache.kv_heads if cache else 0,
        cache.head_dim if cache else 0, _ptr(positions), _ptr(row_seq), _ptr(inv_freq), q_heads, write_cache,
        _ptr(sq_in), sq_items, sq_stride, _ptr(pre_x), pre_x.stride(0) if pre_x is not None else 0, _ptr(pre_w),
        (DT_BF16 if pre_w.dtype == torch.bfloat16 else DT_F32) if pre_w is not None else DT_F32, _ptr(pre_sq),
        sm_count(), gemm.error_word(weight.device).data_ptr(), ctx.stream), "gemv_fused")
    ctx.prenormed = Prenormed(epilogue.then_norm, pre_x, pre_sq, -(-n // 16)) if pre_x is not None else None
    return None if epi in (EPI_ADD, EPI_ROPE) else Partials(out)
