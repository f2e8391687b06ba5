"""Python launchers for the engine's CUDA kernels.

Every function takes torch tensors that live on the GPU, checks what the kernel cannot check
for itself (device, contiguity, element type), and calls the kernel's `extern "C"` launcher
through ctypes on the current CUDA stream.  A non-zero status raises `KernelLaunchError`.
Nothing here computes on the CPU: without the compiled libraries the calls fail.
"""

from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from ..errors import KernelLaunchError
from . import build

DT_F32, DT_BF16 = 0, 1
_DTYPE_CODE = {torch.float32: DT_F32, torch.bfloat16: DT_BF16}

_STATUS_TEXT = {1: "element type not supported by this kernel", 2: "size not supported by this kernel",
                3: "pointer or stride not aligned as the kernel needs"}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelLaunchError(f"element type {dtype} is not supported (float32 or bfloat16)") from None


LAUNCHES = [0]   # launcher calls so far (each launches one kernel; the sampler launches two)


def _check(status: int, what: str) -> None:
    LAUNCHES[0] += 1
    if status == 0:
        return
    if status >= 2000:
        raise KernelLaunchError(f"{what}: CUDA driver error {status - 2000}")
    if status >= 1000:
        raise KernelLaunchError(f"{what}: CUDA runtime error {status - 1000}")
    raise KernelLaunchError(f"{what}: {_STATUS_TEXT.get(status, f'status {status}')}")


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _dev(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelLaunchError("kernel arguments must be CUDA tensors; the engine has no CPU path")


B200_SMS = 148     # what planning assumes where no device can be asked (host-only tests)
_sm_count = None


def sm_count() -> int:
    """Streaming multiprocessors of the current CUDA device, asked once."""
    global _sm_count
    if _sm_count is None:
        _sm_count = (torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
                     if torch.cuda.is_available() else B200_SMS)
    return _sm_count


def stream_handle() -> int:
    return torch.cuda.current_stream().cuda_stream


class CacheView:
    """What a kernel needs to address one cache (one run of a layer) inside its group's pool."""

    __slots__ = ("k_ptr", "v_ptr", "block_table", "page_stride", "table_stride", "page_tokens",
                 "kv_heads", "head_dim", "dtype", "pool_ptr", "pool_elems")

    def __init__(self, k_ptr, v_ptr, block_table, page_stride, table_stride, page_tokens, kv_heads,
                 head_dim, dtype, pool_ptr=0, pool_elems=0):
        self.pool_ptr, self.pool_elems = pool_ptr, pool_elems     # the group's whole storage (for TMA)
        self.k_ptr, self.v_ptr = k_ptr, v_ptr
        self.block_table = block_table
        self.page_stride, self.table_stride = page_stride, table_stride
        self.page_tokens, self.kv_heads, self.head_dim = page_tokens, kv_heads, head_dim
        self.dtype = dtype


class _Plain:
    def __init__(self):
        lib = build.load_library("plain_kernels.cu")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        lib.llm_embed_gather.argtypes = [P, I, P, P, I, I, P]
        lib.llm_add_rmsnorm.argtypes = [P, P, I, I, L, P, I, P, I, P, I, I, F, P]
        lib.llm_matmul_plain.argtypes = [P, I, P, I, P, I, I, I, I, L, L, P]
        lib.llm_rope_cache_write.argtypes = [P, I, I, L, P, I, P, P, P, L, I, I, I, I, P, P, P, I, I, I, P]
        lib.llm_attention_plain.argtypes = [P, P, I, P, P, P, L, I, I, I, I, P, P, I, I, F, I, P]
        lib.llm_swiglu.argtypes = [P, I, I, L, P, I, I, I, P]
        lib.llm_argmax_rows.argtypes = [P, P, I, I, P]
        lib.llm_sample_rows.argtypes = [P, P, P, P, I, I, P]
        for name in ("llm_embed_gather", "llm_add_rmsnorm", "llm_matmul_plain", "llm_rope_cache_write",
                     "llm_attention_plain", "llm_swiglu", "llm_argmax_rows", "llm_sample_rows"):
            getattr(lib, name).restype = c_int
        self.lib = lib


_plain: Optional[_Plain] = None


def plain() -> _Plain:
    global _plain
    if _plain is None:
        _plain = _Plain()
    return _plain


class Partials:
    """A result that may still be a sum: `n` partial results of identical shape stacked along the
    first axis of `tensor` ([n, rows, width]); n == 1 is a finished result.  Kernels that consume
    a projection (the norm's residual add, the rotation, SwiGLU) add the partials in index order,
    which lets a matrix product split its inner dimension over more thread blocks without a
    reduction pass of its own."""

    __slots__ = ("tensor", "n")

    def __init__(self, tensor: torch.Tensor, n: int = 1):
        self.tensor, self.n = tensor, n

    @property
    def stride(self) -> int:
        return self.tensor.stride(0) if self.n > 1 else 0

    @property
    def rows(self) -> int:
        return self.tensor.shape[-2]

    @property
    def width(self) -> int:
        return self.tensor.shape[-1]


class AddTo:
    """Asks a product to add its result into the float32 residual stream itself.  `then_norm`
    (optional) is the norm part that will read the stream next, if it is one whose factor is a
    single number per row (`prenormable`, with `tensors["weight"]` and `params["eps"]`): a kernel
    that can then also leaves bfloat16(new residual * weight) and the rows' sums of squares, from
    which the next product norms its input without reading the stream again (`Prenormed`)."""

    __slots__ = ("residual", "then_norm")

    def __init__(self, residual: torch.Tensor, then_norm=None):
        self.residual = residual
        self.then_norm = then_norm if getattr(then_norm, "prenormable", False) else None


class Prenormed:
    """What an adding product left for the norm `norm`: `x` [rows, width] bfloat16 = residual *
    weight, `sq` [items, 32] float32 parts of every row's sum of squares."""

    __slots__ = ("norm", "x", "sq", "items")

    def __init__(self, norm, x, sq, items):
        self.norm, self.x, self.sq, self.items = norm, x, sq, items


class RotateAndCache:
    """Asks the [q; k; v] product to rotate q and k by position, write q to `q_out` and put k and
    v into the cache (what `rope_cache_write` does as a kernel of its own)."""

    __slots__ = ("q_out", "cache", "positions", "row_seq", "inv_freq", "q_heads", "write_cache")

    def __init__(self, q_out, cache, positions, row_seq, inv_freq, q_heads, write_cache):
        self.q_out, self.cache, self.positions, self.row_seq = q_out, cache, positions, row_seq
        self.inv_freq, self.q_heads, self.write_cache = inv_freq, q_heads, write_cache


class LazyNorm:
    """rms_norm(residual rows) * weight that has not been computed: a product that can norm its
    own input takes it as it is, everything else calls `materialize()`."""

    __slots__ = ("ctx", "residual", "weight", "eps", "rows", "row_index", "buffer", "prenormed")

    def __init__(self, ctx, residual, weight, eps, rows, row_index, buffer, prenormed=None):
        self.ctx, self.residual, self.weight, self.eps = ctx, residual, weight, eps
        self.rows, self.row_index, self.buffer = rows, row_index, buffer
        self.prenormed = prenormed      # a `Prenormed` for this norm, if the last adding product left one

    def materialize(self) -> torch.Tensor:
        out = self.ctx.ws.get(self.buffer, (self.rows, self.residual.shape[-1]), self.ctx.dtype)
        add_rmsnorm(self.residual, None, self.weight, out, self.eps, self.rows, self.row_index, self.ctx.stream)
        return out


def materialize(h):
    return h.materialize() if isinstance(h, LazyNorm) else h


def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, n_tokens: int, stream=None) -> None:
    _dev(table, ids, out)
    _check(plain().lib.llm_embed_gather(table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(),
                                        out.data_ptr(), n_tokens, table.shape[1],
                                        stream if stream is not None else stream_handle()),
           "embed_gather")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[Partials], weight: torch.Tensor,
                out: Optional[torch.Tensor], eps: float, rows: int,
                row_index: Optional[torch.Tensor] = None, stream=None) -> None:
    """residual[r] += sum(delta partials)[r]; out[i] = rms_norm(residual[r]) * weight, r = row_index[i] or i."""
    _dev(residual, weight, out)
    hidden = residual.shape[-1]
    d_t = delta.tensor if delta is not None else None
    _check(plain().lib.llm_add_rmsnorm(
        residual.data_ptr(), _ptr(d_t), dtype_code(d_t.dtype) if d_t is not None else DT_F32,
        delta.n if delta is not None else 0, delta.stride if delta is not None else 0,
        weight.data_ptr(), dtype_code(weight.dtype), _ptr(out),
        dtype_code(out.dtype) if out is not None else DT_F32, _ptr(row_index), rows, hidden, eps,
        stream if stream is not None else stream_handle()), "add_rmsnorm")


def matmul_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, m: int, stream=None) -> None:
    """out[:m] = a[:m] @ w.T with w stored [out features, in features]."""
    _dev(a, w, out)
    n, k = w.shape
    if a.shape[-1] != k or out.shape[-1] != n or a.stride(-1) != 1 or out.stride(-1) != 1 or not w.is_contiguous():
        raise KernelLaunchError(f"matmul_plain: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _check(plain().lib.llm_matmul_plain(a.data_ptr(), dtype_code(a.dtype), w.data_ptr(), dtype_code(w.dtype),
                                        out.data_ptr(), dtype_code(out.dtype), m, n, k, a.stride(-2),
                                        out.stride(-2), stream if stream is not None else stream_handle()),
           "matmul_plain")


def rope_cache_write(qkv: Partials, q_out: torch.Tensor, cache: CacheView, positions: torch.Tensor,
                     row_seq: torch.Tensor, inv_freq: Optional[torch.Tensor], q_heads: int,
                     write_cache: bool, n_tokens: int, stream=None) -> None:
    _dev(qkv.tensor, q_out, positions, row_seq, inv_freq)
    _check(plain().lib.llm_rope_cache_write(
        qkv.tensor.data_ptr(), dtype_code(qkv.tensor.dtype), qkv.n, qkv.stride, q_out.data_ptr(),
        dtype_code(q_out.dtype), cache.k_ptr, cache.v_ptr, cache.block_table.data_ptr(), cache.page_stride,
        cache.table_stride, cache.page_tokens, cache.kv_heads, cache.head_dim, positions.data_ptr(),
        row_seq.data_ptr(), _ptr(inv_freq), q_heads, 1 if write_cache else 0, n_tokens,
        stream if stream is not None else stream_handle()), "rope_cache_write")


def attention_plain(q: torch.Tensor, out: torch.Tensor, cache: CacheView, positions: torch.Tensor,
                    row_seq: torch.Tensor, q_heads: int, n_tokens: int, scale: float, window: int,
                    stream=None) -> None:
    _dev(q, out, positions, row_seq)
    if q.dtype != out.dtype or q.dtype != cache.dtype:
        raise KernelLaunchError("attention_plain: q, out and the cache must share one element type")
    _check(plain().lib.llm_attention_plain(
        q.data_ptr(), out.data_ptr(), dtype_code(q.dtype), cache.k_ptr, cache.v_ptr,
        cache.block_table.data_ptr(), cache.page_stride, cache.table_stride, cache.page_tokens,
        cache.kv_heads, cache.head_dim, positions.data_ptr(), row_seq.data_ptr(), q_heads, n_tokens,
        scale, window, stream if stream is not None else stream_handle()), "attention_plain")


def swiglu(gate_up: Partials, out: torch.Tensor, n_tokens: int, stream=None) -> None:
    _dev(gate_up.tensor, out)
    inter = out.shape[-1]
    _check(plain().lib.llm_swiglu(gate_up.tensor.data_ptr(), dtype_code(gate_up.tensor.dtype), gate_up.n,
                                  gate_up.stride, out.data_ptr(), dtype_code(out.dtype), n_tokens, inter,
                                  stream if stream is not None else stream_handle()), "swiglu")


def argmax_rows(logits: torch.Tensor, out: torch.Tensor, rows: int, stream=None) -> None:
    _dev(logits, out)
    _check(plain().lib.llm_argmax_rows(logits.data_ptr(), out.data_ptr(), rows, logits.shape[-1],
                                       stream if stream is not None else stream_handle()), "argmax_rows")


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
                out: torch.Tensor, rows: int, stream=None) -> None:
    _dev(logits, temperature, uniform, out)
    _check(plain().lib.llm_sample_rows(logits.data_ptr(), temperature.data_ptr(), uniform.data_ptr(),
                                       out.data_ptr(), rows, logits.shape[-1],
                                       stream if stream is not None else stream_handle()), "sample_rows")
