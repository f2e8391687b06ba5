"""Launcher of the tcgen05 bfloat16 matrix product (csrc/gemm_tcgen05.cu): tensor maps, choice of
the token tile and of the K split, and the device error word that bounded waits report to."""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Dict, Optional, Tuple

import torch

from ..errors import KernelLaunchError
from . import build
from .lib import DT_BF16, DT_F32, AddTo, LazyNorm, Partials, Prenormed, _check, _ptr, sm_count

BM, BK = 128, 64
SPLIT_MAX_ROWS = 256          # steps with more rows never split K
_lib = None
_error_word: Optional[torch.Tensor] = None


def lib():
    global _lib
    if _lib is None:
        l = build.load_library("gemm_tcgen05.cu")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_gemm_tensor_map.argtypes = [P, P, L, L, L, I]
        l.llm_gemm_tensor_map.restype = c_int
        l.llm_gemm_bf16.argtypes = [P, P, P, I, I, I, I, L, L, I, I, I, I, I, I, P, I, L, F, F, P, L, P, I, P, L, P, P]
        l.llm_gemm_bf16.restype = c_int
        _lib = l
    return _lib


def error_word(device) -> torch.Tensor:
    global _error_word
    if _error_word is None:
        _error_word = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_word


def check_errors() -> None:
    """Reads the device error word (synchronises); raises if a kernel gave up on a wait."""
    if _error_word is not None:
        code = int(_error_word.item())
        if code:
            _error_word.zero_()
            role = {1: "gemm TMA producer", 2: "gemm MMA issuer", 3: "gemm epilogue", 11: "attention loader",
                    12: "attention MMA issuer", 13: "attention softmax",
                    14: "attention (shared memory not 1024-byte aligned)", 21: "few-token product, producer",
                    22: "few-token product, consumer", 31: "decode attention"}.get(code, f"code {code}")
            raise KernelLaunchError(f"a kernel gave up ({role}): a bounded wait ran out; the result is invalid")


def supports(weight: torch.Tensor) -> bool:
    n, k = weight.shape
    return (weight.dtype == torch.bfloat16 and weight.is_cuda and weight.is_contiguous()
            and k % 8 == 0 and weight.data_ptr() % 16 == 0)


def tensor_map(base_ptr: int, rows: int, cols: int, row_stride: int, box_rows: int) -> ctypes.Array:
    buf = (ctypes.c_ubyte * 128)()
    _check(lib().llm_gemm_tensor_map(ctypes.addressof(buf), base_ptr, rows, cols, row_stride, box_rows),
           "gemm tensor map")
    return buf


class GemmPlan:
    """A weight matrix ready for the kernel: its tensor map and the maps of the activation buffers
    it has been multiplied with."""

    def __init__(self, weight: torch.Tensor):
        self.weight = weight
        self.n, self.k = weight.shape
        self.weight_maps: Dict[int, ctypes.Array] = {}
        self.map_w = self.weight_map(BM)
        self.act_maps: Dict[Tuple[int, int, int], ctypes.Array] = {}

    def weight_map(self, box_rows: int) -> ctypes.Array:
        m = self.weight_maps.get(box_rows)
        if m is None:
            m = tensor_map(self.weight.data_ptr(), self.n, self.k, self.k, box_rows)
            self.weight_maps[box_rows] = m
        return m

    def act_map(self, a: torch.Tensor, bn: int) -> ctypes.Array:
        """`bn`: rows of the box (the token tile)."""
        key = (a.data_ptr(), bn, a.stride(0))
        m = self.act_maps.get(key)
        if m is None:
            esize = a.element_size()
            storage_left = a.untyped_storage().nbytes() - a.storage_offset() * esize
            capacity = max(a.shape[0], storage_left // (a.stride(0) * esize))
            m = tensor_map(a.data_ptr(), capacity, self.k, a.stride(0), bn)
            self.act_maps[key] = m
        return m


def plan_for(weight: torch.Tensor) -> Optional[GemmPlan]:
    if not supports(weight):
        return None
    return GemmPlan(weight)


def token_tile(rows: int) -> int:
    for bn in (16, 32, 64, 128):
        if rows <= bn:
            return bn
    # beyond 128 rows the tile follows the row count in steps of 16: a step of 129 to 160 rows ran a tenth
    # faster than with a tile of 256 tokens, most of which were padding
    return min(256, -(-rows // 16) * 16)


def choose_splits(rows: int, n: int, k: int, bn: int) -> int:
    """How many thread blocks share the K range of one output tile: enough to put about two
    blocks on every SM, at least four 64-wide K blocks each, and partial results (float32, written
    and read back through the L2 cache, not HBM) of at most about the weight's own bytes."""
    if rows > SPLIT_MAX_ROWS:
        return 1
    tiles = -(-n // BM) * -(-rows // bn)
    k_blocks = -(-k // BK)
    splits = min(k_blocks // 4, (2 * sm_count()) // tiles, max(1, k // (4 * rows)))
    splits = max(1, splits)
    per = -(-k_blocks // splits)
    return -(-k_blocks // per)


def max_splits(n: int, k: int) -> int:
    """The most blocks `choose_splits` ever puts on one output tile of an [n, k] weight, whatever
    the number of rows: the scratch for partial results is sized for it once, so that its address
    never changes under a captured graph."""
    return max(1, min(-(-k // BK) // 4, (2 * sm_count()) // -(-n // BM)))


TOKENS_ON_ROWS_ABOVE = 240    # steps with more rows put 128 tokens on the MMA rows (orientation 1); measured: a step
                              # of 256 rows takes 2.32 ms that way and 2.53 ms with the weights on the MMA rows, one of 224 rows 2.5 and 2.23
# The SwiGLU product changes over earlier: with the weights on the MMA rows a block holds only 64
# outputs, so from about a hundred tokens on the other orientation's wider tiles measured faster
# (TinyLlama's feed-forward at 128 / 256 tokens: 16 / 19 us against 23 / 48 us; at 48 / 64 / 80 / 96 tokens 16.3 us
# that way, whatever the count, against 14.9 / 16.8 / 18.5 / 20.2 us).
SWIGLU_TOKENS_ON_ROWS_ABOVE = 60


def feature_tile(rows: int, n_out: int, swiglu: bool) -> int:
    """Orientation 1: how many weight rows a tile takes (a multiple of 16 up to 256; of 32 with
    SwiGLU, whose tile is half gate rows and half up rows).  Every SM works through
    ceil(tiles / SMs) tiles and a tile's time grows with its width, so the product of the two is
    minimised; a small fixed cost per tile breaks ties towards wider tiles.  Wide tiles (192 rows
    and more) of a product with more tiles than SMs run in the persistent kernel, whose tiles
    measured about an eighth cheaper (no pipeline refill per tile, the epilogue off the critical path)."""
    forced = os.environ.get("BARE_CUDA_B200_GEMM_BN")     # experiments only
    if forced:
        return int(forced)
    step = 32 if swiglu else 16
    best, best_cost = 256, None
    for bn in range(256, 63, -step):
        # between 160 and 256 a tile is too big for two blocks per SM with three stages each, yet
        # more than one tile per SM needs that overlap: only SwiGLU tiles (two stages) use the range
        if not swiglu and 160 < bn < 256:
            continue
        out_per_tile = bn // 2 if swiglu else bn
        tiles = -(-rows // BM) * -(-n_out // out_per_tile)
        cost = -(-tiles // sm_count()) * (bn / 256.0 + 0.12)
        if bn >= 192 and tiles > sm_count():
            cost *= 0.88
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = bn, cost
    return best


NO_EXTRA = (0, 0, 0, 0.0, 0.0, 0, 0, 0, 0, 0, 0)     # no row factor on the way in, nothing prepared on the way out


def takes_prenormed(rows: int, swiglu: bool) -> bool:
    """Whether a step of `rows` rows runs in the orientation whose epilogue can apply a norm's
    factor per row (tokens on the MMA rows), so that the product can take a `LazyNorm` that a
    product before it prepared."""
    return rows > (SWIGLU_TOKENS_ON_ROWS_ABOVE if swiglu else TOKENS_ON_ROWS_ABOVE)


def run(ctx, plan: GemmPlan, a, rows: int, out_dtype: torch.dtype, buffer: str,
        allow_partials: bool, swiglu: bool, epilogue=None) -> Optional[Partials]:
    """`a`: a bfloat16 matrix, or a `LazyNorm` whose `prenormed` a product before this one left
    (`takes_prenormed` steps only).  `epilogue`: with an `AddTo` whose norm can be prepared, a
    many-token step adds the product into the float32 residual stream itself, leaves bfloat16(new
    residual * that norm's weight) and the rows' sums of squares for the product that reads the
    norm next (`ctx.prenormed`), and None comes back; otherwise the plain result comes back and the
    epilogue stays the caller's."""
    extra_in = NO_EXTRA[:5]
    if isinstance(a, LazyNorm):
        pre = a.prenormed
        if pre is None or a.row_index is not None or not takes_prenormed(rows, swiglu):
            a = a.materialize()
        else:
            extra_in = (pre.sq.data_ptr(), pre.items, pre.sq.stride(0), float(pre.x.shape[-1]), a.eps)
            a = pre.x
    ctx.prenormed = None
    if a.dtype != torch.bfloat16 or a.stride(-1) != 1 or a.shape[-1] != plan.k or a.data_ptr() % 16 or a.stride(0) % 8:
        raise KernelLaunchError(f"gemm_tcgen05: activations {tuple(a.shape)} {a.dtype} do not fit weight "
                                f"[{plan.n}, {plan.k}]")
    err = error_word(a.device)
    l = lib()
    code = DT_BF16 if out_dtype == torch.bfloat16 else DT_F32
    if takes_prenormed(rows, swiglu):
        n_out = plan.n // 2 if swiglu else plan.n
        bn = feature_tile(rows, n_out, swiglu)
        extra_out = NO_EXTRA[5:]
        out, then = None, None
        if (isinstance(epilogue, AddTo) and epilogue.then_norm is not None and not swiglu
                and epilogue.residual.dtype == torch.float32 and epilogue.residual.shape[-1] == n_out
                and epilogue.residual.stride(-1) == 1 and epilogue.residual.stride(0) % 4 == 0 and n_out % 4 == 0
                and epilogue.residual.data_ptr() % 16 == 0):
            then = epilogue.then_norm
            pre_w = then.tensors["weight"]
            if pre_w.is_cuda and pre_w.data_ptr() % 16 == 0 and pre_w.dtype in (torch.float32, torch.bfloat16):
                out = epilogue.residual
                f_tiles = -(-n_out // bn)
                pre_x = ctx.ws.get("prenormed.rows.x", (rows, n_out), torch.bfloat16)
                # one row of parts per feature tile (a tile is at least 64 wide), as long as the largest step
                most_tiles = -(-n_out // 64)
                pre_sq = ctx.ws.get("prenormed.rows.sq", (most_tiles, ctx.ws.max_rows), torch.float32, max_rows=most_tiles)
                extra_out = (pre_x.data_ptr(), pre_x.stride(0), pre_w.data_ptr(),
                             DT_BF16 if pre_w.dtype == torch.bfloat16 else DT_F32, pre_sq.data_ptr(), pre_sq.stride(0))
        fused = out is not None
        if not fused:
            out = ctx.ws.get(buffer, (rows, n_out), out_dtype)
        _check(l.llm_gemm_bf16(ctypes.addressof(plan.weight_map(bn // 2 if swiglu else bn)),
                               ctypes.addressof(plan.act_map(a, BM)), out.data_ptr(), DT_F32 if fused else code, rows,
                               n_out, plan.k, out.stride(0), 0, 1, bn, 1 if swiglu else 0, 1, n_out if swiglu else 0,
                               1 if fused else 0, *extra_in, *extra_out, err.data_ptr(), ctx.stream),
               "gemm_tcgen05 (tokens on rows)")
        if fused:
            ctx.prenormed = Prenormed(then, pre_x, pre_sq, f_tiles)
            return None
        return Partials(out)
    bn = token_tile(rows)
    if swiglu:
        inter = plan.n // 2
        out = ctx.ws.get(buffer, (rows, inter), out_dtype)
        if -(-inter // (BM // 2)) * -(-rows // bn) >= sm_count():
            # 64 gate rows and the matching 64 up rows share a block's 128 MMA rows: SwiGLU in the
            # epilogue and no partial results, when that alone gives every SM a block
            _check(l.llm_gemm_bf16(ctypes.addressof(plan.weight_map(BM // 2)), ctypes.addressof(plan.act_map(a, bn)),
                                   out.data_ptr(), code, rows, inter, plan.k, out.stride(0), 0, 1, bn, 1, 0, inter, 0,
                                   *NO_EXTRA, err.data_ptr(), ctx.stream), "gemm_tcgen05 (swiglu)")
            return Partials(out)
        # a narrow feed-forward: stream [gate; up] as one product split over K so that every SM takes
        # part, and add the partial results inside the SwiGLU kernel
        from . import lib as K
        full = run(ctx, plan, a, rows, torch.float32, buffer + ".gate_up", True, False)
        K.swiglu(full, out, rows, ctx.stream)
        return Partials(out)
    splits = choose_splits(rows, plan.n, plan.k, bn) if (allow_partials and out_dtype == torch.float32) else 1
    if splits > 1:
        out = ctx.ws.get(buffer + ".partials", (splits, rows, plan.n), torch.float32, max_rows=SPLIT_MAX_ROWS,
                         max_lead=max_splits(plan.n, plan.k))
        stride = out.stride(0)
    else:
        out = ctx.ws.get(buffer, (rows, plan.n), out_dtype)
        stride = 0
    _check(l.llm_gemm_bf16(ctypes.addressof(plan.map_w), ctypes.addressof(plan.act_map(a, bn)), out.data_ptr(),
                           DT_BF16 if out_dtype == torch.bfloat16 else DT_F32, rows, plan.n, plan.k,
                           out.stride(-2), stride, splits, bn, 0, 0, 0, 0, *NO_EXTRA, err.data_ptr(), ctx.stream),
           "gemm_tcgen05")
    return Partials(out, splits)
