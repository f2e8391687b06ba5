"""Launcher of the paged attention kernels: csrc/attention_mma.cu (every head size and batch
shape), csrc/attention_tcgen05.cu (prompt portions, head sizes 64 and 128) and
csrc/attention_decode.cu (steps of very few tokens per request, head sizes 64 and 128); one
library per head size, the per-step list of row tiles, and the choice of how many thread blocks
split a tile's keys."""

from __future__ import annotations

import ctypes
import math
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Dict, Optional

import numpy as np
import torch

from . import build
from ..errors import KernelLaunchError
from .lib import CacheView, _check, sm_count

KEY_BLOCK = 64
COUNTER_WORDS = 4096          # per-tile split counters at the start of the scratch (see the kernel)
_libs: Dict[int, object] = {}
_tc_libs: Dict[int, object] = {}
_decode_libs: Dict[int, object] = {}
TC_HEAD_DIMS = (64, 128)      # head sizes the tcgen05 prefill kernel and the decode kernel are built for
DECODE_MAX_TILES = 65535 // 4 # (tiles x kv heads) up to which the cluster decode kernel runs


def supports(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 128


def defines(head_dim: int):
    return (f"-DHEAD_DIM={head_dim}",)


def lib(head_dim: int):
    l = _libs.get(head_dim)
    if l is None:
        l = build.load_library("attention_mma.cu", defines(head_dim))
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_attention_mma.argtypes = [P, P, P, P, P, L, I, I, I, I, P, P, P, P, P, I, I, I, P, I, F, I, P]
        l.llm_attention_mma.restype = c_int
        l.llm_attention_scratch_floats.argtypes = [I, I, I, I]
        l.llm_attention_scratch_floats.restype = c_longlong
        l.llm_attention_prefill_rows.restype = c_int
        _libs[head_dim] = l
    return l


def tc_lib(head_dim: int):
    """The tcgen05 prefill kernel's library for this head size."""
    l = _tc_libs.get(head_dim)
    if l is None:
        l = build.load_library("attention_tcgen05.cu", defines(head_dim))
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_attention_tcgen05.argtypes = [P, P, I, P, P, P, P, P, L, I, I, I, I, P, P, P, P, P, I, I, F, I, P, P]
        l.llm_attention_tcgen05.restype = c_int
        l.llm_attention_tc_pool_map.argtypes = [P, P, L, I]
        l.llm_attention_tc_pool_map.restype = c_int
        l.llm_attention_tc_rows.restype = c_int
        _tc_libs[head_dim] = l
    return l


def decode_lib(head_dim: int):
    """The cluster decode kernel's library for this head size."""
    l = _decode_libs.get(head_dim)
    if l is None:
        l = build.load_library("attention_decode.cu", defines(head_dim))
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_attention_decode.argtypes = [P, P, L, I, P, P, P, P, P, L, I, I, I, I, P, P, P, P, P, I, I, I, I, F, I, P, P]
        l.llm_attention_decode.restype = c_int
        l.llm_attention_decode_pool_map.argtypes = [P, P, L, I]
        l.llm_attention_decode_pool_map.restype = c_int
        l.llm_attention_decode_key_block.restype = c_int
        l.key_block = int(l.llm_attention_decode_key_block())
        _decode_libs[head_dim] = l
    return l


class AttentionPlan:
    def __init__(self, head_dim: int, heads: int, kv_heads: int):
        self.head_dim, self.heads, self.kv_heads = head_dim, heads, kv_heads
        self.group = heads // kv_heads
        self.lib = lib(head_dim)
        self.prefill_rows = int(self.lib.llm_attention_prefill_rows())
        self.tc = None
        if head_dim in TC_HEAD_DIMS:
            self.tc = tc_lib(head_dim)
            self.prefill_rows = int(self.tc.llm_attention_tc_rows())
        self.decode = None
        if head_dim in TC_HEAD_DIMS and not os.environ.get("BARE_CUDA_B200_NO_DECODE_ATTENTION"):
            self.decode = decode_lib(head_dim)
        self._host = None
        self._dev = None
        self._scratch = None
        self._pool_maps = {}
        self._decode_maps = {}

    def decode_map(self, cache: CacheView):
        """The decode kernel's tensor map over a cache group's pool (boxes of at most 64 rows)."""
        box_rows = math.gcd(self.decode.key_block, cache.page_tokens)
        key = (cache.pool_ptr, cache.pool_elems, box_rows)
        m = self._decode_maps.get(key)
        if m is None:
            m = (ctypes.c_ubyte * 128)()
            _check(self.decode.llm_attention_decode_pool_map(ctypes.addressof(m), cache.pool_ptr,
                                                             cache.pool_elems // self.head_dim, box_rows),
                   "attention decode pool map")
            self._decode_maps[key] = m
        return m, box_rows

    def decode_usable(self, cache: CacheView) -> bool:
        return self.decode is not None and cache.pool_ptr != 0 and math.gcd(self.decode.key_block, cache.page_tokens) >= 8

    def pool_map(self, cache: CacheView):
        """The TMA tensor map over a cache group's whole pool (one per pool) and its box height."""
        box_rows = math.gcd(128, cache.page_tokens)
        key = (cache.pool_ptr, cache.pool_elems, box_rows)
        m = self._pool_maps.get(key)
        if m is None:
            m = (ctypes.c_ubyte * 128)()
            _check(self.tc.llm_attention_tc_pool_map(ctypes.addressof(m), cache.pool_ptr,
                                                     cache.pool_elems // self.head_dim, box_rows), "attention pool map")
            self._pool_maps[key] = m
        return m, box_rows

    def tc_usable(self, cache: CacheView) -> bool:
        return self.tc is not None and cache.pool_ptr != 0 and math.gcd(128, cache.page_tokens) >= 8

    def buffers(self, ctx, n: int, device):
        """A pinned and the device int32 buffer for the tile list, sized once for the largest step
        so that the device address never changes (captured CUDA graphs keep it).  The pinned side
        is one of four taken in turn; `sent()` records the event that guards its reuse (the copy
        reads pinned memory when the GPU gets to it, possibly after the host has begun another step)."""
        if self._host is None or self._host[0].numel() < 2 * n:
            most = -(-ctx.max_rows * self.group // 64) + ctx.max_seqs + 8
            cap = 2 * max(n, most)
            self._host = [torch.empty(cap, dtype=torch.int32).pin_memory() for _ in range(4)]
            self._host_events = [None] * 4
            self._host_turn = 0
            self._dev = torch.empty(cap, dtype=torch.int32, device=device)
        self._host_turn = (self._host_turn + 1) % 4
        if self._host_events[self._host_turn] is not None:
            self._host_events[self._host_turn].synchronize()
        return self._host[self._host_turn], self._dev

    def sent(self) -> None:
        if self._host_events[self._host_turn] is None:
            self._host_events[self._host_turn] = torch.cuda.Event()
        self._host_events[self._host_turn].record()

    def scratch(self, ctx, floats: int, device) -> torch.Tensor:
        """Scratch for split keys; a split step has at most (2 * sm_count()) + tiles * kv_heads items."""
        if self._scratch is None or self._scratch.numel() < floats:
            most = COUNTER_WORDS + ((2 * sm_count()) + (ctx.max_seqs + 8) * self.kv_heads) * 16 * (self.head_dim + 1)
            self._scratch = torch.zeros(max(floats, most), dtype=torch.float32, device=device)   # counters start at zero
        return self._scratch


def plan_for(head_dim: int, heads: int, kv_heads: int) -> Optional[AttentionPlan]:
    if not supports(head_dim):
        return None
    return AttentionPlan(head_dim, heads, kv_heads)


def step_tiles(ctx, plan: AttentionPlan):
    """The step's row tiles for this head grouping: built once per step and shared by all layers."""
    key = ("attention_tiles", plan.group, plan.kv_heads, plan.head_dim)
    cached = ctx.extras.get(key)
    if cached is not None:
        return cached
    g = plan.group
    rows_per_tile = 16 if ctx.max_q_len * g <= 16 else plan.prefill_rows
    counts = [-(-q * g // rows_per_tile) for q in ctx.host_q_len]
    pad = ctx.pad_seqs if rows_per_tile == 16 else 0     # padded decode steps keep a fixed grid
    n_tiles = sum(counts) + pad
    host, dev = plan.buffers(ctx, n_tiles, ctx.token_ids.device)
    h = host.numpy()
    at = 0
    for s, c in enumerate(counts):
        h[at: at + c] = s
        h[n_tiles + at: n_tiles + at + c] = np.arange(c, dtype=np.int32)
        at += c
    h[at: n_tiles] = -1
    h[n_tiles + at: 2 * n_tiles] = 0
    dev[: 2 * n_tiles].copy_(host[: 2 * n_tiles], non_blocking=True)
    plan.sent()
    n_splits = 1
    use_decode = rows_per_tile == 16 and plan.decode is not None and n_tiles * plan.kv_heads <= DECODE_MAX_TILES
    if rows_per_tile == 16 and not use_decode:
        key_blocks = -(-ctx.max_kv_len // KEY_BLOCK)
        n_splits = max(1, min(key_blocks, -(-(2 * sm_count()) // (n_tiles * plan.kv_heads))))
        if os.environ.get("BARE_CUDA_B200_ATTN_SPLITS"):     # experiments only
            n_splits = min(key_blocks, int(os.environ["BARE_CUDA_B200_ATTN_SPLITS"]))
        if n_tiles * plan.kv_heads > COUNTER_WORDS:
            n_splits = 1
    dec_splits = dec_slots = 0
    if use_decode:
        # The cluster decode kernel: up to 8 blocks of 4 warps share a tile, a warp keeps one key
        # block in flight.  Measured at a context of 2,048 (batches 8 to 64): the kernel is fastest
        # with about two blocks per SM in all, and with a power of two of them per tile (batch 64:
        # 26.7 us with one block per tile, 32 with two or four; batch 32: 13.4 us with two, 20.9 / 16.1 with
        # one / four; batch 16: 8.5 us with four, 12.1 / 12.6 with two / eight).  The number does not depend
        # on the context length (a short context leaves some warps without a key block), so a captured
        # graph of the step stays valid while the requests grow.
        dec_splits = 1
        while dec_splits < 8 and n_tiles * plan.kv_heads * dec_splits * 2 <= 2 * sm_count():
            dec_splits *= 2
        dec_slots = 1
        if os.environ.get("BARE_CUDA_B200_ATTN_SPLITS"):     # experiments only
            dec_splits = max(1, min(8, int(os.environ["BARE_CUDA_B200_ATTN_SPLITS"])))
    out = (dev[:n_tiles], dev[n_tiles: 2 * n_tiles], n_tiles, rows_per_tile, n_splits, dec_splits, dec_slots)
    ctx.extras[key] = out
    return out


def run(ctx, plan: AttentionPlan, q: torch.Tensor, out: torch.Tensor, cache: CacheView, scale: float,
        window: int) -> None:
    tile_seq, tile_index, n_tiles, rows_per_tile, n_splits, dec_splits, dec_slots = step_tiles(ctx, plan)
    if dec_splits and plan.decode_usable(cache):
        from . import gemm
        pool_map, box_rows = plan.decode_map(cache)
        _check(plan.decode.llm_attention_decode(
            ctypes.addressof(pool_map), cache.pool_ptr, cache.pool_elems // plan.head_dim, box_rows, q.data_ptr(),
            out.data_ptr(), cache.k_ptr, cache.v_ptr, cache.block_table.data_ptr(), cache.page_stride,
            cache.table_stride, cache.page_tokens, cache.kv_heads, cache.head_dim, ctx.seq_q_start.data_ptr(),
            ctx.seq_q_len.data_ptr(), ctx.seq_kv_len.data_ptr(), tile_seq.data_ptr(), tile_index.data_ptr(), n_tiles,
            dec_splits, dec_slots, plan.heads, scale, window, gemm.error_word(q.device).data_ptr(), ctx.stream),
            "attention_decode")
        return
    if plan.tc is not None and rows_per_tile != 16:
        if not plan.tc_usable(cache):
            raise KernelLaunchError(f"attention_tcgen05: cache pages of {cache.page_tokens} positions are not supported "
                                    "(the page size must share a factor of at least 8 with 128)")
        from . import gemm
        pool_map, box_rows = plan.pool_map(cache)
        _check(plan.tc.llm_attention_tcgen05(
            ctypes.addressof(pool_map), cache.pool_ptr, box_rows, q.data_ptr(), out.data_ptr(), cache.k_ptr, cache.v_ptr, cache.block_table.data_ptr(), cache.page_stride,
            cache.table_stride, cache.page_tokens, cache.kv_heads, cache.head_dim, ctx.seq_q_start.data_ptr(),
            ctx.seq_q_len.data_ptr(), ctx.seq_kv_len.data_ptr(), tile_seq.data_ptr(), tile_index.data_ptr(), n_tiles,
            plan.heads, scale, window, gemm.error_word(q.device).data_ptr(), ctx.stream), "attention_tcgen05")
        return
    scratch_ptr = 0
    if n_splits > 1:
        floats = plan.lib.llm_attention_scratch_floats(n_tiles, plan.kv_heads, n_splits, rows_per_tile)
        scratch_ptr = plan.scratch(ctx, int(floats), q.device).data_ptr()
    _check(plan.lib.llm_attention_mma(
        q.data_ptr(), out.data_ptr(), cache.k_ptr, cache.v_ptr, cache.block_table.data_ptr(), cache.page_stride,
        cache.table_stride, cache.page_tokens, cache.kv_heads, cache.head_dim, ctx.seq_q_start.data_ptr(),
        ctx.seq_q_len.data_ptr(), ctx.seq_kv_len.data_ptr(), tile_seq.data_ptr(), tile_index.data_ptr(), n_tiles,
        rows_per_tile, n_splits, scratch_ptr, plan.heads, scale, window, ctx.stream), "attention_mma")
