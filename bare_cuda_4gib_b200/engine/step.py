"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A batch may hold portions of prompts beside single decoded tokens, cut anywhere; each request's
tokens are appended after what it has cached, the step runs only the tokens it is given, and
logits come back only for the places that were asked for
(cuongvng/bare-cuda-4gib accepts the same batches mechanically in Model::forward_rows,
engine/src/model.cpp:452-616, but computes logits for every row and never mixes).

Per step the host builds one block of int32 metadata in pinned memory - token ids, positions,
the batch sequence of every row, wanted rows, per-sequence lengths, and every cache group's
block-table rows - and sends it with one asynchronous copy.  Kernels read all variable data
from that block, so a step of the same padded shape can be replayed as a CUDA graph.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..errors import EngineError
from ..parts.base import CallContext


@dataclass
class StepEntry:
    """One request's share of a step: its slot, its next tokens and the places among them whose
    logits are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class Workspace:
    """Named activation buffers, allocated once for the largest step and handed out as views."""

    def __init__(self, device, max_rows: int):
        self.device, self.max_rows = device, max_rows
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}

    def get(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype, max_rows: Optional[int] = None) -> torch.Tensor:
        """A [rows, width] (or [n, rows, width]) view; the rows axis is sized for the largest step
        (or for `max_rows` when the caller only uses the buffer for small steps)."""
        rows_axis = len(shape) - 2
        full = list(shape)
        full[rows_axis] = max(min(self.max_rows, max_rows) if max_rows else self.max_rows, shape[rows_axis])
        need = int(np.prod(full))
        key = (name, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < need:
            buf = torch.empty(need, dtype=dtype, device=self.device)
            self._buffers[key] = buf
        view = buf[:need].view(full)
        return view[: shape[0]] if rows_axis == 0 else view[:, : shape[1]]

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


class StepContext:
    """What the parts see of a step."""

    def __init__(self):
        self.n_tokens = 0
        self.n_seqs = 0
        self.n_want = 0
        self.dtype = torch.float32
        self.stream = 0
        self.ws: Optional[Workspace] = None
        self.token_ids = self.positions = self.row_seq = self.want_rows = None
        self.seq_slot = self.seq_q_start = self.seq_q_len = self.seq_kv_len = None
        self.calls: List[CallContext] = []
        self.use_fast_gemm = True
        self.use_fast_attention = True
        # host copies, for parts that plan their launches from the batch's shape
        self.host_q_len: List[int] = []
        self.host_kv_len: List[int] = []
        self.max_q_len = 0
        self.max_kv_len = 0
        self.extras: Dict[str, object] = {}


class StepRunner:
    def __init__(self, model, cache: CacheManager, *, max_step_tokens: int, max_batch_seqs: Optional[int] = None,
                 use_fast_gemm: bool = True, use_fast_attention: bool = True, use_cuda_graphs: bool = True):
        if model.device is None or model.device.type != "cuda":
            raise EngineError("the step function needs a model bound on a CUDA device; there is no CPU path")
        self.model, self.cache = model, cache
        self.device = model.device
        self.max_step_tokens = int(max_step_tokens)
        self.max_batch_seqs = int(max_batch_seqs or cache.max_seqs)
        self.vocab = model.spec.vocab_size
        self.ws = Workspace(self.device, self.max_step_tokens)
        T, S, P, G = self.max_step_tokens, self.max_batch_seqs, cache.max_blocks, len(cache.groups)
        self._sizes = (T, S, P, G)
        total = 4 * T + 4 * S + G * S * P
        self._host = torch.empty(total, dtype=torch.int32).pin_memory()
        self._host_np = self._host.numpy()
        self._dev = torch.empty(total, dtype=torch.int32, device=self.device)
        self.ctx = StepContext()
        self.ctx.ws = self.ws
        self.ctx.dtype = model.dtype
        self.ctx.use_fast_gemm, self.ctx.use_fast_attention = use_fast_gemm, use_fast_attention
        off = 0

        def take(n):
            nonlocal off
            view = (self._host_np[off: off + n], self._dev[off: off + n])
            off += n
            return view

        self._token_ids, self._positions, self._row_seq, self._want = take(T), take(T), take(T), take(T)
        self._seq_slot, self._seq_q_start, self._seq_q_len, self._seq_kv_len = take(S), take(S), take(S), take(S)
        self._tables = []
        for _ in range(G):
            h, d = take(S * P)
            self._tables.append((h.reshape(S, P), d.view(S, P)))
        c = self.ctx
        c.token_ids, c.positions, c.row_seq, c.want_rows = (self._token_ids[1], self._positions[1],
                                                            self._row_seq[1], self._want[1])
        c.seq_slot, c.seq_q_start, c.seq_q_len, c.seq_kv_len = (self._seq_slot[1], self._seq_q_start[1],
                                                                self._seq_q_len[1], self._seq_kv_len[1])
        c.calls = []
        for i, call in enumerate(model.order):
            table = self._tables[cache.cache_group[i][0]][1] if i in cache.cache_group else None
            view = cache.cache_view(i, table) if table is not None else None
            c.calls.append(CallContext(i, view, call.cache_from is None, cache.states.get(i)))

    # ------------------------------------------------------------------
    def validate(self, entries: Sequence[StepEntry]) -> Tuple[int, int]:
        if not entries:
            raise EngineError("step: an empty batch")
        if len(entries) > self.max_batch_seqs:
            raise EngineError(f"step: {len(entries)} requests in one batch, the engine takes {self.max_batch_seqs}")
        seen = set()
        total = n_want = 0
        for e in entries:
            if e.slot in seen:
                raise EngineError(f"step: slot {e.slot} appears twice in one batch")
            seen.add(e.slot)
            n = len(e.tokens)
            if n == 0:
                raise EngineError(f"step: slot {e.slot} brings no tokens")
            length = self.cache.length(e.slot)
            if length + n > self.cache.max_tokens:
                raise EngineError(f"step: slot {e.slot} would hold {length + n} tokens, the cache holds "
                                  f"{self.cache.max_tokens} per request")
            for t in e.tokens:
                if not (0 <= int(t) < self.vocab):
                    raise EngineError(f"step: token id {t} is outside the vocabulary (0..{self.vocab - 1})")
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise EngineError(f"step: wanted place {w} is outside the {n} tokens of slot {e.slot}")
            total += n
            n_want += len(e.want)
        if total > self.max_step_tokens:
            raise EngineError(f"step: {total} tokens in one batch, the engine takes {self.max_step_tokens}")
        return total, n_want

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs the batch; returns float32 logits [wanted, vocab] on the device, in the order of
        the entries and of each entry's `want` (None if nothing is wanted)."""
        total, n_want = self.validate(entries)
        if not self.cache.can_reserve([(e.slot, len(e.tokens)) for e in entries]):
            from ..errors import OutOfPages
            raise OutOfPages("out of pages: the batch needs more pages than the pools have free "
                             f"(free per group: {[g.pool.free_pages for g in self.cache.groups]})")
        for e in entries:
            self.cache.reserve(e.slot, len(e.tokens))
        c = self.ctx
        row = w = 0
        c.host_q_len, c.host_kv_len = [], []
        for s, e in enumerate(entries):
            n = len(e.tokens)
            length = self.cache.length(e.slot)
            self._token_ids[0][row: row + n] = e.tokens
            self._positions[0][row: row + n] = np.arange(length, length + n, dtype=np.int32)
            self._row_seq[0][row: row + n] = s
            for place in e.want:
                self._want[0][w] = row + int(place)
                w += 1
            self._seq_slot[0][s] = e.slot
            self._seq_q_start[0][s] = row
            self._seq_q_len[0][s] = n
            self._seq_kv_len[0][s] = length + n
            c.host_q_len.append(n)
            c.host_kv_len.append(length + n)
            row += n
        slots = [e.slot for e in entries]
        for gi in range(len(self.cache.groups)):
            self.cache.block_table_rows(gi, slots, self._tables[gi][0])
        self._dev.copy_(self._host, non_blocking=True)
        c.n_tokens, c.n_seqs, c.n_want = total, len(entries), n_want
        c.max_q_len, c.max_kv_len = max(c.host_q_len), max(c.host_kv_len)
        c.stream = torch.cuda.current_stream().cuda_stream
        c.extras.clear()
        logits = self.model.forward(c)
        for e in entries:
            self.cache.commit(e.slot, len(e.tokens))
        return logits
