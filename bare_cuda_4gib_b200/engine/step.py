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

import gc
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..errors import EngineError
from ..kernels import lib as K
from ..parts.base import CallContext


@dataclass
class StepEntry:
    """One request's share of a step: its slot, its next tokens and the places among them whose
    logits are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class Workspace:
    """Named activation buffers, allocated once for the largest step and handed out as views.

    A buffer's address is part of every CUDA graph that was captured while it was in use, so a
    buffer is never freed while the workspace lives: callers state the largest extent they can
    ever ask for (`max_rows`, `max_lead`), and should a request still outgrow its buffer, the old
    one is kept (`retired`) beside the new one, so that a graph captured earlier keeps writing
    into memory that is still this workspace's own.  `generation` counts such replacements."""

    def __init__(self, device, max_rows: int):
        self.device, self.max_rows = device, max_rows
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self.retired: List[torch.Tensor] = []
        self.generation = 0

    def get(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype, max_rows: Optional[int] = None,
            max_lead: Optional[int] = None) -> torch.Tensor:
        """A [rows, width] (or [n, rows, width]) view; the rows axis is sized for the largest step
        (or for `max_rows` when the caller only uses the buffer for small steps), the leading axis
        of a three-dimensional buffer for `max_lead` (the most the caller will ever stack)."""
        rows_axis = len(shape) - 2
        full = list(shape)
        full[rows_axis] = max(min(self.max_rows, max_rows) if max_rows else self.max_rows, shape[rows_axis])
        if rows_axis == 1 and max_lead:
            full[0] = max(full[0], int(max_lead))
        need = int(np.prod(full))
        key = (name, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < need:
            if buf is not None:
                self.retired.append(buf)
                self.generation += 1
            buf = torch.empty(need, dtype=dtype, device=self.device)
            self._buffers[key] = buf
        if rows_axis == 0:
            return buf[:need].view(full)[: shape[0]]
        # the stride of the leading axis follows from the rows axis and the width only, so it is
        # the same whatever `lead` a call asks for
        per = full[1] * int(np.prod(full[2:]))
        return buf[: shape[0] * per].view([shape[0]] + full[1:])[:, : shape[1]]

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in list(self._buffers.values()) + self.retired)


class StepContext:
    """What the parts see of a step."""

    def __init__(self):
        self.n_tokens = 0          # rows the kernels run (a padded decode step runs a few idle rows)
        self.n_seqs = 0
        self.n_want = 0
        self.pad_seqs = 0          # idle sequences appended to reach a graph-friendly batch size
        self.max_rows = 0          # the most rows any step brings
        self.max_seqs = 0
        self.dtype = torch.float32
        self.stream = 0
        self.ws: Optional[Workspace] = None
        self.token_ids = self.positions = self.row_seq = self.want_rows = None
        self.seq_slot = self.seq_q_start = self.seq_q_len = self.seq_kv_len = None
        self.calls: List[CallContext] = []
        self.use_fast_gemm = True
        self.use_fast_attention = True
        # host copies, for parts that plan their launches from the batch's shape
        self.host_slots: List[int] = []
        self.host_q_len: List[int] = []
        self.host_kv_len: List[int] = []
        self.max_q_len = 0
        self.max_kv_len = 0
        self.extras: Dict[object, object] = {}
        self.residual = None       # the float32 residual stream while a layer runs
        self.following_norm = None # the norm part that reads the stream after the part that runs now
        self.norm_after_layer = None
        self.prenormed = None      # what the last adding product left for that norm (kernels.lib.Prenormed)


def padded_batch(n: int) -> int:
    """Decode batches are padded to 1, 2, 4, 8 and then multiples of 8, so few graphs cover all sizes."""
    for b in (1, 2, 4, 8):
        if n <= b:
            return b
    return -(-n // 8) * 8


class StepRunner:
    MAX_GRAPHS = 64

    def __init__(self, model, cache: CacheManager, *, max_step_tokens: int, max_batch_seqs: Optional[int] = None,
                 use_fast_gemm: bool = True, use_fast_attention: bool = True, use_cuda_graphs: bool = True):
        if model.device is None or model.device.type != "cuda":
            raise EngineError("the step function needs a model bound on a CUDA device; there is no CPU path")
        self.model, self.cache = model, cache
        self.device = model.device
        self.max_batch_seqs = int(max_batch_seqs or cache.max_seqs)
        self.max_step_tokens = max(int(max_step_tokens), padded_batch(self.max_batch_seqs))
        self.vocab = model.spec.vocab_size
        self.ws = Workspace(self.device, self.max_step_tokens)
        self.use_cuda_graphs = use_cuda_graphs and model.graph_safe
        self._graphs: Dict[object, object] = {}
        self._seen = set()
        self._iota = np.arange(self.max_step_tokens + 8, dtype=np.int32)
        self.argmax = torch.zeros(self.max_step_tokens, dtype=torch.int32, device=self.device)   # per wanted row
        T, S, P, G = self.max_step_tokens, padded_batch(self.max_batch_seqs), cache.max_blocks, len(cache.groups)
        self._sizes = (T, S, P, G)
        total = 4 * T + 4 * S + G * S * P
        self._host_np = np.zeros(total, dtype=np.int32)        # where a step's metadata is put together
        # ... and what is sent: a few pinned copies taken in turn, each guarded by an event, because
        # the asynchronous copy reads pinned memory when the GPU gets to it, which may be after the
        # host has begun the next step (a caller need not wait for a step before it starts another)
        self._send = [torch.empty(total, dtype=torch.int32).pin_memory() for _ in range(4)]
        self._send_np = [t.numpy() for t in self._send]
        self._sent = [None] * len(self._send)
        self._turn = 0
        self._dev = torch.zeros(total, dtype=torch.int32, device=self.device)
        self.ctx = StepContext()
        self.ctx.ws = self.ws
        self.ctx.dtype = model.dtype
        self.ctx.max_rows, self.ctx.max_seqs = T, S
        self.ctx.use_fast_gemm, self.ctx.use_fast_attention = use_fast_gemm, use_fast_attention
        off = 0

        def take(n):
            nonlocal off
            view = (self._host_np[off: off + n], self._dev[off: off + n])
            off += n
            return view

        # small per-sequence arrays and block tables first, per-row arrays last: a decode step then
        # sends one short prefix of the block instead of all of it
        self._seq_slot, self._seq_q_start, self._seq_q_len, self._seq_kv_len = take(S), take(S), take(S), take(S)
        self._tables = []
        for _ in range(G):
            h, d = take(S * P)
            self._tables.append((h.reshape(S, P), d.view(S, P)))
        self._rows_offset = off
        self._row_capacity = T
        rows_h, rows_d = take(4 * T)
        # the four per-row arrays are interleaved in blocks sized for the step at hand; see _row_views
        self._rows_h, self._rows_d = rows_h, rows_d
        c = self.ctx
        c.seq_slot, c.seq_q_start, c.seq_q_len, c.seq_kv_len = (self._seq_slot[1], self._seq_q_start[1],
                                                                self._seq_q_len[1], self._seq_kv_len[1])
        c.calls = []
        for i, call in enumerate(model.order):
            views, states = [], []
            for j in range(len(cache.demands[i])):
                where = cache.group_of(i, j)
                views.append(cache.cache_view(i, self._tables[where[0]][1], j) if where is not None else None)
                states.append(cache.state_of(i, j))
            c.calls.append(CallContext(i, views, call.cache_from is None, states))

    def _row_views(self, rows: int):
        """token ids, positions, batch sequence of a row, wanted rows: four arrays of `rows` entries at
        the start of the per-row region (so the upload is one prefix of the block)."""
        h, d = self._rows_h, self._rows_d
        return [(h[i * rows: (i + 1) * rows], d[i * rows: (i + 1) * rows]) for i in range(4)]

    def metadata_bytes(self, n_tokens: int, n_seqs: int) -> int:
        """Bytes of step metadata sent to the device for a batch of this shape."""
        return (self._rows_offset + 4 * n_tokens) * 4

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
            if min(e.tokens) < 0 or max(e.tokens) >= self.vocab:
                bad = next(t for t in e.tokens if not (0 <= int(t) < self.vocab))
                raise EngineError(f"step: token id {bad} is outside the vocabulary (0..{self.vocab - 1})")
            if e.want and (min(e.want) < 0 or max(e.want) >= n):
                bad = next(w for w in e.want if not (0 <= int(w) < n))
                raise EngineError(f"step: wanted place {bad} is outside the {n} tokens of slot {e.slot}")
            total += n
            n_want += len(e.want)
        if total > self.max_step_tokens:
            raise EngineError(f"step: {total} tokens in one batch, the engine takes {self.max_step_tokens}")
        return total, n_want

    def step(self, entries: Sequence[StepEntry], device_fed: bool = False) -> Optional[torch.Tensor]:
        """Runs the batch; returns float32 logits [wanted, vocab] on the device, in the order of
        the entries and of each entry's `want` (None if nothing is wanted).  With `device_fed`
        (one token per entry) the token ids are not the entries' but the argmax of the previous
        step's wanted rows, row i for entry i, copied on the device: the caller need not have read
        them yet."""
        decode, n_want = self.begin(entries, device_fed=device_fed)
        logits = self._run(self.ctx, decode, entries)
        self.finish(entries)
        return None if logits is None else logits[:n_want]

    def finish(self, entries: Sequence[StepEntry]) -> None:
        """Moves the requests' lengths once every layer has written the step's keys and values."""
        for e in entries:
            self.cache.commit(e.slot, len(e.tokens))

    def begin(self, entries: Sequence[StepEntry], device_fed: bool = False) -> Tuple[bool, int]:
        """Validates the batch, takes its pages, builds and sends the step's metadata and lets the
        parts plan; after this `self.ctx` describes the step.  Returns (pure decode step, wanted rows)."""
        total, n_want = self.validate(entries)
        self.cache.reserve_batch([(e.slot, len(e.tokens)) for e in entries])     # all or nothing
        c = self.ctx
        n_seqs = len(entries)
        # a pure decode step (one token and its logits per request) is padded to a few fixed batch
        # sizes with idle rows, so that one captured graph serves every step of that size
        decode = self.use_cuda_graphs and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
        pad = padded_batch(n_seqs) - n_seqs if decode else 0
        rows, seqs, wanted = total + pad, n_seqs + pad, n_want + pad
        (tok_h, tok_d), (pos_h, pos_d), (rs_h, rs_d), (want_h, want_d) = self._row_views(rows)
        c.token_ids, c.positions, c.row_seq, c.want_rows = tok_d, pos_d, rs_d, want_d
        row = w = 0
        if all(len(e.tokens) == 1 for e in entries):
            # one token per request (the decode step): fill whole arrays at once
            lengths = [self.cache.lengths[e.slot] for e in entries]
            tok_h[:n_seqs] = [e.tokens[0] for e in entries]
            pos_h[:n_seqs] = lengths
            rs_h[:n_seqs] = self._iota[:n_seqs]
            self._seq_slot[0][:n_seqs] = [e.slot for e in entries]
            self._seq_q_start[0][:n_seqs] = self._iota[:n_seqs]
            self._seq_q_len[0][:n_seqs] = 1
            c.host_kv_len = [k + 1 for k in lengths]
            self._seq_kv_len[0][:n_seqs] = c.host_kv_len
            c.host_q_len = [1] * n_seqs
            for s, e in enumerate(entries):
                if e.want:
                    want_h[w] = s
                    w += 1
            row = n_seqs
        else:
            c.host_q_len, c.host_kv_len = [], []
            for s, e in enumerate(entries):
                n = len(e.tokens)
                length = self.cache.length(e.slot)
                tok_h[row: row + n] = e.tokens
                pos_h[row: row + n] = np.arange(length, length + n, dtype=np.int32)
                rs_h[row: row + n] = s
                for place in e.want:
                    want_h[w] = row + int(place)
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
        # idle rows: token 0 at position 0 of a sequence that holds no page and whose state row is
        # the spare one that no request owns
        for i in range(pad):
            s = n_seqs + i
            tok_h[row], pos_h[row], rs_h[row], want_h[w] = 0, 0, s, row
            self._seq_slot[0][s], self._seq_q_start[0][s] = self.cache.idle_slot, row
            self._seq_q_len[0][s], self._seq_kv_len[0][s] = 0, 0
            for gi in range(len(self.cache.groups)):
                self._tables[gi][0][s].fill(-1)
            row += 1
            w += 1
        used = self._rows_offset + 4 * rows
        turn, self._turn = self._turn, (self._turn + 1) % len(self._send)
        if self._sent[turn] is not None:
            self._sent[turn].synchronize()       # the copy that last read this buffer has run (almost always long ago)
        self._send_np[turn][:used] = self._host_np[:used]
        self._dev[:used].copy_(self._send[turn][:used], non_blocking=True)
        if self._sent[turn] is None:
            self._sent[turn] = torch.cuda.Event()
        self._sent[turn].record()
        if device_fed:
            if any(len(e.tokens) != 1 for e in entries):
                raise EngineError("step: device-fed token ids need one token per request")
            tok_d[:n_seqs].copy_(self.argmax[:n_seqs], non_blocking=True)
        c.n_tokens, c.n_seqs, c.n_want, c.pad_seqs = rows, seqs, wanted, pad
        c.max_q_len, c.max_kv_len = max(c.host_q_len), max(c.host_kv_len)
        c.host_slots = slots
        c.stream = torch.cuda.current_stream().cuda_stream
        c.extras.clear()
        self.model.plan_step(c)
        return decode, n_want

    # ------------------------------------------------------------------ CUDA graphs
    def _graph_key(self, c: StepContext, decode: bool, entries) -> Optional[tuple]:
        plans = tuple(sorted((str(k), v[2:]) for k, v in c.extras.items()
                             if isinstance(k, tuple) and k and k[0] == "attention_tiles"))
        if decode:
            return ("decode", c.n_seqs, plans)
        return ("general", tuple(c.host_q_len), tuple(tuple(e.want) for e in entries), plans)

    def _forward(self, c: StepContext):
        """The model's forward pass plus the argmax of every wanted row (greedy requests need
        nothing else, so it rides in the same launch sequence or graph)."""
        logits = self.model.forward(c)
        if logits is not None:
            K.argmax_rows(logits, self.argmax, c.n_want, c.stream)
        return logits

    def _run(self, c: StepContext, decode: bool, entries):
        if not self.use_cuda_graphs:
            return self._forward(c)
        key = self._graph_key(c, decode, entries)
        held = self._graphs.get(key)
        if held is not None:
            held[0].replay()
            K.LAUNCHES[0] += held[2]              # the kernels the graph launches
            return held[1]
        if key not in self._seen or len(self._graphs) >= self.MAX_GRAPHS:
            if len(self._seen) < 4096:
                self._seen.add(key)
            return self._forward(c)               # first time: run directly (also sizes the workspace)
        graph = torch.cuda.CUDAGraph()
        before = K.LAUNCHES[0]
        # Destroying a CUDA graph is not permitted while a stream captures, and Python's collector
        # may do just that to the graphs of an engine that was dropped earlier: collect now, and keep
        # the collector off until the capture has ended.
        gc.collect()
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph):
                c.stream = torch.cuda.current_stream().cuda_stream
                logits = self._forward(c)
        finally:
            if collecting:
                gc.enable()
        launched = K.LAUNCHES[0] - before
        K.LAUNCHES[0] = before
        c.stream = torch.cuda.current_stream().cuda_stream
        self._graphs[key] = (graph, logits, launched)
        graph.replay()
        K.LAUNCHES[0] += launched
        return logits
