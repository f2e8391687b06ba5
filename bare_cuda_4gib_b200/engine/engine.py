"""The Python entry points.

`LLMEngine` loads a model folder and owns model, cache manager, step function, sampler and
scheduler on the calling thread: `generate` (one request, greedy unless told otherwise) and
`generate_batch` follow Model::generate / Model::generate_batch of cuongvng/bare-cuda-4gib
(engine/src/model.cpp:667-716).

`Engine` is the asynchronous engine with the surface of the reference's Python module
`llm_engine_py.Engine` (server/bindings.cc:70-106 over engine/src/async_engine.cpp): a worker
thread owns everything that touches the GPU; `submit` returns (status, message) with status ok /
invalid / busy / unavailable without touching the GPU; `poll` returns (id, token, index, finish)
tuples; a failure on the worker ends every live request with finish "error" and makes the engine
refuse new work.
"""

from __future__ import annotations

import threading
from collections import deque
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..cache.manager import CacheManager
from ..errors import EngineError
from ..sampling.params import SamplingParams
from ..sampling.sampler import DeviceSampler
from .model import load_model, random_model
from .scheduler import (FINISH_CANCELLED, FINISH_ERROR, Request, Scheduler, SchedulerStats, TokenEvent)
from .step import StepEntry, StepRunner

VRAM_HEADROOM = 256 << 20   # left free when the pool is fitted to memory (engine/include/llm/model.h:19)


class ModelExecutor:
    """Runs a batch through the step function and samples the wanted rows."""

    def __init__(self, runner: StepRunner):
        self.runner = runner
        self.sampler = DeviceSampler(runner.device, runner.max_step_tokens)
        # two buffers: a step's ids may still be unread when the next step's copy is queued
        self._pinned = [torch.empty(runner.max_step_tokens, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._turn = 0

    def run(self, entries: Sequence[StepEntry], params: Sequence[SamplingParams], rngs: Sequence) -> List[int]:
        return self.collect(self.launch(entries, params, rngs))

    def launch(self, entries: Sequence[StepEntry], params: Sequence[SamplingParams], rngs: Sequence,
               device_fed: bool = False):
        """Starts a step and returns a handle for `collect`.  A step of greedy rows only is left
        running: its argmax is copied to pinned memory behind it and an event marks the copy.
        `device_fed`: the step's token ids are the argmax of the step before it (same requests in
        the same order), taken on the device."""
        logits = self.runner.step(entries, device_fed=device_fed)
        if logits is None:
            return (None, 0, None, [])
        rows = len(params)
        if all(p.greedy() for p in params):
            buffer = self._pinned[self._turn]
            self._turn ^= 1
            buffer[:rows].copy_(self.runner.argmax[:rows], non_blocking=True)
            done = torch.cuda.Event()
            done.record()
            return (buffer, rows, done, None)
        return (None, rows, None, self.sampler.sample(logits, params, rngs, self.runner.argmax))

    def collect(self, handle) -> List[int]:
        buffer, rows, done, tokens = handle
        if tokens is not None:
            return tokens
        done.synchronize()
        return buffer[:rows].tolist()


class LLMEngine:
    def __init__(self, model_path, max_tokens: int = 1024, max_seqs: int = 8, kv_pages: int = 0,
                 dtype: str = "bfloat16", page_tokens: int = 64, max_step_tokens: Optional[int] = None,
                 policy: str = "reserve", device: str = "cuda", use_fast_gemm: bool = True,
                 use_fast_attention: bool = True, use_cuda_graphs: bool = True, random=None):
        """`random=(config, seed)`: no folder is read; the model of that typed configuration gets
        seeded random weights generated on the device (the values `write_random_model` would have
        written with that seed from this device), and `model_path` may be None."""
        if not torch.cuda.is_available():
            raise EngineError("no CUDA device: the engine has no CPU path")
        if random is not None:
            self.config = random[0]
            self.model = random_model(random[0], int(random[1]), dtype, device)
        else:
            self.model, self.config = load_model(model_path, dtype, device)
        if max_tokens > self.model.spec.max_positions:
            raise EngineError(f"max_tokens {max_tokens} exceeds the model's {self.model.spec.max_positions} positions")
        if max_seqs <= 0:
            raise EngineError("max_seqs must be positive")
        demands = self.model.cache_demands()
        blocks = -(-max_tokens // page_tokens)
        wanted = max_seqs * blocks
        if kv_pages <= 0:
            probe = CacheManager(demands, page_tokens=page_tokens, max_seqs=1, max_tokens=page_tokens,
                                 num_pages=1, dtype=self.model.dtype, allocate=False)
            page_bytes = max(sum(g.bytes for g in probe.groups), 1)
            free, _total = torch.cuda.mem_get_info()
            kv_pages = int(min(wanted, max(0, free - VRAM_HEADROOM) // page_bytes))
            if kv_pages < blocks:
                raise EngineError(f"too little GPU memory for one sequence of {max_tokens} tokens "
                                  f"({kv_pages} pages fit, {blocks} are needed)")
        self.cache = CacheManager(demands, page_tokens=page_tokens, max_seqs=max_seqs, max_tokens=max_tokens,
                                  num_pages=kv_pages, dtype=self.model.dtype, device=device)
        self.max_step_tokens = int(max_step_tokens or min(max_tokens, 2048) + max_seqs)
        self.runner = StepRunner(self.model, self.cache, max_step_tokens=self.max_step_tokens,
                                 max_batch_seqs=max_seqs, use_fast_gemm=use_fast_gemm,
                                 use_fast_attention=use_fast_attention, use_cuda_graphs=use_cuda_graphs)
        self.executor = ModelExecutor(self.runner)
        self.policy = policy
        self.scheduler = Scheduler(self.cache, self.executor, max_step_tokens=self.max_step_tokens, policy=policy,
                                   vocab_size=self.model.spec.vocab_size)

    # sizes, as the reference's model summary line reports them (bench/src/main.cc:83-88)
    @property
    def max_tokens(self) -> int: return self.cache.max_tokens
    @property
    def max_seqs(self) -> int: return self.cache.max_seqs
    @property
    def kv_pages(self) -> int: return self.scheduler.limits.kv_pages
    @property
    def vocab_size(self) -> int: return self.model.spec.vocab_size

    def summary(self) -> str:
        mib = 1024.0 * 1024.0
        return (f"[llm] {len(self.model.order)} layers, hidden {self.model.spec.hidden_size}, vocab "
                f"{self.model.spec.vocab_size} | weights {self.model.weight_bytes() / mib:.1f} MiB, workspace "
                f"{self.runner.ws.bytes() / mib:.1f} MiB, cache {sum(g.bytes for g in self.cache.groups) / mib:.1f} "
                f"MiB ({self.kv_pages} pages, max batch {self.max_seqs})")

    def generate(self, prompt: Sequence[int], new_tokens: int, sampling: Optional[SamplingParams] = None,
                 stop_ids: Sequence[int] = (), on_token: Optional[Callable[[int, int], None]] = None) -> List[int]:
        """One request through the scheduler; returns the generated ids."""
        out = self.generate_batch([list(prompt)], new_tokens, sampling=sampling, stop_ids=stop_ids,
                                  on_token=(lambda rid, i, t: on_token(i, t)) if on_token else None)
        return out[0]

    def score(self, ids: Sequence[int]) -> torch.Tensor:
        """Logits at every position of `ids` (float32 [len, vocab], on the host): one fresh request
        fed in portions under the step's token budget, nothing sampled.  What the reference's tools
        read with `forward` + `logits_host` (bench/src/ppl_main.cc:104-105, batch_check_main.cc:121-123)."""
        if not self.scheduler.idle:
            raise EngineError("score: the scheduler still holds requests")
        ids = list(ids)
        if not ids or len(ids) > self.max_tokens:
            raise EngineError(f"score: {len(ids)} ids do not fit a cache of {self.max_tokens} tokens")
        slot = self.cache.acquire_slot()
        rows = []
        try:
            portion = max(1, self.max_step_tokens - 1)
            for at in range(0, len(ids), portion):
                piece = ids[at: at + portion]
                rows.append(self.runner.step([StepEntry(slot, piece, list(range(len(piece))))]).float().cpu())
        finally:
            self.cache.release_slot(slot)
        return torch.cat(rows, 0)

    def generate_batch(self, prompts: Sequence[Sequence[int]], new_tokens: int,
                       sampling: Optional[SamplingParams] = None, stop_ids: Sequence[int] = (),
                       on_token: Optional[Callable[[int, int, int], None]] = None) -> List[List[int]]:
        if not self.scheduler.idle:
            raise EngineError("generate_batch: the scheduler still holds requests")
        for i, prompt in enumerate(prompts):
            self.scheduler.submit(Request(id=i, prompt=list(prompt), max_new_tokens=new_tokens,
                                          stop_ids=list(stop_ids), sampling=sampling or SamplingParams()))
        out: List[List[int]] = [[] for _ in prompts]
        while not self.scheduler.idle:
            for e in self.scheduler.step():
                if e.token >= 0:
                    out[e.id].append(e.token)
                    if on_token:
                        on_token(e.id, e.index, e.token)
        return out


class Engine:
    """The asynchronous engine: any thread may submit, cancel and poll."""

    def __init__(self, model_path, max_tokens: int = 1024, max_seqs: int = 8, kv_pages: int = 0,
                 max_waiting: int = 64, **options):
        self._max_waiting = max_waiting
        self._in = threading.Condition()
        self._out = threading.Condition()
        self._inbox: List[Request] = []
        self._cancels: List[int] = []
        self._live = set()
        self._outbox = deque()
        self._ready = self._stopping = self._stopped = False
        self._failure = ""
        self._injected = ""
        self._load_error: Optional[BaseException] = None
        self._stats = SchedulerStats()
        self._limits = None
        self._vocab = 0
        self._check: Optional[Callable[[Request], str]] = None
        self._worker = threading.Thread(target=self._run, name="llm-engine-worker", daemon=True,
                                        args=(model_path, max_tokens, max_seqs, kv_pages, options))
        self._worker.start()
        with self._in:
            self._in.wait_for(lambda: self._ready or self._load_error is not None)
        if self._load_error is not None:
            self._worker.join()
            raise self._load_error

    # ------------------------------------------------------------------ any thread
    def submit(self, id: int, prompt: Sequence[int], max_new_tokens: int, stop_ids: Sequence[int] = (),
               temperature: float = 0.0, top_p: float = 1.0, top_k: int = 0, seed: int = -1,
               timeout_ms: int = 0) -> Tuple[str, str]:
        request = Request(id, list(prompt), max_new_tokens, list(stop_ids),
                          SamplingParams(temperature, top_p, top_k, seed), timeout_ms)
        error = self._check(request)
        if error:
            return "invalid", error
        with self._in:
            if self._failure or self._stopping:
                return "unavailable", self._failure or "the engine has stopped"
            if self._max_waiting > 0 and len(self._live) >= self._limits.max_seqs + self._max_waiting:
                return "busy", "the waiting line is full"
            if id in self._live:
                return "invalid", f"request id {id} is already live"
            self._live.add(id)
            self._inbox.append(request)
            self._in.notify_all()
        return "ok", ""

    def cancel(self, id: int) -> None:
        with self._in:
            self._cancels.append(id)
            self._in.notify_all()

    def poll(self, timeout_ms: int = 100) -> List[Tuple[int, int, int, str]]:
        with self._out:
            if not self._outbox and not self._stopped:
                self._out.wait(timeout_ms / 1000.0)
            events = list(self._outbox)
            self._outbox.clear()
        return [(e.id, e.token, e.index, e.finish) for e in events]

    def stop(self) -> None:
        with self._in:
            self._stopping = True
            self._in.notify_all()
        if self._worker.is_alive():
            self._worker.join()
        with self._out:
            self._stopped = True
            self._out.notify_all()

    def stats(self) -> Dict[str, float]:
        with self._in:
            d = self._stats.as_dict()
            d["waiting"] += len(self._inbox)
        return d

    @property
    def healthy(self) -> bool:
        with self._in:
            return not self._failure
    @property
    def failure(self) -> str:
        with self._in:
            return self._failure
    @property
    def max_tokens(self) -> int: return self._limits.max_tokens
    @property
    def max_seqs(self) -> int: return self._limits.max_seqs
    @property
    def kv_pages(self) -> int: return self._limits.kv_pages
    @property
    def vocab_size(self) -> int: return self._vocab

    def _fail_for_test(self, message: str) -> None:
        """Makes the worker raise on its next loop, to exercise the failure path (host only)."""
        with self._in:
            self._injected = message
            self._in.notify_all()

    # ------------------------------------------------------------------ worker thread
    def _publish(self, events: List[TokenEvent]) -> None:
        if not events:
            return
        with self._in:
            for e in events:
                if e.finish:
                    self._live.discard(e.id)
        with self._out:
            self._outbox.extend(events)
            self._out.notify_all()

    def _run(self, model_path, max_tokens, max_seqs, kv_pages, options) -> None:
        try:
            engine = options.pop("_engine_factory", LLMEngine)(model_path, max_tokens=max_tokens, max_seqs=max_seqs,
                                                               kv_pages=kv_pages, **options)
            scheduler = engine.scheduler
        except BaseException as e:  # noqa: BLE001 - handed to the constructor's caller
            with self._in:
                self._load_error = e
                self._in.notify_all()
            return
        with self._in:
            self._limits, self._vocab, self._check = scheduler.limits, engine.vocab_size, scheduler.check
            self._ready = True
            self._in.notify_all()
        try:
            while True:
                with self._in:
                    self._in.wait_for(lambda: self._stopping or self._inbox or self._cancels
                                      or not scheduler.idle or self._injected)
                    if self._stopping:
                        break
                    if self._injected:
                        raise EngineError(self._injected)
                    inbox, self._inbox = self._inbox, []
                    cancels, self._cancels = self._cancels, []
                for request in inbox:       # submits before cancels
                    scheduler.submit(request)
                cancelled = [TokenEvent(i, -1, -1, FINISH_CANCELLED) for i in cancels if scheduler.cancel(i)]
                self._publish(cancelled)
                self._publish(scheduler.step())
                with self._in:
                    self._stats = scheduler.stats()
        except BaseException as e:  # noqa: BLE001 - every live request learns of it
            with self._in:
                self._failure = f"{type(e).__name__}: {e}"
                live = sorted(self._live)
                self._inbox.clear()
            self._publish([TokenEvent(i, -1, -1, FINISH_ERROR) for i in live])
