"""Continuous batching above the step function.

Each step the scheduler ends requests past their deadline, gives every running request that has
finished its prompt one decode row, spends what is left of the token budget
(`max_step_tokens`) on prompt portions of admitted requests in arrival order, admits waiting
requests in order while a slot and pages allow, runs ONE batch through the executor, samples,
emits events, and frees what finished.

It keeps the request model of cuongvng/bare-cuda-4gib (engine/include/llm/scheduler.h:19-54,
engine/src/scheduler.cpp:28-208): `Request`, `TokenEvent`, `SchedulerStats`, first-come
first-served admission with head-of-line blocking, the stop token is emitted, a request ends
with "length" when it has generated its target, and the last generated token is never fed back.
What differs: the reference prefills a whole prompt at admission, one request after another,
before the decode pass of the same step; here prompts are cut into portions under the budget and
share the batch with decode rows.

Running ahead.  In steady decoding the host's share of a step (planning, metadata, reading the
sampled ids back) would leave the GPU idle between steps.  With an executor that can launch a step
and hand its tokens over later (`launch` / `collect`), a step of decode rows only, all greedy, is
left in flight when `step()` returns; the next call first launches the following step for the same
requests, whose token ids the device takes from the argmax of the step in flight, and only then
collects that step's tokens and emits its events.  So events arrive one call late while this lasts,
and a request that turns out to have ended (a stop id) has run one row too many, which is
dropped.  Anything else - a request about to reach its length, someone waiting, a deadline,
sampling on the host, pages that do not fit - ends the run and the scheduler goes on step by step.

When pages run out.  Two policies:
* "reserve" (the reference's, default): a request is admitted only if the pages of its whole run
  (prompt + target - 1 positions) fit beside what is already promised, so an admitted request
  can never run out of pages.
* "on_demand": a request is admitted when its next portion's pages are free.  If the pool
  cannot cover a step, the most recently admitted running request is preempted: its pages and
  slot are given back and it returns to the FRONT of the waiting line with
  prompt <- prompt + generated tokens (recomputed later; its sampling generator continues).
  A request that cannot fit alone is refused at submit.
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Tuple

from ..cache.manager import CacheManager
from ..errors import EngineError
from ..sampling.params import SamplingParams, check_sampling, rng_for
from .step import StepEntry

FINISH_NONE, FINISH_STOP, FINISH_LENGTH = "", "stop", "length"
FINISH_CANCELLED, FINISH_TIMEOUT, FINISH_ERROR = "cancelled", "timeout", "error"


@dataclass
class Request:
    id: int = 0
    prompt: List[int] = field(default_factory=list)
    max_new_tokens: int = 16
    stop_ids: List[int] = field(default_factory=list)   # generating any of these ends the request
    sampling: SamplingParams = field(default_factory=SamplingParams)
    timeout_ms: int = 0                                  # from submit; 0 never times out


@dataclass
class TokenEvent:
    """One generated token, or a request ending without one (token -1)."""

    id: int = 0
    token: int = -1
    index: int = -1      # position among this request's generated tokens
    finish: str = FINISH_NONE


@dataclass
class SchedulerStats:
    running: int = 0
    waiting: int = 0
    kv_pages_used: int = 0
    kv_pages_committed: int = 0
    kv_pages_total: int = 0
    steps: int = 0              # batches run
    prefill_tokens: int = 0     # prompt tokens run through the model
    decode_tokens: int = 0      # decode rows
    prefill_chunks: int = 0     # prompt portions
    preemptions: int = 0
    busy_seconds: float = 0.0

    def as_dict(self) -> Dict[str, float]:
        return dict(self.__dict__)


@dataclass
class EngineLimits:
    max_tokens: int = 0      # per request, prompt plus generated
    max_seqs: int = 0
    kv_pages: int = 0        # pages of the smallest pool
    max_step_tokens: int = 0


class _Live:
    __slots__ = ("request", "deadline", "tokens", "fed", "generated", "target", "slot", "pages", "rng",
                 "admitted_at", "original_prompt_len")

    def __init__(self, request: Request, deadline: float):
        self.request = request
        self.deadline = deadline
        self.tokens: List[int] = list(request.prompt)   # everything known: prompt, then generated
        self.fed = 0                                     # how many of `tokens` are in the cache
        self.generated = 0
        self.target = 0
        self.slot = -1
        self.pages = 0
        self.rng = rng_for(request.sampling)
        self.admitted_at = 0
        self.original_prompt_len = len(request.prompt)


class _InFlight:
    """A launched step whose tokens have not been collected."""

    __slots__ = ("handle", "wanted", "chain")

    def __init__(self, handle, wanted, chain):
        self.handle, self.wanted = handle, wanted
        self.chain = chain      # a step of greedy decode rows only: the next one may be launched from its argmax


class Scheduler:
    """Not thread-safe; one thread calls everything.  `executor.run(entries, params, rngs)` must
    return one sampled token per wanted row (see `engine.ModelExecutor`)."""

    def __init__(self, cache: CacheManager, executor, *, max_step_tokens: int, policy: str = "reserve",
                 vocab_size: int = 0):
        """`vocab_size` (when known): a prompt with an id outside it is refused at submission, not by
        the step function in the middle of a batch that other requests share."""
        if policy not in ("reserve", "on_demand"):
            raise EngineError(f"unknown page policy '{policy}' (reserve or on_demand)")
        self.cache, self.executor, self.policy = cache, executor, policy
        self.vocab_size = int(vocab_size)
        self.limits = EngineLimits(cache.max_tokens, cache.max_seqs,
                                   min((g.num_pages for g in cache.groups), default=0), int(max_step_tokens))
        self.waiting: Deque[_Live] = deque()
        self.running: List[_Live] = []
        self.committed = [0] * len(cache.groups)
        self.totals = SchedulerStats()
        self._admissions = 0
        self._inflight: Optional[_InFlight] = None
        self._can_run_ahead = hasattr(executor, "launch") and hasattr(executor, "collect")

    # ------------------------------------------------------------------ validity
    def target_tokens(self, prompt_len: int, max_new_tokens: int) -> int:
        """A request stops early at max_tokens; its last token is never cached."""
        return min(max_new_tokens, self.limits.max_tokens - prompt_len + 1)

    def pages_needed(self, prompt_len: int, max_new_tokens: int) -> List[int]:
        positions = prompt_len + self.target_tokens(prompt_len, max_new_tokens) - 1
        return self.cache.pages_for_tokens(max(positions, 1), self.limits.max_step_tokens)

    def check(self, request: Request) -> str:
        """Empty if the request can ever run, else why not."""
        n = len(request.prompt)
        if n == 0:
            return "empty prompt"
        if request.max_new_tokens <= 0:
            return "max_new_tokens must be positive"
        if n > self.limits.max_tokens:
            return f"prompt has {n} tokens, the engine holds {self.limits.max_tokens} per sequence"
        if self.vocab_size and not (0 <= min(request.prompt) and max(request.prompt) < self.vocab_size):
            bad = next(t for t in request.prompt if not (0 <= t < self.vocab_size))
            return f"token id {bad} is outside the vocabulary (0..{self.vocab_size - 1})"
        for gi, pages in enumerate(self.pages_needed(n, request.max_new_tokens)):
            total = self.cache.groups[gi].num_pages
            if pages > total:
                return f"request needs {pages} KV pages, the pool holds {total}"
        return check_sampling(request.sampling)

    # ------------------------------------------------------------------ requests
    def submit(self, request: Request) -> None:
        error = self.check(request)
        if error:
            raise EngineError(f"scheduler: request {request.id}: {error}")
        deadline = time.monotonic() + request.timeout_ms / 1000.0 if request.timeout_ms > 0 else float("inf")
        self.waiting.append(_Live(request, deadline))

    def cancel(self, request_id: int) -> bool:
        for live in list(self.waiting):
            if live.request.id == request_id:
                self.waiting.remove(live)
                return True
        for live in self.running:
            if live.request.id == request_id:
                self._retire(live)
                self.running.remove(live)
                return True
        return False

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running and self._inflight is None

    def stats(self) -> SchedulerStats:
        s = SchedulerStats(**self.totals.__dict__)
        s.running, s.waiting = len(self.running), len(self.waiting)
        s.kv_pages_used = max(self.cache.pages_in_use(), default=0)
        s.kv_pages_committed = max(self.committed, default=0)
        s.kv_pages_total = self.limits.kv_pages
        return s

    # ------------------------------------------------------------------ one step
    def step(self) -> List[TokenEvent]:
        start = time.monotonic()
        try:
            return self._run_step()
        finally:
            self.totals.busy_seconds += time.monotonic() - start

    def _retire(self, live: _Live) -> None:
        self.cache.release_slot(live.slot)
        if self.policy == "reserve":
            for gi, p in enumerate(live.pages):
                self.committed[gi] -= p
        live.slot = -1

    def _expire(self, events: List[TokenEvent]) -> None:
        now = time.monotonic()
        for live in [l for l in self.waiting if l.deadline <= now]:
            self.waiting.remove(live)
            events.append(TokenEvent(live.request.id, -1, -1, FINISH_TIMEOUT))
        for live in [l for l in self.running if l.deadline <= now]:
            self._retire(live)
            self.running.remove(live)
            events.append(TokenEvent(live.request.id, -1, -1, FINISH_TIMEOUT))

    def _admit(self) -> None:
        """In order; a request that does not fit yet blocks the ones behind it."""
        while self.waiting and self.cache.free_slots > 0:
            live = self.waiting[0]
            if self.policy == "reserve":
                need = self.pages_needed(len(live.tokens), live.request.max_new_tokens - live.generated)
                if any(self.committed[gi] + need[gi] > g.num_pages for gi, g in enumerate(self.cache.groups)):
                    break
                live.pages = need
                for gi, p in enumerate(need):
                    self.committed[gi] += p
            else:
                first = min(len(live.tokens), self.limits.max_step_tokens)
                need = self.cache.pages_for_tokens(first, self.limits.max_step_tokens)
                if any(need[gi] > g.pool.free_pages for gi, g in enumerate(self.cache.groups)):
                    break
                live.pages = need
            self.waiting.popleft()
            live.slot = self.cache.acquire_slot()
            live.fed = 0
            if live.target == 0:
                live.target = self.target_tokens(live.original_prompt_len, live.request.max_new_tokens)
            self._admissions += 1
            live.admitted_at = self._admissions
            self.running.append(live)

    def _plan(self) -> List[Tuple[_Live, int]]:
        """(request, tokens to feed): decode rows first, then prompt portions in admission order."""
        budget = self.limits.max_step_tokens
        plan: List[Tuple[_Live, int]] = []
        for live in self.running:
            if len(live.tokens) - live.fed == 1 and live.generated > 0 and budget > 0:
                plan.append((live, 1))
                budget -= 1
        for live in sorted(self.running, key=lambda l: l.admitted_at):
            pending = len(live.tokens) - live.fed
            if budget <= 0:
                break
            if pending >= 1 and not (pending == 1 and live.generated > 0):
                n = min(pending, budget)
                plan.append((live, n))
                budget -= n
        return plan

    def _preempt_one(self, events: List[TokenEvent]) -> bool:
        """Gives the most recently admitted request's pages back; False if only one is running."""
        if len(self.running) <= 1:
            return False
        victim = max(self.running, key=lambda l: l.admitted_at)
        self.running.remove(victim)
        self._retire(victim)
        victim.fed = 0
        self.waiting.appendleft(victim)
        self.totals.preemptions += 1
        return True

    def _run_step(self) -> List[TokenEvent]:
        events: List[TokenEvent] = []
        if self._inflight is not None:
            ahead = self._launch_ahead()
            self._collect(events)
            if ahead is not None:
                self._inflight = ahead
                return events
        self._expire(events)
        self._admit()
        if not self.running:
            return events
        while True:
            plan = self._plan()
            if self.cache.can_reserve([(live.slot, n) for live, n in plan]):
                break
            if self.policy == "reserve":
                raise EngineError("scheduler: out of pages although every running request's pages were reserved")
            if not self._preempt_one(events):
                # a single request is left and it does not fit: shrink its portion to what the pool can hold
                live, n = plan[0]
                while n > 1 and not self.cache.can_reserve([(live.slot, n)]):
                    n //= 2
                if not self.cache.can_reserve([(live.slot, n)]):
                    raise EngineError("scheduler: out of pages with a single running request")
                plan = [(live, n)]
                break
        entries, params, rngs, wanted = [], [], [], []
        for live, n in plan:
            chunk = live.tokens[live.fed: live.fed + n]
            last = live.fed + n == len(live.tokens)
            entries.append(StepEntry(live.slot, chunk, [n - 1] if last else []))
            if last:
                params.append(live.request.sampling)
                rngs.append(live.rng)
                wanted.append(live)
            if n == 1 and live.generated > 0 and last:
                self.totals.decode_tokens += 1
            else:
                self.totals.prefill_tokens += n
                self.totals.prefill_chunks += 1
        self.totals.steps += 1
        for live, n in plan:
            live.fed += n
        if not self._can_run_ahead:
            self._emit(wanted, self.executor.run(entries, params, rngs), events)
            return events
        chain = (bool(wanted) and len(wanted) == len(plan) and all(n == 1 for _, n in plan)
                 and all(p.greedy() for p in params))
        self._inflight = _InFlight(self.executor.launch(entries, params, rngs), wanted, chain)
        if not chain:
            self._collect(events)
        return events

    def _emit(self, wanted, tokens, events: List[TokenEvent]) -> None:
        """Books one sampled token per wanted row; rows of requests that ended meanwhile are dropped."""
        finished = []
        for live, token in zip(wanted, tokens):
            if live.slot < 0:
                continue
            token = int(token)
            event = TokenEvent(live.request.id, token, live.generated)
            live.generated += 1
            live.tokens.append(token)
            if token in live.request.stop_ids:
                event.finish = FINISH_STOP
            elif live.generated >= live.target:
                event.finish = FINISH_LENGTH
            events.append(event)
            if event.finish:
                finished.append(live)
        for live in finished:
            self._retire(live)
            self.running.remove(live)

    def _collect(self, events: List[TokenEvent]) -> None:
        flight, self._inflight = self._inflight, None
        self._emit(flight.wanted, self.executor.collect(flight.handle), events)

    def _launch_ahead(self) -> Optional[_InFlight]:
        """The step after the one in flight, for the same requests, with token ids taken on the
        device from that step's argmax; None if anything could change the batch."""
        flight = self._inflight
        if not flight.chain or self.waiting or len(flight.wanted) != len(self.running):
            return None
        for live in flight.wanted:
            # still running, no deadline, and the token in flight is not its last
            if live.slot < 0 or live.deadline != float("inf") or live.generated + 1 >= live.target:
                return None
        if not self.cache.can_reserve([(live.slot, 1) for live in flight.wanted]):
            return None
        entries = [StepEntry(live.slot, [0], [0]) for live in flight.wanted]   # ids come from the device
        params = [live.request.sampling for live in flight.wanted]
        handle = self.executor.launch(entries, params, [live.rng for live in flight.wanted], device_fed=True)
        for live in flight.wanted:
            live.fed += 1
        self.totals.steps += 1
        self.totals.decode_tokens += len(entries)
        return _InFlight(handle, flight.wanted, True)
