"""The asynchronous engine on the host (no GPU): the scenarios of cuongvng/bare-cuda-4gib's
engine/tests/test_async_engine.cu:84-208 against `Engine` with a stand-in for the GPU side - a real
`Scheduler` over a host-only cache manager and an executor that 'samples' 1000 + (tokens the slot
holds), so a request's ids do not depend on what else is in the batch."""

import threading
import time

import pytest

from bare_cuda_4gib_b200.cache import CacheDemand, CacheManager
from bare_cuda_4gib_b200.engine.engine import Engine
from bare_cuda_4gib_b200.engine.scheduler import Request, Scheduler
from bare_cuda_4gib_b200.errors import EngineError
from bare_cuda_4gib_b200.parts.base import KVCacheRequest

VOCAB = 5000
STEPS = 12


class SlowExecutor:
    def __init__(self, cache, delay):
        self.cache, self.delay = cache, delay

    def run(self, entries, params, rngs):
        time.sleep(self.delay)
        out = []
        for e in entries:
            self.cache.reserve(e.slot, len(e.tokens))
            self.cache.commit(e.slot, len(e.tokens))
            if e.want:
                out.append(1000 + self.cache.length(e.slot))
        return out


class FakeEngine:
    """What `Engine`'s worker needs of an engine: a scheduler and the vocabulary size."""

    def __init__(self, model_path, max_tokens, max_seqs, kv_pages, delay=0.001, budget=32):
        if model_path == "/nonexistent/model":
            raise EngineError(f"cannot read {model_path}/config.json")
        cache = CacheManager([CacheDemand(KVCacheRequest(1, 16))], page_tokens=8, max_seqs=max_seqs,
                             max_tokens=max_tokens, num_pages=kv_pages or None, allocate=False)
        self.cache = cache
        self.scheduler = Scheduler(cache, SlowExecutor(cache, delay), max_step_tokens=budget, vocab_size=VOCAB)
        self.vocab_size = VOCAB


def make_engine(**kw):
    kw.setdefault("max_tokens", 128)
    kw.setdefault("max_seqs", 4)
    return Engine("fake", _engine_factory=FakeEngine, **kw)


class Drain:
    """Collects events by request id until a number of requests have finished."""

    def __init__(self, engine):
        self.engine, self.got, self.finish, self.finish_events = engine, {}, {}, {}

    def until(self, n_finished, limit_s=20.0):
        deadline = time.time() + limit_s
        while len(self.finish) < n_finished:
            assert time.time() < deadline, f"only {len(self.finish)} of {n_finished} requests finished"
            for rid, token, index, finish in self.engine.poll(20):
                if token >= 0:
                    assert index == len(self.got.setdefault(rid, []))
                    self.got[rid].append(token)
                if finish:
                    self.finish[rid] = finish
                    self.finish_events[rid] = self.finish_events.get(rid, 0) + 1


def alone(prompt, steps):
    """The ids the scheduler gives the request when nothing else runs."""
    fake = FakeEngine("fake", 128, 1, 0, delay=0.0)
    fake.scheduler.submit(Request(0, list(prompt), steps))
    out = []
    while not fake.scheduler.idle:
        out += [e.token for e in fake.scheduler.step() if e.token >= 0]
    return out


PROMPTS = [[(7 * i + j) % VOCAB for j in range(3 + 5 * i)] for i in range(9)]


def test_load_failure_raises_from_the_constructor():
    with pytest.raises(EngineError, match="cannot read"):
        Engine("/nonexistent/model", _engine_factory=FakeEngine)


def test_refusals_never_reach_the_worker():
    engine = make_engine()
    try:
        assert engine.submit(100, [], 4)[0] == "invalid"
        assert engine.submit(101, PROMPTS[0], 0)[0] == "invalid"
        status, message = engine.submit(102, [3, VOCAB + 1], 4)
        assert status == "invalid" and str(VOCAB + 1) in message and engine.healthy
        assert engine.submit(103, [1] * 200, 4)[0] == "invalid"                # longer than a sequence may get
        assert engine.max_tokens == 128 and engine.max_seqs == 4 and engine.vocab_size == VOCAB
    finally:
        engine.stop()


def test_three_submitter_threads_get_the_ids_of_a_request_alone():
    engine = make_engine()
    drain = Drain(engine)
    refused = []
    n = len(PROMPTS)

    def submit(t):
        for p in range(t, n, 3):
            status, message = engine.submit(p, PROMPTS[p], STEPS)
            if status != "ok":
                refused.append((p, status, message))
            time.sleep(0.002)

    threads = [threading.Thread(target=submit, args=(t,)) for t in range(3)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    try:
        assert not refused
        drain.until(n)
        for p in range(n):
            assert drain.got[p] == alone(PROMPTS[p], STEPS), p
            assert drain.finish[p] == "length" and drain.finish_events[p] == 1
        st = engine.stats()
        assert st["running"] == 0 and st["waiting"] == 0 and st["kv_pages_used"] == 0
        assert st["decode_tokens"] == n * (STEPS - 1)
    finally:
        engine.stop()


def test_live_id_refused_cancel_gives_one_event_and_frees_the_id():
    engine = make_engine(delay=0.005)
    drain = Drain(engine)
    try:
        assert engine.submit(200, PROMPTS[0], 100)[0] == "ok"
        status, message = engine.submit(200, PROMPTS[1], 1)
        assert status == "invalid" and "200" in message
        time.sleep(0.03)
        engine.cancel(200)
        drain.until(1)
        assert drain.finish[200] == "cancelled" and drain.finish_events[200] == 1
        assert 0 < len(drain.got.get(200, [])) < 100
        time.sleep(0.05)
        assert all(not finish for _i, _t, _x, finish in engine.poll(10))       # no second finish event
        assert engine.submit(200, PROMPTS[1], 1)[0] == "ok"                    # the id is free again
        drain.finish.pop(200)
        drain.got.pop(200)
        drain.until(1)
        assert drain.finish[200] == "length" and drain.got[200] == alone(PROMPTS[1], 1)
        engine.cancel(999)                                                       # unknown id: nothing happens
        assert engine.healthy
    finally:
        engine.stop()


def test_full_waiting_line_answers_busy_and_what_was_accepted_finishes():
    engine = make_engine(max_seqs=1, max_waiting=2, delay=0.005)
    drain = Drain(engine)
    try:
        results = [engine.submit(i, PROMPTS[i % len(PROMPTS)], STEPS)[0] for i in range(10)]
        accepted, busy = results.count("ok"), results.count("busy")
        assert busy > 0 and accepted + busy == 10
        assert 1 + 2 <= accepted <= 1 + 2 + 1          # one running plus the line, unless one finished meanwhile
        drain.until(accepted)
        assert len(drain.finish) == accepted and set(drain.finish.values()) == {"length"}
    finally:
        engine.stop()


def test_worker_failure_ends_every_live_request_and_refuses_new_work():
    engine = make_engine(delay=0.005)
    drain = Drain(engine)
    try:
        assert engine.submit(300, PROMPTS[0], 100)[0] == "ok"
        assert engine.submit(301, PROMPTS[2], 100)[0] == "ok"
        time.sleep(0.03)
        engine._fail_for_test("injected failure")
        drain.until(2)
        assert drain.finish[300] == "error" and drain.finish[301] == "error"
        assert not engine.healthy and "injected failure" in engine.failure
        status, message = engine.submit(302, PROMPTS[0], 4)
        assert status == "unavailable" and "injected failure" in message
    finally:
        engine.stop()
    assert engine.poll(10) == [] or engine.poll(10) == []


def test_stop_with_live_requests_returns():
    engine = make_engine(delay=0.005)
    assert engine.submit(1, PROMPTS[3], 100)[0] == "ok"
    assert engine.submit(2, PROMPTS[4], 100)[0] == "ok"
    time.sleep(0.02)
    started = time.time()
    engine.stop()
    assert time.time() - started < 5.0
    assert engine.submit(3, PROMPTS[0], 4)[0] == "unavailable"
    engine.stop()                                        # a second stop is harmless
