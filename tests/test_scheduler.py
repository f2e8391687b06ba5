"""The scheduler's decisions on the host, with a stand-in executor (no GPU): admission order,
token budget and portions, decode rows first, finishing, cancel, timeout, both page policies."""

import time

import pytest

from bare_cuda_4gib_b200.cache import CacheDemand, CacheManager
from bare_cuda_4gib_b200.engine.scheduler import Request, Scheduler
from bare_cuda_4gib_b200.errors import EngineError
from bare_cuda_4gib_b200.parts.base import KVCacheRequest
from bare_cuda_4gib_b200.sampling import SamplingParams


class FakeExecutor:
    """Commits what the step function would and 'samples' 1000 + (tokens the slot holds)."""

    def __init__(self, cache):
        self.cache, self.batches = cache, []

    def run(self, entries, params, rngs):
        self.batches.append([(e.slot, len(e.tokens), list(e.want)) for e in entries])
        out = []
        for e in entries:
            self.cache.reserve(e.slot, len(e.tokens))
            self.cache.commit(e.slot, len(e.tokens))
            if e.want:
                out.append(1000 + self.cache.length(e.slot))
        self.cache.check_consistency()
        return out


def make(pages=16, max_seqs=3, max_tokens=64, budget=16, policy="reserve", page_tokens=8):
    cache = CacheManager([CacheDemand(KVCacheRequest(1, 16))], page_tokens=page_tokens, max_seqs=max_seqs,
                         max_tokens=max_tokens, num_pages=pages, allocate=False)
    ex = FakeExecutor(cache)
    return Scheduler(cache, ex, max_step_tokens=budget, policy=policy), ex, cache


def drain(s, limit=500):
    events = []
    for _ in range(limit):
        if s.idle:
            break
        events += s.step()
    assert s.idle
    return events


def test_check_refusals():
    s, _, _ = make()
    assert s.check(Request(1, [], 4)) == "empty prompt"
    assert "positive" in s.check(Request(1, [1], 0))
    assert "per sequence" in s.check(Request(1, [1] * 65, 4))
    assert "temperature" in s.check(Request(1, [1], 4, sampling=SamplingParams(temperature=-1)))
    assert "top_p" in s.check(Request(1, [1], 4, sampling=SamplingParams(top_p=0.0)))
    small, _, _ = make(pages=2)
    assert "KV pages" in small.check(Request(1, [1] * 30, 4))
    with pytest.raises(EngineError):
        small.submit(Request(1, [1] * 30, 4))
    assert s.check(Request(1, [1, 2], 4)) == ""


def test_prompt_is_cut_into_portions_under_the_budget_and_decodes_ride_along():
    s, ex, cache = make(budget=16)
    s.submit(Request(1, list(range(40)), 3))
    s.submit(Request(2, list(range(5)), 4))
    events = drain(s)
    first = ex.batches[0]
    assert first == [(0, 16, [])]                                  # 16 of request 1's 40 tokens
    assert ex.batches[1] == [(0, 16, [])]
    assert ex.batches[2] == [(0, 8, [7]), (1, 5, [4])]             # its rest, then request 2 under the same budget
    assert ex.batches[3] == [(0, 1, [0]), (1, 1, [0])]             # both decode
    assert sum(n for b in ex.batches for _, n, _ in b) <= 16 * len(ex.batches)
    by = {i: [e for e in events if e.id == i] for i in (1, 2)}
    assert [e.index for e in by[1]] == [0, 1, 2] and by[1][-1].finish == "length"
    assert [e.index for e in by[2]] == [0, 1, 2, 3] and by[2][-1].finish == "length"
    assert by[1][0].token == 1040 and by[1][1].token == 1041      # the last generated token is never fed back
    st = s.stats()
    assert st.prefill_tokens == 45 and st.prefill_chunks == 4 and st.decode_tokens == 2 + 3
    assert cache.pages_in_use() == [0] and st.kv_pages_committed == 0


def test_decode_rows_come_first_and_late_arrivals_join():
    s, ex, _ = make(budget=8)
    s.submit(Request(1, [1, 2, 3], 10))
    s.step()
    s.submit(Request(2, list(range(20)), 2))
    s.step()
    assert ex.batches[1] == [(0, 1, [0]), (1, 7, [])]              # the decode row, then what is left of the budget
    drain(s)


def test_fcfs_head_of_line_blocking_reserve_policy():
    s, ex, cache = make(pages=8, max_seqs=3, budget=64)
    s.submit(Request(1, [1] * 30, 10))     # 39 positions -> 5 pages
    s.submit(Request(2, [1] * 30, 10))     # 5 more do not fit beside it
    s.submit(Request(3, [1] * 2, 2))       # would fit, but waits behind request 2
    events = s.step()
    assert len(s.running) == 1 and len(s.waiting) == 2 and s.stats().kv_pages_committed == 5
    events += drain(s)
    order = [e.id for e in events if e.index == 0]
    assert order == [1, 2, 3]
    assert cache.pages_in_use() == [0]


def test_stop_id_is_emitted_and_finishes():
    s, ex, _ = make()
    s.submit(Request(1, [1, 2, 3], 10, stop_ids=[1005]))
    events = drain(s)
    assert [e.token for e in events] == [1003, 1004, 1005] and events[-1].finish == "stop"
    s.submit(Request(2, [1, 2, 3], 10, stop_ids=[1003]))           # finished at prefill
    events = drain(s)
    assert [(e.token, e.finish) for e in events] == [(1003, "stop")]


def test_target_is_cut_at_max_tokens():
    s, ex, _ = make(max_tokens=10)
    s.submit(Request(1, [1] * 8, 100))
    events = drain(s)
    assert len(events) == 3 and events[-1].finish == "length"       # 8 + 3 - 1 = 10 positions


def test_cancel_waiting_and_running_frees_pages():
    s, ex, cache = make(max_seqs=1)
    s.submit(Request(1, [1] * 10, 50))
    s.submit(Request(2, [1] * 10, 50))
    s.step()
    assert s.cancel(2) and s.cancel(1) and not s.cancel(7)
    assert s.idle and cache.pages_in_use() == [0] and cache.free_slots == 1


def test_timeout_ends_waiting_and_running():
    s, ex, cache = make(max_seqs=1)
    s.submit(Request(1, [1] * 4, 1000, timeout_ms=30))
    s.submit(Request(2, [1] * 4, 5, timeout_ms=30))
    s.step()
    time.sleep(0.05)
    events = s.step()
    assert sorted((e.id, e.finish, e.token) for e in events) == [(1, "timeout", -1), (2, "timeout", -1)]
    assert s.idle and cache.pages_in_use() == [0]


def test_on_demand_policy_preempts_the_newest_and_recomputes():
    s, ex, cache = make(pages=6, max_seqs=3, budget=32, policy="on_demand")
    for i in (1, 2, 3):
        s.submit(Request(i, [1] * 14, 20))       # each grows to 33 positions = 5 pages; the pool has 6
    events = drain(s, 2000)
    st = s.stats()
    assert st.preemptions > 0
    for i in (1, 2, 3):
        mine = [e for e in events if e.id == i]
        assert [e.index for e in mine] == list(range(20)) and mine[-1].finish == "length"
        assert [e.token for e in mine] == [1014 + k for k in range(20)]      # same tokens as without preemption
    assert cache.pages_in_use() == [0]
    with pytest.raises(EngineError, match="policy"):
        Scheduler(cache, ex, max_step_tokens=8, policy="other")


def test_reserve_policy_never_runs_out():
    s, ex, cache = make(pages=10, max_seqs=3, budget=12)
    for i in range(8):
        s.submit(Request(i, [1] * (5 + 3 * i), 6))
    events = drain(s, 2000)
    assert s.stats().preemptions == 0
    assert sorted({e.id for e in events if e.finish == "length"}) == list(range(8))


# ----------------------------------------------------------------------------- running ahead

class AsyncFakeExecutor(FakeExecutor):
    """The stand-in with `launch` / `collect`: what a step 'samples' is fixed at launch, handed
    over at collection; a device-fed step must follow a collected-or-pending step of the same slots."""

    def __init__(self, cache, stop_token_at=None):
        super().__init__(cache)
        self.pending, self.launched, self.fed_from_device = 0, 0, 0
        self.stop_token_at = stop_token_at or {}     # slot length -> token to 'sample' instead

    def launch(self, entries, params, rngs, device_fed=False):
        if device_fed:
            assert self.pending == 1, "a device-fed step needs the step before it still in flight"
            assert all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
            assert [e.slot for e in entries] == self.last_slots
            self.fed_from_device += 1
        tokens = self.run(entries, params, rngs)
        tokens = [self.stop_token_at.get(t - 1000, t) for t in tokens]
        self.last_slots = [e.slot for e in entries]
        self.pending += 1
        self.launched += 1
        assert self.pending <= 2
        return tokens

    def collect(self, handle):
        self.pending -= 1
        return handle


def make_async(stop_token_at=None, **kw):
    s, _, cache = make(**kw)
    ex = AsyncFakeExecutor(cache, stop_token_at)
    s.executor, s._can_run_ahead = ex, True
    return s, ex, cache


def test_running_ahead_gives_the_same_events_one_call_late():
    def run(asynchronous):
        s, ex, _ = (make_async if asynchronous else make)(pages=32, max_seqs=3, budget=16)
        s.submit(Request(1, list(range(10)), 6))
        s.submit(Request(2, list(range(3)), 9))
        per_call = []
        while not s.idle:
            per_call.append([(e.id, e.token, e.index, e.finish) for e in s.step()])
        return per_call, ex, s

    sync_calls, _, _ = run(False)
    async_calls, ex, s = run(True)
    flat = lambda calls: [e for c in calls for e in c]
    assert sorted(flat(sync_calls)) == sorted(flat(async_calls))           # the same tokens, indices and endings
    for rid in (1, 2):                                                     # each request's events in order
        assert [e for e in flat(sync_calls) if e[0] == rid] == [e for e in flat(async_calls) if e[0] == rid]
    assert ex.fed_from_device >= 3                                         # it did run ahead
    assert any(not c for c in async_calls[1:-1])                           # and events came a call late
    assert ex.pending == 0 and s.stats().decode_tokens == 5 + 8


def test_running_ahead_drops_the_row_of_a_request_that_stopped():
    # request 1 'samples' its stop id when its slot holds 12 tokens; the step launched ahead of that
    # news has one row too many for it, which must not become an event
    s, ex, cache = make_async(stop_token_at={12: 77}, pages=32, max_seqs=3, budget=16)
    s.submit(Request(1, list(range(10)), 20, stop_ids=[77]))
    s.submit(Request(2, list(range(4)), 8))
    events = drain(s)
    one = [e for e in events if e.id == 1]
    assert [e.token for e in one] == [1010, 1011, 77] and one[-1].finish == "stop"
    two = [e for e in events if e.id == 2]
    assert len(two) == 8 and two[-1].finish == "length"
    assert cache.free_slots == 3 and cache.groups[0].pool.pages_in_use == 0
    cache.check_consistency()


def test_running_ahead_stops_for_waiting_requests_deadlines_and_sampling():
    s, ex, _ = make_async(pages=32, max_seqs=1, budget=16)
    s.submit(Request(1, list(range(4)), 5))
    s.submit(Request(2, list(range(4)), 3))          # waits for the only slot: nothing runs ahead meanwhile
    while not any(e.id == 1 and e.finish for e in s.step()):
        assert ex.fed_from_device == 0
    drain(s)
    s, ex, _ = make_async(pages=32, max_seqs=2, budget=16)
    s.submit(Request(1, list(range(4)), 6, timeout_ms=60000))
    drain(s)
    assert ex.fed_from_device == 0
    s, ex, _ = make_async(pages=32, max_seqs=2, budget=16)
    s.submit(Request(1, list(range(4)), 6, sampling=SamplingParams(temperature=0.7, seed=1)))
    drain(s)
    assert ex.fed_from_device == 0
    s, ex, _ = make_async(pages=32, max_seqs=2, budget=16)
    s.submit(Request(1, list(range(4)), 6))
    s.step(); s.step(); s.step()
    assert ex.fed_from_device >= 1
    assert s.cancel(1) and not s.idle                # a step is still in flight
    assert s.step() == [] and s.idle                 # its row is dropped


@pytest.mark.parametrize("policy", ["reserve", "on_demand"])
@pytest.mark.parametrize("asynchronous", [False, True])
@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_random_arrivals_and_cancellations_lose_nothing(policy, asynchronous, seed):
    """Requests of random lengths arrive between steps and some are cancelled: every request ends
    exactly once, its tokens are those it would get alone, and slots and pages all come back."""
    import random
    rng = random.Random(seed)
    maker = make_async if asynchronous else make
    s, ex, cache = maker(pages=rng.choice([9, 14, 40]), max_seqs=rng.choice([2, 3, 4]), max_tokens=64,
                         budget=rng.choice([6, 16, 40]), policy=policy)
    todo = [(i, rng.randrange(1, 30), rng.randrange(1, 12)) for i in range(14)]
    prompt_len = {i: p for i, p, _ in todo}
    wanted = {i: n for i, _, n in todo}
    events, cancelled, submitted = [], set(), set()
    for _ in range(4000):
        while todo and rng.random() < 0.4:
            i, p, n = todo.pop(0)
            s.submit(Request(i, [1] * p, n))
            submitted.add(i)
        if submitted - cancelled and rng.random() < 0.05:
            victim = rng.choice(sorted(submitted - cancelled))
            if s.cancel(victim):
                cancelled.add(victim)
        events += s.step()
        if not todo and s.idle:
            break
    assert s.idle and not todo
    for i in sorted(submitted):
        mine = [e for e in events if e.id == i and e.token >= 0]
        assert [e.index for e in mine] == list(range(len(mine)))
        assert [e.token for e in mine] == [1000 + prompt_len[i] + k for k in range(len(mine))]
        endings = [e.finish for e in events if e.id == i and e.finish]
        if i in cancelled:
            assert len(mine) <= wanted[i] and endings in ([], ["cancelled"])
        else:
            assert len(mine) == wanted[i] and endings == ["length"]
    assert cache.free_slots == cache.max_seqs and cache.pages_in_use() == [0]
    cache.check_consistency()
