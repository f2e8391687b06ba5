"""Generation through the entry points against the plain implementation's cacheless greedy decode."""

import random

import pytest
import torch

import helpers as H
import plain_llama as pl

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_plain(name, dtype):
    from bare_cuda_4gib_b200.engine.engine import LLMEngine

    folder, page = H.model_folder(name), H.TINY[name][1]
    cfg = H.TINY[name][0]
    rng = random.Random(21)
    prompt = H.random_ids(rng, 19, cfg["vocab_size"])
    steps = 40
    engine = LLMEngine(folder, max_tokens=len(prompt) + steps, max_seqs=2, dtype=dtype, page_tokens=page)
    got = engine.generate(prompt, steps)
    model = H.plain_model(folder)
    if dtype == "float32":
        assert got == pl.greedy_decode(model, prompt, steps)
    else:
        # bfloat16 may pick the other of two near-equal logits: accept a different id only where the
        # plain logits of the two ids differ by less than the bfloat16 tolerance, then follow the engine
        ids = list(prompt)
        for t in got:
            logits = pl.forward_logits(model, ids)[-1]
            best = int(torch.argmax(logits))
            if t != best:
                gap = float(logits[best] - logits[t]) / float(logits.abs().max())
                assert gap <= H.TOLERANCE["bfloat16"], f"token {t} instead of {best}: gap {gap:.3e}"
            ids.append(t)


def test_batch_equals_alone_with_chunked_prompts():
    """Several requests through the scheduler with a small token budget give the ids each gives alone."""
    from bare_cuda_4gib_b200.engine.engine import LLMEngine

    folder, page = H.model_folder("B"), 32
    rng = random.Random(5)
    prompts = [H.random_ids(rng, n, 320) for n in (3, 45, 100, 17, 64)]
    alone = LLMEngine(folder, max_tokens=140, max_seqs=1, dtype="float32", page_tokens=page)
    want = [alone.generate(p, 24) for p in prompts]
    batch = LLMEngine(folder, max_tokens=140, max_seqs=3, dtype="float32", page_tokens=page, max_step_tokens=24)
    got = batch.generate_batch(prompts, 24)
    assert got == want
    assert batch.scheduler.stats().prefill_chunks > len(prompts)
    assert batch.cache.pages_in_use() == [0]


def test_on_demand_preemption_recomputes():
    """With too few pages for everyone, the on-demand policy preempts and still gives the same ids."""
    from bare_cuda_4gib_b200.engine.engine import LLMEngine

    folder, page = H.model_folder("A"), 16
    rng = random.Random(8)
    prompts = [H.random_ids(rng, n, 256) for n in (30, 28, 33, 25)]
    alone = LLMEngine(folder, max_tokens=96, max_seqs=1, dtype="float32", page_tokens=page)
    want = [alone.generate(p, 40) for p in prompts]
    tight = LLMEngine(folder, max_tokens=96, max_seqs=4, kv_pages=11, dtype="float32", page_tokens=page,
                      policy="on_demand")
    got = tight.generate_batch(prompts, 40)
    assert got == want
    assert tight.scheduler.stats().preemptions > 0
    assert tight.cache.pages_in_use() == [0]


def test_seeded_sampling_same_alone_and_batched():
    from bare_cuda_4gib_b200.engine.engine import LLMEngine
    from bare_cuda_4gib_b200.sampling.params import SamplingParams

    folder, page = H.model_folder("A"), 16
    rng = random.Random(9)
    prompts = [H.random_ids(rng, n, 256) for n in (5, 12, 9)]
    params = SamplingParams(temperature=0.9, seed=1234)
    alone = LLMEngine(folder, max_tokens=64, max_seqs=1, dtype="float32", page_tokens=page)
    want = [alone.generate(p, 20, sampling=params) for p in prompts]
    batch = LLMEngine(folder, max_tokens=64, max_seqs=3, dtype="float32", page_tokens=page)
    assert batch.generate_batch(prompts, 20, sampling=params) == want
    assert want[0] != alone.generate(prompts[0], 20)          # it does sample
    topk = SamplingParams(temperature=0.8, top_k=5, top_p=0.9, seed=7)
    assert batch.generate_batch(prompts, 10, sampling=topk) == [alone.generate(p, 10, sampling=topk) for p in prompts]


def test_async_engine_surface():
    from bare_cuda_4gib_b200.engine.engine import Engine

    folder = H.model_folder("A")
    engine = Engine(str(folder), max_tokens=64, max_seqs=2, max_waiting=1, dtype="float32", page_tokens=16)
    try:
        assert engine.vocab_size == 256 and engine.max_seqs == 2 and engine.healthy
        assert engine.submit(1, [], 4)[0] == "invalid"
        assert engine.submit(1, [1, 2, 3], 40) == ("ok", "")
        status, message = engine.submit(1, [1, 2, 3], 4)       # 40 steps cannot have run yet: the id is live
        assert status == "invalid" and "already live" in message
        assert engine.submit(3, [1, 999], 4)[0] == "invalid"   # an id outside the vocabulary of 256
        assert engine.submit(2, [4, 5], 3, temperature=-1.0)[0] == "invalid"
        events = []
        for _ in range(200):
            events += engine.poll(50)
            if any(e[0] == 1 and e[3] for e in events):
                break
        mine = [e for e in events if e[0] == 1]
        assert [e[2] for e in mine if e[1] >= 0][:4] == [0, 1, 2, 3] and mine[-1][3] == "length"
        assert engine.stats()["decode_tokens"] >= 3
        engine._fail_for_test("injected")
        for _ in range(100):
            if not engine.healthy:
                break
            engine.poll(20)
        assert not engine.healthy and "injected" in engine.failure
        assert engine.submit(5, [1], 1)[0] == "unavailable"
    finally:
        engine.stop()


@pytest.mark.parametrize("graphs", [False, True])
def test_steps_started_without_waiting_keep_their_own_metadata(graphs):
    """A caller may start step after step without waiting for the GPU (the step's metadata is
    copied from pinned memory when the GPU gets to it): every step must still see its own positions,
    lengths and tables.  Steps of changing shape, started back to back, against the same steps
    with a full synchronisation after each."""
    from bare_cuda_4gib_b200.cache.manager import CacheManager
    from bare_cuda_4gib_b200.engine.model import load_model
    from bare_cuda_4gib_b200.engine.step import StepEntry, StepRunner

    folder, page = H.model_folder("B"), 32
    model, cfg = load_model(folder, "bfloat16", "cuda")
    rng = random.Random(5)
    vocab = cfg.vocab_size
    plan = [[(0, 9), (1, 3)], [(0, 1), (1, 1)], [(0, 1), (1, 1)], [(0, 1), (1, 5), (2, 7)], [(0, 1), (1, 1), (2, 1)],
            [(0, 1), (1, 1), (2, 1)], [(2, 2)], [(0, 1), (1, 1), (2, 1)], [(0, 1), (1, 1), (2, 1)], [(0, 1), (1, 1), (2, 1)]]
    tokens = [[(s, [rng.randrange(vocab) for _ in range(n)]) for s, n in step] for step in plan]

    def run(wait):
        cache = CacheManager(model.cache_demands(), page_tokens=page, max_seqs=4, max_tokens=128, num_pages=16,
                             dtype=model.dtype, device="cuda")
        runner = StepRunner(model, cache, max_step_tokens=64, max_batch_seqs=4, use_cuda_graphs=graphs)
        slots = [cache.acquire_slot() for _ in range(3)]
        kept = []
        for step in tokens:
            logits = runner.step([StepEntry(slots[s], ids, [len(ids) - 1]) for s, ids in step])
            kept.append(logits.clone())
            if wait:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        return kept

    for a, b in zip(run(True), run(False)):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_stop_ids_and_lengths_while_running_ahead(dtype):
    """Greedy requests decode with the scheduler a step ahead; one of them stops on a token id it
    generates midway, the others run to different lengths.  Every request must give exactly the
    tokens it gives alone up to its end, the stop token included, and everything must be given back."""
    from bare_cuda_4gib_b200.engine.engine import LLMEngine
    from bare_cuda_4gib_b200.engine.scheduler import Request

    folder, page = H.model_folder("A"), H.TINY["A"][1]
    vocab = H.TINY["A"][0]["vocab_size"]
    rng = random.Random(33)
    prompts = [H.random_ids(rng, n, vocab) for n in (9, 21, 5, 14)]
    lengths = [30, 12, 25, 18]
    engine = LLMEngine(folder, max_tokens=64, max_seqs=4, dtype=dtype, page_tokens=page)
    alone = [engine.generate(p, n) for p, n in zip(prompts, lengths)]
    # request 0 stops at the first token of its own run that did not occur earlier in that run, at or after index 6
    stop_at = next(i for i in range(6, 30) if alone[0][i] not in alone[0][:i])
    stop_id = alone[0][stop_at]
    sched = engine.scheduler
    for i, (p, n) in enumerate(zip(prompts, lengths)):
        sched.submit(Request(id=i, prompt=p, max_new_tokens=n, stop_ids=[stop_id] if i == 0 else []))
    got = {i: [] for i in range(4)}
    finish = {}
    fed = 0
    launch = engine.executor.launch

    def counting(entries, params, rngs, device_fed=False):
        nonlocal fed
        fed += device_fed
        return launch(entries, params, rngs, device_fed=device_fed)

    engine.executor.launch = counting
    while not sched.idle:
        for e in sched.step():
            if e.token >= 0:
                got[e.id].append(e.token)
            if e.finish:
                finish[e.id] = e.finish
    assert fed > 5, "the scheduler never ran ahead"
    assert got[0] == alone[0][: stop_at + 1] and finish[0] == "stop"
    for i in (1, 2, 3):
        assert got[i] == alone[i] and finish[i] == "length"
    assert engine.cache.free_slots == 4 and all(g.pool.pages_in_use == 0 for g in engine.cache.groups)
    engine.cache.check_consistency()


@pytest.mark.parametrize("policy", ["reserve", "on_demand"])
def test_many_random_requests_match_their_solo_runs(policy):
    """Forty requests of random lengths, stop ids and arrival times through a small engine (four
    slots, few pages, so admission blocks and, on demand, requests are preempted and recomputed; the
    scheduler runs ahead whenever it can): float32, so every request must produce exactly the tokens
    of the plain greedy decode, cut at its stop id or length."""
    from bare_cuda_4gib_b200.engine.engine import LLMEngine
    from bare_cuda_4gib_b200.engine.scheduler import Request

    folder, page = H.model_folder("A"), H.TINY["A"][1]
    vocab = H.TINY["A"][0]["vocab_size"]
    model = H.plain_model(folder)
    rng = random.Random(77 if policy == "reserve" else 78)
    engine = LLMEngine(folder, max_tokens=96, max_seqs=4, kv_pages=8, dtype="float32", page_tokens=page,
                       max_step_tokens=24, policy=policy)
    requests, expected = [], {}
    for i in range(40):
        prompt = H.random_ids(rng, rng.randrange(1, 40), vocab)
        new = rng.randrange(1, 30)
        full = pl.greedy_decode(model, prompt, new)
        stop = []
        if rng.random() < 0.4 and new > 3:
            stop = [full[rng.randrange(1, new)]]
            full = full[: min(i for i, t in enumerate(full) if t in stop) + 1]
        requests.append(Request(id=i, prompt=prompt, max_new_tokens=new, stop_ids=stop))
        expected[i] = full
    sched = engine.scheduler
    got = {i: [] for i in range(40)}
    done = set()
    pending = list(requests)
    while pending or not sched.idle:
        for _ in range(rng.randrange(0, 3)):           # requests arrive while others run
            if pending:
                sched.submit(pending.pop(0))
        for e in sched.step():
            if e.token >= 0:
                got[e.id].append(e.token)
            if e.finish:
                assert e.finish in ("stop", "length") and e.id not in done
                done.add(e.id)
    assert done == set(range(40))
    for i in range(40):
        assert got[i] == expected[i], (i, got[i], expected[i])
    assert engine.cache.free_slots == 4 and all(g.pool.pages_in_use == 0 for g in engine.cache.groups)
    engine.cache.check_consistency()
    if policy == "on_demand":
        assert sched.stats().preemptions > 0, "the pool was never short: the test does not reach preemption"
