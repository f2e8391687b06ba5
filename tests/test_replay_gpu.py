"""The engine against the plain implementation in every way of cutting requests into steps:
whole, decoded tail, portions of changing size, and mixed batches over a small pool."""

import random

import pytest

import helpers as H

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


def _requests(name, seed, lengths):
    rng = random.Random(seed)
    vocab = H.TINY[name][0]["vocab_size"]
    return {f"r{i}": H.random_ids(rng, n, vocab) for i, n in enumerate(lengths)}


LENGTHS = {"A": [1, 2, 17, 40, 97, 128], "B": [3, 31, 33, 64, 100, 200]}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole(name, dtype):
    folder, page = H.model_folder(name), H.TINY[name][1]
    requests = _requests(name, 1, LENGTHS[name])
    steps = H.trace_whole(requests)
    got = H.Replayer(folder, dtype, page, H.peak_tokens(steps, page)).run(steps)
    H.check_against_plain(folder, requests, got, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_decode_tail(name, dtype):
    folder, page = H.model_folder(name), H.TINY[name][1]
    requests = _requests(name, 2, LENGTHS[name][2:])
    steps = H.trace_decode_tail(requests, 32)
    got = H.Replayer(folder, dtype, page, H.peak_tokens(steps, page), shuffle_seed=3).run(steps)
    H.check_against_plain(folder, requests, got, dtype, expect_all=False)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_portions(name, dtype):
    folder, page = H.model_folder(name), H.TINY[name][1]
    requests = _requests(name, 3, LENGTHS[name][2:])
    steps = H.trace_portions(requests, random.Random(5))
    got = H.Replayer(folder, dtype, page, H.peak_tokens(steps, page), shuffle_seed=4).run(steps)
    H.check_against_plain(folder, requests, got, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_small_pool(name, dtype):
    folder, page = H.model_folder(name), H.TINY[name][1]
    longest = H.TINY[name][0]["max_position_embeddings"]
    rng = random.Random(11)
    lengths = [rng.randrange(3, longest // 2) for _ in range(10)] + [longest]
    requests = _requests(name, 4, lengths)
    budget = 2 * longest   # far fewer pages than all requests together need
    steps = H.trace_mixed(requests, random.Random(6), live=4, budget_tokens=budget, page=page)
    assert H.peak_tokens(steps, page) <= budget
    rep = H.Replayer(folder, dtype, page, budget, shuffle_seed=9)
    got = rep.run(steps)
    H.check_against_plain(folder, requests, got, dtype)
    pool = rep.cache.groups[0].pool
    assert pool.acquired_total > pool.num_pages, "the pool was never reused"
    assert pool.pages_in_use == 0
