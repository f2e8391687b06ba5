"""The cache manager's bookkeeping on the host: no page lost, held twice or freed twice, under
random orders of requests; windows give pages back; state slots are zeroed."""

import random

import pytest

from bare_cuda_4gib_b200.cache import CacheDemand, CacheManager, PagePool
from bare_cuda_4gib_b200.errors import CacheError, OutOfPages
from bare_cuda_4gib_b200.parts.base import KVCacheRequest, StateRequest


def test_pool_order_exhaustion_and_bad_releases():
    pool = PagePool(4)
    assert [pool.acquire() for _ in range(4)] == [0, 1, 2, 3]
    with pytest.raises(OutOfPages):
        pool.acquire()
    pool.release(2)
    assert pool.acquire() == 2 and pool.high_water == 4
    pool.release(1)
    with pytest.raises(CacheError, match="twice"):
        pool.release(1)
    with pytest.raises(CacheError, match="not a page"):
        pool.release(9)


def test_pool_random_steps_against_a_model():
    rng = random.Random(0)
    pool, held = PagePool(37), set()
    pool.shuffle_free_list(5)
    for _ in range(20000):
        if held and (rng.random() < 0.5 or not pool.free_pages):
            page = rng.choice(sorted(held))
            pool.release(page)
            held.remove(page)
        else:
            page = pool.acquire()
            assert page not in held
            held.add(page)
        assert pool.pages_in_use == len(held) and pool.free_pages == 37 - len(held)


def _manager(window=None, pages=20, max_seqs=4, page_tokens=16, layers=3, shared=False):
    kv = KVCacheRequest(2, 16, window)
    demands = [CacheDemand(kv) for _ in range(layers)]
    if shared:
        demands.append(CacheDemand(kv, cache_from=0))
    return CacheManager(demands, page_tokens=page_tokens, max_seqs=max_seqs, max_tokens=160, num_pages=pages,
                        allocate=False)


def test_reserve_commit_release_and_limits():
    m = _manager()
    s = m.acquire_slot()
    m.reserve(s, 17)
    assert m.pages_in_use() == [2] and m.length(s) == 0
    m.commit(s, 17)
    m.reserve(s, 1)                      # position 17 is in the second page already
    assert m.pages_in_use() == [2]
    m.commit(s, 1)
    with pytest.raises(CacheError, match="limit"):
        m.reserve(s, 160)
    m.release_slot(s)
    assert m.pages_in_use() == [0]
    with pytest.raises(CacheError):
        m.release_slot(s)
    with pytest.raises(CacheError):
        m.length(s)


def test_out_of_pages_takes_nothing():
    m = _manager(pages=3)
    a, b = m.acquire_slot(), m.acquire_slot()
    m.reserve(a, 30)
    m.commit(a, 30)
    with pytest.raises(OutOfPages):
        m.reserve(b, 40)
    assert m.pages_in_use() == [2] and not m.can_reserve([(b, 40)]) and m.can_reserve([(b, 16)])
    m.check_consistency()


def test_groups_by_need_and_borrowed_caches():
    demands = [CacheDemand(KVCacheRequest(2, 16)), CacheDemand(KVCacheRequest(2, 16, window=24)),
               CacheDemand(KVCacheRequest(2, 16)), CacheDemand(KVCacheRequest(2, 16), cache_from=0),
               CacheDemand(None, StateRequest((4, 3)))]
    m = CacheManager(demands, page_tokens=8, max_seqs=2, max_tokens=64, num_pages=10, allocate=True, device="cpu")
    assert len(m.groups) == 2 and m.groups[0].members == [(0, 0), (2, 0)] and m.groups[1].members == [(1, 0)]
    assert m.group_of(3) == m.group_of(0) and m.group_of(4) is None
    assert m.groups[0].page_stride == 2 * (2 * 2 * 8 * 16)
    with pytest.raises(CacheError, match="earlier run"):
        CacheManager([CacheDemand(KVCacheRequest(1, 16), cache_from=0)], page_tokens=8, max_seqs=1, max_tokens=8)
    # state slots: written by a request, zero for the next one that takes the slot
    s = m.acquire_slot()
    m.state_of(4)[s].fill_(5.0)
    m.release_slot(s)
    assert m.acquire_slot() == s and float(m.state_of(4)[s].abs().sum()) == 0.0


def test_window_gives_pages_back_as_it_moves():
    m = _manager(window=20, pages=6, page_tokens=8, layers=1)
    s = m.acquire_slot()
    held = []
    for step in range(100):
        m.reserve(s, 1)
        m.commit(s, 1)
        held.append(m.pages_in_use()[0])
        m.check_consistency()
    assert max(held) <= 4                       # ceil((20 + 1) / 8) + 1 pages at most
    table = m.groups[0].tables[s]
    assert table[0] == -1 and table[-1] >= 0
    assert m.groups[0].pool.acquired_total > 6  # pages were used again
    first_needed = (100 - 1 - 20 + 1) // 8       # first key of the last query / page
    assert all(p == -1 for p in table[:first_needed]) and all(p >= 0 for p in table[first_needed:])
    assert m.pages_for_tokens(1000, 1)[0] <= 4


@pytest.mark.parametrize("window", [None, 40])
def test_random_orders_of_requests(window):
    rng = random.Random(3)
    m = _manager(window=window, pages=24, max_seqs=5, shared=True)
    for g in m.groups:
        g.pool.shuffle_free_list(1)
    live = {}
    for it in range(3000):
        move = rng.random()
        if (move < 0.15 or not live) and m.free_slots:
            live[m.acquire_slot()] = 0
        elif move < 0.25 and live:
            s = rng.choice(sorted(live))
            m.release_slot(s)
            del live[s]
        elif live:
            s = rng.choice(sorted(live))
            n = rng.choice([1, 1, 1, 2, 7, 16, 33])
            if live[s] + n > m.max_tokens:
                continue
            if m.can_reserve([(s, n)]):
                m.reserve(s, n)
                m.commit(s, n)
                live[s] += n
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(s, n)
        m.check_consistency()
        for s, n in live.items():
            assert m.length(s) == n
            table = m.groups[0].tables[s]
            first = m.groups[0].first_needed_block(n)
            # every position a later query can see has a page
            assert all(table[b] >= 0 for b in range(first if n else 0, -(-n // 16)))
    for s in list(live):
        m.release_slot(s)
    assert m.pages_in_use() == [0] and m.free_slots == 5


def test_a_block_with_two_mixers_states_two_demands():
    """A block defined here arranges an attention-like mixer beside a recurrent one: it states two
    demands per run, the manager serves both, and a run that borrows another run's cache borrows
    both - without a change to the generic model."""
    import bare_cuda_4gib_b200.models  # noqa: F401
    from bare_cuda_4gib_b200.config import LlamaConfig
    from bare_cuda_4gib_b200.engine.model import Model
    from bare_cuda_4gib_b200.models.llama import llama_spec
    from bare_cuda_4gib_b200.parts import register_block
    from bare_cuda_4gib_b200.parts.block import PreNormBlock
    from bare_cuda_4gib_b200.parts.spec import LayerCall

    @register_block("toy_two_mixers")
    class TwoMixers(PreNormBlock):
        def cache_demands(self):
            return [(self.mixer.cache_request(), None),                       # the attention's pages
                    (KVCacheRequest(1, 8, window=16), StateRequest((5,)))]    # a second mixer: a small windowed cache and state

    cfg = LlamaConfig.from_dict(dict(architectures=["LlamaForCausalLM"], vocab_size=32, hidden_size=32, num_hidden_layers=2,
                                     num_attention_heads=2, num_key_value_heads=1, head_dim=16, intermediate_size=48))
    spec = llama_spec(cfg)
    spec.layers[1].block = "toy_two_mixers"
    spec.order = [LayerCall(0), LayerCall(1), LayerCall(1, cache_from=1)]
    model = Model(spec)
    demands = model.cache_demands()
    assert [len(d) for d in demands] == [1, 2, 2] and demands[2][1].cache_from == 1
    m = CacheManager(demands, page_tokens=8, max_seqs=2, max_tokens=32, allocate=True, device="cpu")
    assert len(m.groups) == 2                                                  # attention pages; the windowed second cache
    assert m.group_of(0) == (0, 0) and m.group_of(1) == (0, 1) and m.group_of(1, 1) == (1, 0)
    assert m.group_of(2) == m.group_of(1) and m.group_of(2, 1) == m.group_of(1, 1)      # borrowed, both
    assert m.state_of(1, 1).shape == (2 + 1, 5) and m.state_of(2, 1) is m.state_of(1, 1) and m.state_of(1, 0) is None
    s = m.acquire_slot()
    m.reserve(s, 20)
    m.commit(s, 20)
    m.check_consistency()
    assert m.pages_in_use() == [3, 3]
    m.release_slot(s)
    assert m.pages_in_use() == [0, 0]
