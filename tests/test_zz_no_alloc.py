"""The attention entry point that allocates nothing, called through its exported C symbol.

Some users of the library cannot allocate where attention runs (their program has given all GPU
memory to an allocator of its own, or a cudaMalloc would stall their latency-critical loop), so
`llm_attention_mma_static_scratch` keeps its scratch in a fixed array inside the library.  This
test checks that it computes what the ordinary entry point computes - and what dense float64
arithmetic over the same keys and values gives - on two calls in a row (the second call finds the
array full of the first call's data), and that it refuses a size that its array cannot hold.  It is collected last so that a run which stops at the first failure has
already run every other test; it does not depend on them.
"""

import ctypes
import math
import random
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _library(head_dim):
    from bare_cuda_4gib_b200.kernels import attention, build

    path = build.compile_library("attention_mma.cu", attention.defines(head_dim))
    lib = ctypes.CDLL(str(path))
    P, I, L, F = c_void_p, c_int, c_longlong, c_float
    lib.llm_attention_mma.argtypes = [P, P, P, P, P, L, I, I, I, I, P, P, P, P, P, I, I, I, P, I, F, I, P]
    lib.llm_attention_mma.restype = c_int
    lib.llm_attention_mma_static_scratch.argtypes = [P, P, P, P, P, L, I, I, I, I, P, P, P, P, P, I, I, I, I, F, I, P]
    lib.llm_attention_mma_static_scratch.restype = c_int
    lib.llm_attention_scratch_floats.argtypes = [I, I, I, I]
    lib.llm_attention_scratch_floats.restype = c_longlong
    lib.llm_attention_static_scratch_address.restype = c_void_p
    return lib


def _decode_case(seed, kv_lens, heads, kv_heads, d, page):
    """A decode step: one query token per request over a scrambled paged cache."""
    torch.manual_seed(seed)
    n = len(kv_lens)
    blocks = [-(-kv // page) for kv in kv_lens]
    n_pages = sum(blocks) + 1
    elems = 2 * kv_heads * page * d
    storage = torch.randn(n_pages, elems, device=DEV).to(torch.bfloat16)
    table = torch.full((n, max(blocks)), -1, dtype=torch.int32, device=DEV)
    perm = list(range(n_pages))
    random.Random(seed).shuffle(perm)
    at = 0
    for s, b in enumerate(blocks):
        table[s, :b] = torch.tensor(perm[at: at + b], dtype=torch.int32)
        at += b
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return dict(q=torch.randn(n, heads * d, device=DEV).to(torch.bfloat16), storage=storage, table=table,
                elems=elems, q_start=i32(list(range(n))), q_len=i32([1] * n), kv_len=i32(kv_lens),
                tile_seq=i32(list(range(n))), tile_index=i32([0] * n), n=n)


def _dense(case, kv_lens, heads, kv_heads, d, page):
    """The same attention as float64 matrix arithmetic over the gathered keys and values."""
    g = heads // kv_heads
    sv = case["storage"].view(-1, 2, kv_heads, page, d)
    out = torch.zeros(case["n"], heads, d, dtype=torch.float64, device=DEV)
    for s, kv in enumerate(kv_lens):
        pages = case["table"][s, : -(-kv // page)].long()
        k = sv[pages, 0].permute(1, 0, 2, 3).reshape(kv_heads, -1, d)[:, :kv].double()      # [kv_heads, kv, d]
        v = sv[pages, 1].permute(1, 0, 2, 3).reshape(kv_heads, -1, d)[:, :kv].double()
        q = case["q"][s].view(kv_heads, g, d).double()
        p = torch.softmax(torch.einsum("hgd,hkd->hgk", q, k) / math.sqrt(d), -1)
        out[s] = torch.einsum("hgk,hkd->hgd", p, v).reshape(heads, d)
    return out.view(case["n"], heads * d)


def _call(lib, case, heads, kv_heads, d, page, n_splits, static, scratch=None):
    out = torch.full((case["n"], heads * d), float("nan"), device=DEV, dtype=torch.bfloat16)
    st = case["storage"]
    common = [case["q"].data_ptr(), out.data_ptr(), st.data_ptr(), st.data_ptr() + (case["elems"] // 2) * 2,
              case["table"].data_ptr(), case["elems"], case["table"].stride(0), page, kv_heads, d,
              case["q_start"].data_ptr(), case["q_len"].data_ptr(), case["kv_len"].data_ptr(),
              case["tile_seq"].data_ptr(), case["tile_index"].data_ptr(), case["n"], 16, n_splits]
    tail = [heads, 1.0 / math.sqrt(d), 0, torch.cuda.current_stream().cuda_stream]
    if static:
        rc = lib.llm_attention_mma_static_scratch(*common, *tail)
    else:
        rc = lib.llm_attention_mma(*common, scratch.data_ptr(), *tail)
    torch.cuda.synchronize()
    return rc, out


def test_static_scratch_entry_point_matches_the_ordinary_one_twice():
    heads, kv_heads, d, page = 8, 2, 64, 16
    lib = _library(d)
    for round_, (kv_lens, n_splits) in enumerate([([700, 64, 1, 333], 7), ([90, 1500, 257], 11)]):
        case = _decode_case(10 + round_, kv_lens, heads, kv_heads, d, page)
        floats = lib.llm_attention_scratch_floats(case["n"], kv_heads, n_splits, 16)
        scratch = torch.zeros(floats, dtype=torch.float32, device=DEV)    # its leading counters must be zero
        rc, want = _call(lib, case, heads, kv_heads, d, page, n_splits, static=False, scratch=scratch)
        assert rc == 0
        rc, got = _call(lib, case, heads, kv_heads, d, page, n_splits, static=True)
        assert rc == 0
        assert not torch.isnan(got.float()).any()
        # same kernels, same order of sums: the tolerance of the attention kernel tests is ample
        diff = (got.double() - want.double()).abs()
        assert bool((diff <= 4e-3 + 2 ** -7 * want.double().abs()).all()), float(diff.max())
        # ... and against dense float64 arithmetic, which shares nothing with either entry point
        dense = _dense(case, kv_lens, heads, kv_heads, d, page)
        diff = (got.double() - dense).abs()
        assert bool((diff <= 4e-3 + 2 ** -7 * dense.abs()).all()), float(diff.max())
    address = lib.llm_attention_static_scratch_address()
    assert address                                         # known after the calls above


def test_static_scratch_refuses_what_its_array_cannot_hold():
    heads, kv_heads, d, page = 8, 2, 64, 16
    lib = _library(d)
    case = _decode_case(3, [40] * 60, heads, kv_heads, d, page)
    n_splits = 300
    assert lib.llm_attention_scratch_floats(case["n"], kv_heads, n_splits, 16) > (1 << 20)
    rc, out = _call(lib, case, heads, kv_heads, d, page, n_splits, static=True)
    assert rc == 4                                         # LLM_ERR_STATIC_SCRATCH_TOO_SMALL, nothing launched
    assert torch.isnan(out.float()).all()
    rc, out = _call(lib, case, heads, kv_heads, d, page, 1, static=True)   # no split: no scratch, any size
    assert rc == 0 and not torch.isnan(out.float()).any()
