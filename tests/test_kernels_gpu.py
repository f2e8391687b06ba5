"""Each CUDA kernel alone against a plain PyTorch float32 statement of the same operation, at
sizes other than the engine's: widths that are no power of two, ragged tiles, one row."""

import math
import random
import types

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _ctx(max_rows=4096):
    from bare_cuda_4gib_b200.engine.step import Workspace
    return types.SimpleNamespace(ws=Workspace(torch.device(DEV), max_rows), max_rows=max_rows, max_seqs=64,
                                 pad_seqs=0, stream=torch.cuda.current_stream().cuda_stream)


def _close(got, want, rtol, atol):
    got, want = got.double().cpu(), want.double().cpu()
    bad = (got - want).abs() > atol + rtol * want.abs()
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} differ; worst {float((got - want).abs().max()):.3e}"


# ------------------------------------------------------------------------------ plain kernels

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_gather(dtype):
    from bare_cuda_4gib_b200.kernels import lib as K
    table = torch.randn(301, 70, device=DEV).to(dtype)
    ids = torch.tensor([0, 300, 5, 5, 17], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 70, device=DEV)
    K.embed_gather(table, ids, out, 5)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("hidden", [300, 64, 2050])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(hidden, out_dtype):
    from bare_cuda_4gib_b200.kernels import lib as K
    rows, eps = 7, 1e-6
    x = torch.randn(rows, hidden, device=DEV)
    delta = torch.randn(3, rows, hidden, device=DEV)
    w = (1 + 0.1 * torch.randn(hidden, device=DEV))
    res = x.clone()
    out = torch.empty(rows, hidden, device=DEV, dtype=out_dtype)
    K.add_rmsnorm(res, K.Partials(delta, 3), w, out, eps, rows)
    want_res = x.double() + delta.double().sum(0)
    want = want_res * torch.rsqrt(want_res.pow(2).mean(-1, keepdim=True) + eps) * w.double()
    _close(res, want_res, 1e-6, 1e-6)
    if out_dtype == torch.float32:
        _close(out, want, 1e-5, 1e-5)
    else:
        _close(out, want, 2 ** -8, 1e-5)
    # gathered rows, no delta
    index = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, hidden, device=DEV)
    K.add_rmsnorm(res, None, w, out2, eps, 3, index)
    _close(out2, want[index.long()], 1e-5, 1e-5)


@pytest.mark.parametrize("rows,hidden,partials", [(7, 2048, 1), (70, 2048, 2), (300, 352, 1), (257, 4096, 3), (260, 2048, 2), (300, 5120, 1)])
def test_add_rmsnorm_bfloat16_paths(rows, hidden, partials):
    """The bfloat16 step's variants (bfloat16 weight and output): a block per row for few rows, a
    warp per row for many (rows kept in registers, widths up to 4,096), with partial results to
    add, with gathered rows and without anything to add."""
    from bare_cuda_4gib_b200.kernels import lib as K
    eps = 1e-5
    torch.manual_seed(rows + hidden)
    x = torch.randn(rows + 3, hidden, device=DEV)
    delta = torch.randn(partials, rows + 3, hidden, device=DEV)
    w = (1 + 0.1 * torch.randn(hidden, device=DEV)).to(torch.bfloat16)
    res = x.clone()
    out = torch.empty(rows, hidden, device=DEV, dtype=torch.bfloat16)
    K.add_rmsnorm(res, K.Partials(delta, partials) if partials > 1 else K.Partials(delta[0]), w, out, eps, rows)
    want_res = x.double()
    want_res[:rows] += delta.double().sum(0)[:rows]
    want = want_res * torch.rsqrt(want_res.pow(2).mean(-1, keepdim=True) + eps) * w.double()
    _close(res, want_res, 1e-6, 1e-6)           # the rows beyond `rows` are untouched
    _close(out, want[:rows], 2 ** -8, 1e-5)
    index = torch.randperm(rows + 3, device=DEV)[:rows].to(torch.int32)
    out2 = torch.empty(rows, hidden, device=DEV, dtype=torch.bfloat16)
    K.add_rmsnorm(res, None, w, out2, eps, rows, index)
    _close(out2, want[index.long()], 2 ** -8, 1e-5)
    _close(res, want_res, 1e-6, 1e-6)           # nothing to add: the stream is only read


@pytest.mark.parametrize("m,n,k", [(1, 70, 300), (17, 130, 64), (150, 64, 176), (5, 258, 96)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_matmul_plain(m, n, k, dtype):
    from bare_cuda_4gib_b200.kernels import lib as K
    a = torch.randn(m, k, device=DEV).to(dtype)
    w = torch.randn(n, k, device=DEV).to(dtype)
    out = torch.empty(m, n, device=DEV)
    K.matmul_plain(a, w, out, m)
    _close(out, a.double() @ w.double().t(), 1e-5, 1e-4)


def _paged_cache(kv_heads, head_dim, page_tokens, n_pages, dtype):
    from bare_cuda_4gib_b200.kernels.lib import CacheView
    elems = 2 * kv_heads * page_tokens * head_dim
    storage = torch.zeros(n_pages, elems, device=DEV, dtype=dtype)
    table = torch.full((4, 16), -1, dtype=torch.int32, device=DEV)
    esize = storage.element_size()
    view = CacheView(storage.data_ptr(), storage.data_ptr() + (elems // 2) * esize, table, elems, 16,
                     page_tokens, kv_heads, head_dim, dtype)
    return storage, table, view


def _rope_ref(x, pos, inv_freq):
    half = x.shape[-1] // 2
    ang = (pos.float().unsqueeze(-1) * inv_freq).double()
    c, s = torch.cos(ang).unsqueeze(1), torch.sin(ang).unsqueeze(1)
    lo, hi = x[..., :half].double(), x[..., half:].double()
    return torch.cat([lo * c - hi * s, hi * c + lo * s], -1)


@pytest.mark.parametrize("dtype,lens", [(torch.float32, [21, 5]), (torch.bfloat16, [21, 5]), (torch.bfloat16, [75, 8])])
def test_rope_cache_write_and_attention_plain(dtype, lens):
    """Rotation + cache write, then attention over scrambled pages with a window, against dense math
    (75 + 8 tokens of one finished bfloat16 input take the vector kernel)."""
    from bare_cuda_4gib_b200.kernels import lib as K
    heads, kv_heads, d, page, window = 6, 2, 48, 8, 13
    storage, table, view = _paged_cache(kv_heads, d, page, 14, dtype)
    pages = list(range(14))
    random.Random(3).shuffle(pages)
    n0 = -(-lens[0] // page)
    table[0, :n0] = torch.tensor(pages[:n0], dtype=torch.int32)
    table[1, :1] = torch.tensor(pages[n0: n0 + 1], dtype=torch.int32)
    n = sum(lens)
    positions = torch.tensor(list(range(lens[0])) + list(range(lens[1])), dtype=torch.int32, device=DEV)
    row_seq = torch.tensor([0] * lens[0] + [1] * lens[1], dtype=torch.int32, device=DEV)
    width = (heads + 2 * kv_heads) * d
    parts = 1 if n >= 64 else 2                                    # partial results (one: the vector kernel)
    qkv = torch.randn(parts, n, width, device=DEV).to(dtype)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(d // 2, dtype=torch.float32) * 2.0 / d))).to(DEV)
    q = torch.empty(n, heads * d, device=DEV, dtype=dtype)
    K.rope_cache_write(K.Partials(qkv, parts) if parts > 1 else K.Partials(qkv[0]), q, view, positions, row_seq,
                       inv_freq, heads, True, n)
    full = qkv.float().sum(0)
    qr = _rope_ref(full[:, : heads * d].view(n, heads, d), positions, inv_freq)
    kr = _rope_ref(full[:, heads * d: (heads + kv_heads) * d].view(n, kv_heads, d), positions, inv_freq)
    vr = full[:, (heads + kv_heads) * d:].view(n, kv_heads, d).double()
    tol = 1e-5 if dtype == torch.float32 else 2 ** -7
    _close(q.view(n, heads, d), qr, tol, tol)
    out = torch.empty(n, heads * d, device=DEV, dtype=dtype)
    scale = 1.0 / math.sqrt(d)
    K.attention_plain(q, out, view, positions, row_seq, heads, n, scale, window)
    # dense reference from what the kernels stored (q as stored, k/v rounded as the cache holds them)
    qs = q.view(n, heads, d).double()
    ks, vs = kr.to(dtype).double(), vr.to(dtype).double()
    want = torch.zeros(n, heads, d, dtype=torch.float64, device=DEV)
    start = 0
    for L in lens:
        for i in range(L):
            lo = max(0, i - window + 1)
            for h in range(heads):
                kvh = h // (heads // kv_heads)
                s = (ks[start + lo: start + i + 1, kvh] @ qs[start + i, h]) * scale
                p = torch.softmax(s, 0)
                want[start + i, h] = p @ vs[start + lo: start + i + 1, kvh]
        start += L
    _close(out.view(n, heads, d), want, 1e-5 if dtype == torch.float32 else 2 ** -7, 1e-5 if dtype == torch.float32 else 2e-3)


def test_attention_plain_far_key_stands_out():
    """One far key among hundreds gets a large score: the output must be its value row."""
    from bare_cuda_4gib_b200.kernels import lib as K
    heads, kv_heads, d, page = 2, 1, 32, 16
    L = 300
    storage, table, view = _paged_cache(kv_heads, d, page, 19, torch.float32)
    from bare_cuda_4gib_b200.kernels.lib import CacheView
    table = torch.full((1, 32), -1, dtype=torch.int32, device=DEV)
    perm = list(range(19))
    random.Random(1).shuffle(perm)
    table[0, :19] = torch.tensor(perm, dtype=torch.int32)
    view.block_table, view.table_stride = table, 32
    k = 0.01 * torch.randn(L, d, device=DEV)
    v = torch.randn(L, d, device=DEV)
    far = 37
    k[far] = 0
    k[far, 0] = 100.0
    for pos in range(L):
        pg = perm[pos // page]
        storage[pg, (pos % page) * d: (pos % page) * d + d] = k[pos]
        storage[pg, page * d + (pos % page) * d: page * d + (pos % page) * d + d] = v[pos]
    q = torch.zeros(1, heads * d, device=DEV)
    q[0, 0] = 10.0
    q[0, d] = 10.0
    out = torch.empty(1, heads * d, device=DEV)
    positions = torch.tensor([L - 1], dtype=torch.int32, device=DEV)
    row_seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.attention_plain(q, out, view, positions, row_seq, heads, 1, 1.0 / math.sqrt(d), 0)
    _close(out.view(heads, d), v[far].expand(heads, d), 1e-5, 1e-5)


@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                                (torch.bfloat16, torch.bfloat16)])
def test_swiglu(in_dtype, out_dtype):
    from bare_cuda_4gib_b200.kernels import lib as K
    rows, inter = 5, 173
    x = torch.randn(2, rows, 2 * inter, device=DEV).to(in_dtype)
    out = torch.empty(rows, inter, device=DEV, dtype=out_dtype)
    K.swiglu(K.Partials(x, 2), out, rows)
    s = x[0].float() + x[1].float()
    g, u = s[:, :inter].double(), s[:, inter:].double()
    want = g / (1 + torch.exp(-g)) * u
    _close(out, want, 1e-5 if out_dtype == torch.float32 else 2 ** -8, 1e-6)


def test_argmax_rows_ties_and_last():
    from bare_cuda_4gib_b200.kernels import lib as K
    logits = torch.randn(4, 1000, device=DEV)
    logits[1, 10] = logits[1, 700] = 50.0      # tie: the lowest index wins
    logits[2, 999] = 60.0                      # last slot
    logits[3] = 0.0                            # all equal
    out = torch.empty(4, dtype=torch.int32, device=DEV)
    K.argmax_rows(logits, out, 4)
    assert out.tolist() == [int(logits[0].argmax()), 10, 999, 0]


def test_sample_rows_matches_inverse_cdf_walk():
    import plain_llama as pl
    from bare_cuda_4gib_b200.kernels import lib as K
    vocab, rows = 777, 6
    logits = 3 * torch.randn(rows, vocab, device=DEV)
    temps = torch.tensor([0.0, 0.7, 1.0, 1.5, 0.3, 2.0], device=DEV)
    us = torch.tensor([0.5, 0.01, 0.5, 0.999, 0.25, 0.75], device=DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    K.sample_rows(logits, temps, us, out, rows)
    got = out.tolist()
    assert got[0] == int(logits[0].argmax())
    for r in range(1, rows):
        w = pl.sampling_weights(logits[r].cpu(), float(temps[r]))
        want = pl.inverse_cdf_pick(w.tolist(), list(range(vocab)), float(us[r]))
        # float32 sums on the device may move the boundary by one id with negligible mass
        cdf = torch.cumsum(w / w.sum(), 0)
        assert abs(float(cdf[got[r]]) - float(cdf[want])) < 1e-4, (r, got[r], want)


# ------------------------------------------------------------------------------ tcgen05 GEMM

GEMM_SHAPES = [(1, 2560, 2048), (7, 96, 96), (16, 300, 176), (17, 128, 64), (33, 1000, 128),
               (64, 2048, 5632), (100, 512, 256), (200, 640, 320), (257, 384, 192), (700, 256, 512),
               (300, 1000, 96), (1000, 2560, 264), (513, 130, 176), (2048, 2048, 512)]


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tcgen05(m, n, k, out_dtype):
    from bare_cuda_4gib_b200.kernels import gemm
    torch.manual_seed(m * 7 + n)
    ctx = _ctx()
    a = ctx.ws.get("a", (m, k), torch.bfloat16)
    a.copy_(torch.randn(m, k, device=DEV))
    w = torch.randn(n, k, device=DEV).to(torch.bfloat16)
    plan = gemm.plan_for(w)
    assert plan is not None
    res = gemm.run(ctx, plan, a, m, out_dtype, "out", allow_partials=True, swiglu=False)
    gemm.check_errors()
    got = res.tensor.float().sum(0) if res.n > 1 else res.tensor.float()
    want = a.double() @ w.double().t()
    if out_dtype == torch.float32:
        _close(got, want, 1e-5, 1e-4 * math.sqrt(k))
    else:
        _close(got, want, 2 ** -8, 1e-4 * math.sqrt(k))


class _RowNorm:
    """What a product needs to know of the norm that reads the residual stream after it."""

    prenormable = True

    def __init__(self, weight, eps):
        self.tensors, self.params = {"weight": weight}, {"eps": eps}


@pytest.mark.parametrize("m,n,k,bn", [(300, 1000, 96, 0), (513, 132, 176, 0), (2048, 2048, 512, 0), (2048, 5120, 128, 256),
                                      (1100, 3000, 192, 256), (257, 72, 64, 0), (700, 1000, 64, 144), (2048, 2048, 64, 128),
                                      (1500, 1284, 128, 96)])
@pytest.mark.parametrize("w_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05_adds_into_the_residual_and_prepares_the_next_norm(m, n, k, bn, w_dtype, monkeypatch):
    """Many-token products that add themselves into the float32 residual stream (both the
    two-blocks-per-SM kernel and, with wide tiles and more tiles than SMs, the persistent one) and
    leave bfloat16(new residual * the next norm's weight) with the rows' sums of squares; then the
    product that reads that norm, plain and with SwiGLU, against the norm and product in float64."""
    from bare_cuda_4gib_b200.kernels import gemm
    from bare_cuda_4gib_b200.kernels import lib as K
    if bn:
        monkeypatch.setenv("BARE_CUDA_B200_GEMM_BN", str(bn))
    torch.manual_seed(m + n)
    ctx = _ctx()
    a = ctx.ws.get("a", (m, k), torch.bfloat16)
    a.copy_(torch.randn(m, k, device=DEV))
    w = torch.randn(n, k, device=DEV).to(torch.bfloat16)
    residual = torch.randn(m + 5, n, device=DEV)
    before = residual.double().clone()
    eps = 1e-5
    norm = _RowNorm((1 + 0.3 * torch.randn(n, device=DEV)).to(w_dtype), eps)
    assert gemm.run(ctx, gemm.plan_for(w), a, m, torch.float32, "out", True, False,
                    epilogue=K.AddTo(residual[:m], norm)) is None
    gemm.check_errors()
    want = before.clone()
    want[:m] += a.double() @ w.double().t()
    _close(residual, want, 1e-5, 1e-4 * math.sqrt(k))
    pre = ctx.prenormed
    assert pre is not None and pre.norm is norm
    now = residual[:m].double()
    nw = norm.tensors["weight"].double()
    _close(pre.x[:m].float(), now * nw, 2 ** -8, 1e-6)
    sq = pre.sq[: pre.items, :m].double().sum(0)
    _close(sq, now.square().sum(-1), 1e-5, 1e-5)
    monkeypatch.delenv("BARE_CUDA_B200_GEMM_BN", raising=False)
    if n % 8:
        return     # (the consumer's activations need rows of a multiple of 8 elements)
    # ---- the consumers: x = rms_norm(residual) * weight is never formed; the factor goes on the sums.
    # The reference takes the same bfloat16 input (pre.x) and applies the factor in float64, so what
    # is left to differ is the order of the sums and the rounding of the output.
    normed = pre.x[:m].double() * torch.rsqrt(now.square().mean(-1, keepdim=True) + eps)
    _close(normed, now * torch.rsqrt(now.square().mean(-1, keepdim=True) + eps) * nw, 2 ** -8, 1e-6)
    for swiglu in (False, True):
        n2 = 384
        w2 = (torch.randn(n2, n, device=DEV) / math.sqrt(n)).to(torch.bfloat16)
        lazy = K.LazyNorm(ctx, residual, norm.tensors["weight"], eps, m, None, "normed", pre)
        res = gemm.run(ctx, gemm.plan_for(w2), lazy, m, torch.bfloat16, "out2", False, swiglu)
        gemm.check_errors()
        full = normed @ w2.double().t()
        if swiglu:
            gate, up = full[:, : n2 // 2], full[:, n2 // 2:]
            full = gate / (1 + torch.exp(-gate)) * up
        _close(res.tensor.float(), full, 2 ** -8, 1e-4)


def test_gemm_tcgen05_leaves_the_add_to_its_caller_when_no_norm_can_be_prepared():
    """An adding epilogue whose following norm is unknown, or not one whose factor is a single number
    per row, is not the kernel's: the plain product comes back and the residual stream is untouched."""
    from bare_cuda_4gib_b200.kernels import gemm
    from bare_cuda_4gib_b200.kernels import lib as K
    torch.manual_seed(5)
    m, n, k = 300, 256, 128
    ctx = _ctx()
    a = ctx.ws.get("a", (m, k), torch.bfloat16)
    a.copy_(torch.randn(m, k, device=DEV))
    w = torch.randn(n, k, device=DEV).to(torch.bfloat16)
    residual = torch.randn(m, n, device=DEV)
    before = residual.clone()
    other = types.SimpleNamespace(prenormable=False, tensors={"weight": torch.ones(n, device=DEV)}, params={"eps": 1e-5})
    for then in (None, other):
        res = gemm.run(ctx, gemm.plan_for(w), a, m, torch.float32, "out", True, False, epilogue=K.AddTo(residual, then))
        gemm.check_errors()
        assert res is not None and ctx.prenormed is None
        assert torch.equal(residual, before)
        _close(res.tensor.float().sum(0) if res.n > 1 else res.tensor.float(), a.double() @ w.double().t(), 1e-5, 1e-4 * math.sqrt(k))


@pytest.mark.parametrize("m,inter,k", [(3, 176, 64), (40, 5632, 256), (130, 256, 96), (300, 200, 128), (9, 2816, 512),
                                       (700, 176, 64), (2048, 5632, 128), (257, 1000, 96), (90, 1408, 128), (100, 5632, 128),
                                       (200, 1000, 96), (256, 2816, 320)])
def test_gemm_tcgen05_swiglu(m, inter, k):
    from bare_cuda_4gib_b200.kernels import gemm
    torch.manual_seed(m)
    ctx = _ctx()
    a = ctx.ws.get("a", (m, k), torch.bfloat16)
    a.copy_(torch.randn(m, k, device=DEV) * 0.5)
    w = (torch.randn(2 * inter, k, device=DEV) * 0.2).to(torch.bfloat16)
    plan = gemm.plan_for(w)
    res = gemm.run(ctx, plan, a, m, torch.bfloat16, "act", allow_partials=False, swiglu=True)
    gemm.check_errors()
    gu = a.double() @ w.double().t()
    g, u = gu[:, :inter], gu[:, inter:]
    want = g / (1 + torch.exp(-g)) * u
    _close(res.tensor, want, 2 ** -7, 1e-3)


def test_a_bounded_wait_runs_out_and_the_kernel_returns():
    """Every wait inside the pipelined kernels has a limit.  Here one is seen to run out: with the
    test hooks of the GEMM library the producer arms one stage's barrier and issues no copy for it,
    and the wait limit is 2 ms.  The MMA issuer must give up, say so in the error word, the kernel
    must release its tensor memory and return on its own, and the next ordinary launch must be right."""
    import time
    from ctypes import c_int, c_longlong
    from bare_cuda_4gib_b200.errors import KernelLaunchError
    from bare_cuda_4gib_b200.kernels import gemm
    torch.manual_seed(4)
    m, n, k = 40, 256, 256                     # four k blocks, all in the ring at once: only the MMA issuer waits
    ctx = _ctx()
    a = ctx.ws.get("a", (m, k), torch.bfloat16)
    a.copy_(torch.randn(m, k, device=DEV) * 0.5)
    w = (torch.randn(n, k, device=DEV) * 0.2).to(torch.bfloat16)
    plan = gemm.plan_for(w)
    want = a.double() @ w.double().t()
    gemm.check_errors()
    hooks = gemm.lib().llm_gemm_test_hooks
    hooks.argtypes, hooks.restype = [c_longlong, c_int], None
    hooks(2_000_000, 2)
    try:
        started = time.time()
        gemm.run(ctx, plan, a, m, torch.float32, "out", allow_partials=False, swiglu=False)
        torch.cuda.synchronize()               # returns: nothing waits for ever
        took = time.time() - started
        with pytest.raises(KernelLaunchError, match="gemm MMA issuer"):
            gemm.check_errors()
    finally:
        hooks(0, -1)
    assert took < 1.0, f"the kernel took {took:.2f} s to give up"
    res = gemm.run(ctx, plan, a, m, torch.float32, "out", allow_partials=False, swiglu=False)
    gemm.check_errors()
    _close(res.tensor, want, 1e-5, 2e-3)


# ------------------------------------------------------------------------------ tensor-core attention

def _attention_case(seqs, heads, kv_heads, d, page, window, seed, far_key=False, drop_passed=False,
                    poison_tail=True, jumps=()):
    """seqs: [(q_len, kv_len)].  Fills a scrambled paged cache, runs the attention the launcher picks
    and the dense reference.  `drop_passed` (with a window): pages that every query of the step has
    passed are taken out of the block table and filled with NaN, as the cache manager gives them back.
    `poison_tail`: positions at and beyond a request's length in its last page hold NaN, as a page
    may that an earlier, longer request left behind.  `jumps`: [(position, level)]: the key at that
    position scores about `level` (in powers of two) above an ordinary key for every query, so the
    running maximum of a row jumps there."""
    from bare_cuda_4gib_b200.kernels import attention as fast
    from bare_cuda_4gib_b200.kernels.lib import CacheView

    torch.manual_seed(seed)
    g = heads // kv_heads
    max_blocks = max(-(-kv // page) for _, kv in seqs)
    n_pages = sum(-(-kv // page) for _, kv in seqs) + 3
    elems = 2 * kv_heads * page * d
    storage = torch.zeros(n_pages, elems, device=DEV, dtype=torch.bfloat16)
    storage[-1].fill_(float("nan"))           # a page nobody owns: reading it would poison the result
    table = torch.full((len(seqs), max_blocks + 1), -1, dtype=torch.int32, device=DEV)
    perm = list(range(n_pages - 1))
    random.Random(seed).shuffle(perm)
    ks, vs, at = [], [], 0
    for s, (q_len, kv_len) in enumerate(seqs):
        k = torch.randn(kv_len, kv_heads, d, device=DEV).to(torch.bfloat16)
        v = torch.randn(kv_len, kv_heads, d, device=DEV).to(torch.bfloat16)
        if far_key:
            k = (0.05 * k.float()).to(torch.bfloat16)
            k[3 % kv_len] = 0
            k[3 % kv_len, :, 0] = 60.0
        for pos, level in jumps:
            if pos < kv_len:      # score = 8 * k[0] / sqrt(d) in natural units
                k[pos, :, 0] = level * math.log(2.0) * math.sqrt(d) / 8.0
        nb = -(-kv_len // page)
        pages = perm[at: at + nb]
        at += nb
        table[s, :nb] = torch.tensor(pages, dtype=torch.int32)
        sv = storage.view(n_pages, 2, kv_heads, page, d)
        for b, pg in enumerate(pages):
            lo, hi = b * page, min(kv_len, (b + 1) * page)
            sv[pg, 0, :, : hi - lo] = k[lo:hi].transpose(0, 1)
            sv[pg, 1, :, : hi - lo] = v[lo:hi].transpose(0, 1)
            if poison_tail and hi - lo < page:
                sv[pg, :, :, hi - lo:] = float("nan")
        if drop_passed and window > 0:
            passed = max(0, kv_len - q_len - window + 1) // page      # blocks wholly below the first query's window
            for b in range(passed):
                sv[pages[b]] = float("nan")
            table[s, :passed] = -1
        ks.append(k)
        vs.append(v)
    esize = 2
    view = CacheView(storage.data_ptr(), storage.data_ptr() + (elems // 2) * esize, table, elems, table.shape[1],
                     page, kv_heads, d, torch.bfloat16, storage.data_ptr(), storage.numel())
    n = sum(q for q, _ in seqs)
    q = torch.randn(n, heads, d, device=DEV).to(torch.bfloat16)
    if far_key:
        q = torch.zeros_like(q)
        q[:, :, 0] = 4.0
    if jumps:
        q = (0.1 * q.float()).to(torch.bfloat16)
        q[:, :, 0] = 8.0
    starts = [sum(x for x, _ in seqs[:i]) for i in range(len(seqs))]
    ctx = _ctx()
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    ctx.seq_q_start, ctx.seq_q_len, ctx.seq_kv_len = i32(starts), i32([a for a, _ in seqs]), i32([b for _, b in seqs])
    ctx.token_ids = i32([0])
    ctx.host_q_len, ctx.host_kv_len = [a for a, _ in seqs], [b for _, b in seqs]
    ctx.max_q_len, ctx.max_kv_len = max(ctx.host_q_len), max(ctx.host_kv_len)
    ctx.extras = {}
    out = torch.full((n, heads * d), float("nan"), device=DEV, dtype=torch.bfloat16)
    plan = fast.plan_for(d, heads, kv_heads)
    scale = 1.0 / math.sqrt(d)
    fast.run(ctx, plan, q.view(n, heads * d), out, view, scale, window)
    from bare_cuda_4gib_b200.kernels import gemm
    gemm.check_errors()
    want = torch.zeros(n, heads, d, dtype=torch.float64, device=DEV)
    for s, (q_len, kv_len) in enumerate(seqs):
        pos = torch.arange(kv_len - q_len, kv_len, device=DEV)[:, None]
        key = torch.arange(kv_len, device=DEV)[None, :]
        hidden = key > pos
        if window > 0:
            hidden = hidden | (key < pos - window + 1)
        for kvh in range(kv_heads):          # one key/value head at a time keeps the score matrix small
            qs = q[starts[s]: starts[s] + q_len, kvh * g: (kvh + 1) * g].double()            # [q, g, d]
            sc = torch.einsum("qgd,kd->gqk", qs, ks[s][:, kvh].double()) * scale
            sc = sc.masked_fill(hidden[None], float("-inf"))
            want[starts[s]: starts[s] + q_len, kvh * g: (kvh + 1) * g] = \
                torch.einsum("gqk,kd->qgd", torch.softmax(sc, -1), vs[s][:, kvh].double())
    return out.view(n, heads, d), want, ctx


@pytest.mark.parametrize("heads,kv_heads,d,page", [(8, 1, 64, 64), (6, 2, 32, 16), (4, 4, 128, 32), (32, 2, 16, 16),
                                                   (5, 5, 64, 64), (12, 4, 64, 16)])
def test_attention_mma_prefill_and_mixed(heads, kv_heads, d, page):
    # whole prompts, a portion after a cached prefix, and single decode rows beside them
    seqs = [(37, 37), (5, 133), (1, 70), (64, 64), (2, 2), (1, 1), (19, 300)]
    got, want, _ = _attention_case(seqs, heads, kv_heads, d, page, 0, seed=heads + d)
    _close(got, want, 2 ** -7, 4e-3)


@pytest.mark.parametrize("heads,kv_heads,d,page", [(32, 4, 64, 64), (3, 1, 32, 32), (16, 16, 128, 16), (16, 1, 64, 64)])
def test_attention_mma_decode_split(heads, kv_heads, d, page, monkeypatch):
    monkeypatch.setenv("BARE_CUDA_B200_NO_DECODE_ATTENTION", "1")          # the mma.sync kernel's own decode shape
    seqs = [(1, 2048), (1, 1), (1, 65), (1, 700)]
    got, want, ctx = _attention_case(seqs, heads, kv_heads, d, page, 0, seed=d)
    if heads // kv_heads <= 16:
        assert any(v[3] == 16 and v[4] > 1 for k, v in ctx.extras.items())   # the split shape ran
    _close(got, want, 2 ** -7, 4e-3)


def test_attention_mma_window_and_far_key():
    got, want, _ = _attention_case([(40, 200), (1, 150), (90, 90)], 4, 2, 64, 16, 50, seed=1)
    _close(got, want, 2 ** -7, 4e-3)
    # prompt portions behind a window whose passed pages are gone (the tcgen05 kernel at head size 64,
    # the mma.sync kernel at 32)
    for d in (64, 32):
        got, want, _ = _attention_case([(40, 300), (3, 150), (70, 500)], 4, 2, d, 16, 60, seed=3, drop_passed=True)
        _close(got, want, 2 ** -7, 4e-3)
    # one early key dominates every query: the output must be that key's value row
    got, want, _ = _attention_case([(1, 900), (33, 500)], 8, 2, 64, 64, 0, seed=2, far_key=True)
    _close(got, want, 2 ** -7, 4e-3)


@pytest.mark.parametrize("d,heads,kv_heads", [(64, 8, 2), (128, 4, 2)])
@pytest.mark.parametrize("page", [16, 64])
def test_attention_tcgen05_long_contexts_random_data(d, heads, kv_heads, page):
    """Random queries, keys and values at the lengths the benchmark runs: a whole 2,048-token
    prompt, portions after long cached prefixes and a single row beside them.  The kernel's ring of
    key/value stages and its two P buffers wrap many times here, and every key carries weight, so
    a stale stage or a missed key shows in the values."""
    from bare_cuda_4gib_b200.kernels import attention as fast
    seqs = [(2048, 2048), (300, 1500), (5, 1900), (1, 1000), (130, 641)]
    got, want, ctx = _attention_case(seqs, heads, kv_heads, d, page, 0, seed=d + page)
    plan = fast.plan_for(d, heads, kv_heads)
    assert plan.tc is not None and any(v[3] == plan.prefill_rows for k, v in ctx.extras.items())   # the tcgen05 kernel ran
    _close(got, want, 2 ** -7, 4e-3)


@pytest.mark.parametrize("d,heads,kv_heads", [(64, 8, 2), (128, 4, 2)])
def test_attention_tcgen05_rescales_when_a_rows_maximum_jumps(d, heads, kv_heads):
    """With random data a row's maximum settles within its first keys and the accumulated output is
    never rescaled again.  Here single keys score 2^12 above everything before them, in the first
    and in the second half of a block of 128 keys and several blocks apart, so that the
    probabilities already written for the block's first half, the row sums and the accumulator in
    tensor memory all have to be rescaled: a missed or doubled rescale is off by a factor of 4,096."""
    from bare_cuda_4gib_b200.kernels import attention as fast
    jumps = [(200, 12), (300, 24), (700, 36), (1000, 48), (1001, 60)]
    seqs = [(1200, 1200), (300, 1100), (140, 333)]
    got, want, ctx = _attention_case(seqs, heads, kv_heads, d, 64, 0, seed=d, jumps=jumps)
    plan = fast.plan_for(d, heads, kv_heads)
    assert plan.tc is not None and any(v[3] == plan.prefill_rows for k, v in ctx.extras.items())   # the tcgen05 kernel ran
    _close(got, want, 2 ** -7, 4e-3)


@pytest.mark.parametrize("d,heads,kv_heads,page", [(64, 32, 4, 64), (128, 8, 8, 16), (64, 6, 2, 32)])
def test_attention_decode_long_contexts_random_data(d, heads, kv_heads, page):
    """The cluster decode kernel over contexts of up to 2,048 keys of random data, requests of very
    different lengths in one step, with NaN behind each request's last key."""
    seqs = [(1, 2048), (1, 1), (1, 63), (1, 64), (1, 65), (1, 1337), (2, 2000), (1, 511)]
    got, want, ctx = _attention_case(seqs, heads, kv_heads, d, page, 0, seed=3 * d + page)
    assert any(v[5] > 0 for k, v in ctx.extras.items())       # the cluster decode kernel ran
    _close(got, want, 2 ** -7, 4e-3)


# ------------------------------------------------------------------------------ few-token fused product

def _gemv_input(tokens, k, norm, ctx):
    """x as the kernel takes it (a LazyNorm over a residual stream, or a bfloat16 matrix) and as float64."""
    from bare_cuda_4gib_b200.kernels import lib as K
    if norm:
        residual = torch.randn(tokens + 3, k, device=DEV) * 1.5
        weight = (1.0 + 0.1 * torch.randn(k, device=DEV)).to(torch.bfloat16)
        rows = torch.tensor([(i * 2) % (tokens + 3) for i in range(tokens)], dtype=torch.int32, device=DEV)
        eps = 1e-5
        r = residual[rows.long()].double()
        want = r / torch.sqrt((r * r).mean(-1, keepdim=True) + eps) * weight.double()
        # the kernel rounds the normed input to bfloat16 once, as the unfused kernel does
        return K.LazyNorm(ctx, residual, weight, eps, tokens, rows, "normed"), want.to(torch.bfloat16).double()
    x = torch.randn(tokens, k, device=DEV).to(torch.bfloat16)
    return x, x.double()


@pytest.mark.parametrize("tokens,n,k", [(1, 70, 64), (8, 258, 96), (5, 2048, 352), (13, 100, 2048), (16, 33, 2816), (8, 40, 5632),
                                        (3, 1000, 1408)])
@pytest.mark.parametrize("norm", [False, True])
def test_gemv_fused_plain_and_add(tokens, n, k, norm):
    from bare_cuda_4gib_b200.kernels import gemm, gemv
    from bare_cuda_4gib_b200.kernels import lib as K
    torch.manual_seed(tokens * 31 + n)
    ctx = _ctx()
    ctx.dtype = torch.bfloat16
    w = (torch.randn(n, k, device=DEV) * 0.1).to(torch.bfloat16)
    assert gemv.supports(w) and gemv.takes(tokens, k)
    assert not gemv.takes(16, 5632) and not gemv.takes(8, 40)     # x does not fit beside the ring; k no multiple of 32
    x, xd = _gemv_input(tokens, k, norm, ctx)
    want = xd @ w.double().t()
    for out_dtype in (torch.float32, torch.bfloat16):
        got = gemv.run(ctx, w, x, tokens, out_dtype, "out", False, None).tensor
        _close(got, want, 1e-5 if out_dtype == torch.float32 else 2 ** -8, 2e-4 * math.sqrt(k))
    target = torch.randn(tokens, n, device=DEV)
    before = target.double().clone()
    assert gemv.run(ctx, w, x, tokens, torch.float32, "out", False, K.AddTo(target)) is None
    gemm.check_errors()
    _close(target, before + want, 1e-5, 2e-4 * math.sqrt(k))


@pytest.mark.parametrize("tokens,inter,k", [(2, 176, 64), (8, 100, 96), (16, 5632, 2048), (7, 13, 160)])
@pytest.mark.parametrize("norm", [False, True])
def test_gemv_fused_swiglu(tokens, inter, k, norm):
    from bare_cuda_4gib_b200.kernels import gemm, gemv
    torch.manual_seed(inter)
    ctx = _ctx()
    ctx.dtype = torch.bfloat16
    w = (torch.randn(2 * inter, k, device=DEV) * 0.2).to(torch.bfloat16)
    x, xd = _gemv_input(tokens, k, norm, ctx)
    got = gemv.run(ctx, w, x, tokens, torch.bfloat16, "act", True, None).tensor
    gemm.check_errors()
    gu = xd @ w.double().t()
    g, u = gu[:, :inter], gu[:, inter:]
    _close(got, g / (1 + torch.exp(-g)) * u, 2 ** -7, 2e-3)


@pytest.mark.parametrize("heads,kv_heads,d,page", [(6, 2, 48, 8), (32, 4, 64, 64), (3, 1, 128, 32), (4, 4, 16, 16)])
@pytest.mark.parametrize("rotate", [True, False])
def test_gemv_fused_rotation_and_cache_write(heads, kv_heads, d, page, rotate):
    """[q; k; v] product, rotation by position and the write into scrambled pages in one kernel,
    for tokens of two requests at different positions."""
    from bare_cuda_4gib_b200.kernels import gemm, gemv
    from bare_cuda_4gib_b200.kernels import lib as K
    torch.manual_seed(d)
    k_in, tokens = 96, 9
    ctx = _ctx()
    ctx.dtype = torch.bfloat16
    storage, table, view = _paged_cache(kv_heads, d, page, 16, torch.bfloat16)
    pages = list(range(16))
    random.Random(5).shuffle(pages)
    table[0, :8] = torch.tensor(pages[:8], dtype=torch.int32)
    table[1, :8] = torch.tensor(pages[8:], dtype=torch.int32)
    # request 0 brings 6 tokens from position 3 * page - 2 on (crossing a page edge), request 1 three from 0
    p0 = 3 * page - 2
    positions = torch.tensor(list(range(p0, p0 + 6)) + [0, 1, 2], dtype=torch.int32, device=DEV)
    row_seq = torch.tensor([0] * 6 + [1] * 3, dtype=torch.int32, device=DEV)
    width = (heads + 2 * kv_heads) * d
    w = (torch.randn(width, k_in, device=DEV) * 0.2).to(torch.bfloat16)
    x, xd = _gemv_input(tokens, k_in, True, ctx)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(d // 2, dtype=torch.float32) * 2.0 / d))).to(DEV) if rotate else None
    q = torch.full((tokens, heads * d), float("nan"), device=DEV, dtype=torch.bfloat16)
    epilogue = K.RotateAndCache(q, view, positions, row_seq, inv_freq, heads, True)
    assert gemv.run(ctx, w, x, tokens, torch.float32, "qkv", False, epilogue) is None
    gemm.check_errors()
    full = xd @ w.double().t()
    qw = full[:, : heads * d].view(tokens, heads, d)
    kw = full[:, heads * d: (heads + kv_heads) * d].view(tokens, kv_heads, d)
    vw = full[:, (heads + kv_heads) * d:].view(tokens, kv_heads, d)
    if rotate:
        qw, kw = _rope_ref(qw, positions, inv_freq), _rope_ref(kw, positions, inv_freq)
    _close(q.view(tokens, heads, d), qw, 2 ** -7, 2e-3)
    sv = storage.view(16, 2, kv_heads, page, d)
    for t in range(tokens):
        pos, seq = int(positions[t]), int(row_seq[t])
        pg = int(table[seq, pos // page])
        _close(sv[pg, 0, :, pos % page], kw[t], 2 ** -7, 2e-3)
        _close(sv[pg, 1, :, pos % page], vw[t], 2 ** -7, 2e-3)
    # nothing else was written: every other cache position is still zero
    written = torch.zeros(16, page, dtype=torch.bool, device=DEV)
    for t in range(tokens):
        pos, seq = int(positions[t]), int(row_seq[t])
        written[int(table[seq, pos // page]), pos % page] = True
    assert float(sv.float().abs().amax(dim=(1, 2, 4))[~written].max()) == 0.0


# ------------------------------------------------------------------------------ cluster decode attention

@pytest.mark.parametrize("heads,kv_heads,d,page", [(32, 4, 64, 64), (8, 8, 64, 16), (16, 2, 128, 32), (6, 3, 64, 8),
                                                   (16, 1, 128, 64)])
@pytest.mark.parametrize("splits", [0, 1, 3, 8])
def test_attention_decode_cluster(heads, kv_heads, d, page, splits, monkeypatch):
    """Single decode rows of requests of very different lengths (one key, a page's edge, thousands),
    with the number of blocks per cluster forced to 1, 3 and 8 and left to the launcher (0)."""
    if splits:
        monkeypatch.setenv("BARE_CUDA_B200_ATTN_SPLITS", str(splits))
    seqs = [(1, 2049), (1, 1), (1, page), (1, page + 1), (1, 700)]
    got, want, ctx = _attention_case(seqs, heads, kv_heads, d, page, 0, seed=d + splits)
    ran = [v for k, v in ctx.extras.items() if isinstance(k, tuple) and k[0] == "attention_tiles"]
    assert ran and ran[0][5] >= 1, "the cluster decode kernel did not run"
    _close(got, want, 2 ** -7, 4e-3)


def test_attention_decode_two_tokens_window_and_far_key(monkeypatch):
    # two tokens per request still fit the 16 packed rows of a tile when the group has at most 8 heads
    got, want, ctx = _attention_case([(2, 300), (2, 2), (1, 77), (2, 1030)], 16, 2, 64, 16, 0, seed=11)
    assert [v for k, v in ctx.extras.items() if isinstance(k, tuple)][0][5] >= 1
    _close(got, want, 2 ** -7, 4e-3)
    # a window: keys older than 50 positions do not count, whole key blocks below it are never read
    got, want, _ = _attention_case([(1, 200), (2, 150), (1, 40)], 4, 2, 64, 16, 50, seed=12)
    _close(got, want, 2 ** -7, 4e-3)
    # ... and the pages the window has passed are gone from the block table (a key block of 64 then
    # straddles pages that are held and pages that are not)
    for page in (16, 32, 64):
        got, want, ctx = _attention_case([(1, 300), (2, 131), (1, 40), (1, 1000)], 8, 2, 64, page, 70, seed=14,
                                         drop_passed=True)
        assert [v for k, v in ctx.extras.items() if isinstance(k, tuple)][0][5] >= 1
        _close(got, want, 2 ** -7, 4e-3)
    # one early key among a thousand dominates: the output must be that key's value row
    monkeypatch.setenv("BARE_CUDA_B200_ATTN_SPLITS", "8")
    got, want, _ = _attention_case([(1, 1900), (1, 500)], 8, 2, 64, 64, 0, seed=13, far_key=True)
    _close(got, want, 2 ** -7, 4e-3)


@pytest.mark.parametrize("tokens,hidden,inter", [(8, 96, 64), (3, 352, 1408), (16, 2048, 160)])
def test_gemv_fused_add_then_prenormed_input(tokens, hidden, inter):
    """A product that adds into the residual stream and, asked to, leaves bfloat16(residual * w) and
    the rows' sums of squares; the next product norms its input from those.  Both against float64."""
    import types as _types
    from bare_cuda_4gib_b200.kernels import gemm, gemv
    from bare_cuda_4gib_b200.kernels import lib as K
    torch.manual_seed(hidden + tokens)
    ctx = _ctx()
    ctx.dtype = torch.bfloat16
    eps = 1e-6
    norm = _types.SimpleNamespace(prenormable=True, params={"eps": eps, "size": hidden},
                                  tensors={"weight": (1.0 + 0.2 * torch.randn(hidden, device=DEV)).to(torch.bfloat16)})
    residual = torch.randn(tokens + 2, hidden, device=DEV) * 2.0
    before = residual.double().clone()
    w_down = (torch.randn(hidden, inter, device=DEV) * 0.3).to(torch.bfloat16)
    act = torch.randn(tokens, inter, device=DEV).to(torch.bfloat16)
    assert gemv.run(ctx, w_down, act, tokens, torch.float32, "out", False, K.AddTo(residual, norm)) is None
    left = ctx.prenormed
    assert left is not None and left.norm is norm
    now = before.clone()
    now[:tokens] += act.double() @ w_down.double().t()
    _close(residual, now, 1e-5, 1e-4 * math.sqrt(inter))
    # the next product: wanted rows in another order, its input normed from what was left
    rows = torch.tensor(list(reversed(range(tokens))), dtype=torch.int32, device=DEV)
    w_next = (torch.randn(70, hidden, device=DEV) * 0.1).to(torch.bfloat16)
    lazy = K.LazyNorm(ctx, residual, norm.tensors["weight"], eps, tokens, rows, "normed", left)
    got = gemv.run(ctx, w_next, lazy, tokens, torch.float32, "out2", False, None).tensor
    gemm.check_errors()
    r = now[rows.long()]
    x = r / torch.sqrt((r * r).mean(-1, keepdim=True) + eps) * norm.tensors["weight"].double()
    # The input is rounded to bfloat16 once (before the norm's factor here, after it in the unfused
    # kernel: the same relative error 2^-9 / sqrt(3) per element of size ~1), so an output, a sum of
    # `hidden` products with weights of size 0.1, is off by sigma = 2^-9 / sqrt(3) * sqrt(hidden) * 0.1;
    # the bound is 8 sigma.
    sigma = 2.0 ** -9 / math.sqrt(3.0) * math.sqrt(hidden) * 0.1
    _close(got, x @ w_next.double().t(), 0.0, 8 * sigma)
    # without the request nothing is left
    gemv.run(ctx, w_down, act, tokens, torch.float32, "out", False, K.AddTo(residual))
    assert ctx.prenormed is None

