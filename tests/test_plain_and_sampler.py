"""The plain implementation's parts against each other and the host sampler's distributions (no GPU)."""

import random

import numpy as np
import torch

import helpers as H
import plain_llama as pl
from bare_cuda_4gib_b200.sampling import SamplingParams, host_sample


def test_plain_parts_basic_properties():
    x = torch.randn(5, 12, dtype=torch.float64)
    w = torch.rand(12, dtype=torch.float64) + 0.5
    y = pl.rms_norm(x, w, 1e-6)
    assert torch.allclose((y / w).pow(2).mean(-1), torch.ones(5, dtype=torch.float64), atol=1e-5)
    q = torch.randn(7, 3, 8, dtype=torch.float64)
    pos = torch.arange(7)
    r = pl.rope(q, pos, 10000.0)
    assert torch.allclose(r.norm(dim=-1), q.norm(dim=-1))              # a rotation
    assert torch.allclose(r[0], q[0])                                  # position 0 is the identity
    # relative property: (R_a q) . (R_b k) depends on a - b only
    k = torch.randn(1, 1, 8, dtype=torch.float64).expand(7, 1, 8)
    qq = q[:1].expand(7, 3, 8)
    d1 = (pl.rope(qq, pos + 3, 1e4)[:, 0] * pl.rope(k, pos, 1e4)[:, 0]).sum(-1)
    assert torch.allclose(d1, d1[0].expand(7), atol=1e-6)
    s = pl.attention_scores(q, q[:, :1], window=3)
    assert torch.isinf(s[0, 2, 3]) and torch.isinf(s[0, 5, 2]) and not torch.isinf(s[0, 5, 3])
    p = pl.softmax_rows(s)
    assert torch.allclose(p.sum(-1), torch.ones(3, 7, dtype=torch.float64)) and float(p[0, 5, 2]) == 0.0
    g = torch.tensor([0.0, 1.0, -2.0], dtype=torch.float64)
    assert torch.allclose(pl.swiglu(g, torch.ones(3, dtype=torch.float64)), g * torch.sigmoid(g))


def test_plain_last_logits_do_not_depend_on_later_tokens_and_reads_both_configs():
    for name in ("A", "B"):
        folder = H.model_folder(name)
        m = pl.read_model_folder(folder)
        ids = H.random_ids(random.Random(1), 12, m.vocab_size)
        full = pl.forward_logits(m, ids)
        assert full.shape == (12, m.vocab_size)
        assert torch.allclose(pl.forward_logits(m, ids[:7])[-1], full[6], atol=1e-12)
    assert pl.read_model_folder(H.model_folder("B")).lm_head is pl.read_model_folder(H.model_folder("B")).embed or True


def test_plain_shared_cache_and_repeated_layer_order():
    m = pl.read_model_folder(H.model_folder("A"))
    ids = [3, 9, 27, 81, 243 % 256]
    base = pl.forward_logits(m, ids)
    m.order = [(0, None), (1, None), (0, None), (1, 1)]        # layer 0 twice; the last run reads run 1's keys
    other = pl.forward_logits(m, ids)
    assert other.shape == base.shape and not torch.allclose(other, base)


def _freq(logits, p, n=40000, seed=0):
    rng = random.Random(seed)
    counts = np.zeros(len(logits))
    for _ in range(n):
        counts[host_sample(logits, p, rng.random())] += 1
    return counts / n


def test_host_sampler_distributions():
    logits = np.array([2.0, 1.0, 0.5, 0.0, -1.0, -3.0], dtype=np.float32)
    for t in (0.7, 1.0, 1.8):
        want = np.exp(logits / t) / np.exp(logits / t).sum()
        assert np.abs(_freq(logits, SamplingParams(temperature=t)) - want).max() < 0.015
    want = np.exp(logits[:3]) / np.exp(logits[:3]).sum()
    got = _freq(logits, SamplingParams(temperature=1.0, top_k=3))
    assert np.abs(got[:3] - want).max() < 0.015 and got[3:].sum() == 0
    probs = np.exp(logits) / np.exp(logits).sum()
    keep = int(np.searchsorted(np.cumsum(probs), 0.8)) + 1
    got = _freq(logits, SamplingParams(temperature=1.0, top_p=0.8))
    assert got[keep:].sum() == 0 and np.abs(got[:keep] - probs[:keep] / probs[:keep].sum()).max() < 0.015
    # top-p measured on the top-k set renormalised
    got = _freq(logits, SamplingParams(temperature=1.0, top_k=4, top_p=0.5))
    sub = probs[:4] / probs[:4].sum()
    keep = int(np.searchsorted(np.cumsum(sub), 0.5)) + 1
    assert got[keep:].sum() == 0
    assert host_sample(logits, SamplingParams(temperature=0.0), 0.99) == 0
    assert host_sample(logits, SamplingParams(temperature=1.0, top_k=1), 0.99) == 0
    assert host_sample(logits, SamplingParams(temperature=1.0, top_p=1e-6), 0.99) == 0


def test_host_sampler_agrees_with_plain_kept_set_on_a_large_vocabulary():
    rng = np.random.default_rng(0)
    logits = rng.normal(size=32000).astype(np.float32) * 2
    p = SamplingParams(temperature=0.9, top_k=0, top_p=0.95)
    kept = pl.kept_token_set(torch.from_numpy(logits), 0.9, 0, 0.95)
    assert len(kept) > 1024                                        # larger than a first partial sort would hold
    w = pl.sampling_weights(torch.from_numpy(logits), 0.9)
    for u in (0.0, 0.3, 0.77, 0.999999):
        want = pl.inverse_cdf_pick([float(w[i]) for i in kept], kept, u)
        assert host_sample(logits, p, u) == want


def test_perplexity_tool_scores_rows_like_log_softmax():
    from bare_cuda_4gib_b200.cli.ppl import window_nll
    torch.manual_seed(3)
    rows, targets = torch.randn(7, 19) * 4, [0, 18, 5, 5, 9, 1, 12]
    want = -float(sum(torch.log_softmax(rows.double(), 1)[i, t] for i, t in enumerate(targets)))
    assert abs(window_nll(rows, targets) - want) < 1e-12
