"""Shared test tools: the two tiny configurations, model folders with random weights, trace
builders for the ways of cutting requests into steps, an in-process replay driver over the
engine's own step function, and the comparison with the plain implementation."""

from __future__ import annotations

import functools
import pathlib
import random
import tempfile
from typing import Dict, List, Sequence, Tuple

import torch

import plain_llama as pl

# Two tiny Llama configurations that differ in every size and option.
TINY_A = dict(architectures=["LlamaForCausalLM"], vocab_size=256, hidden_size=64, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=176,
              max_position_embeddings=128, rope_theta=10000.0, rms_norm_eps=1e-5,
              tie_word_embeddings=False)
TINY_B = dict(architectures=["LlamaForCausalLM"], vocab_size=320, hidden_size=96, num_hidden_layers=3,
              num_attention_heads=3, num_key_value_heads=1, head_dim=32, intermediate_size=256,
              max_position_embeddings=256, rope_theta=500000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=True)
TINY = {"A": (TINY_A, 16), "B": (TINY_B, 32)}   # configuration, cache page in tokens

# Tolerances, fixed before the first run.  Per logits row: max |got - want| / max |want|.
# float32: the engine's only difference from the float64 plain implementation is float32 rounding.
# bfloat16: activations are rounded to 8 significant bits at ~10 places per layer.
TOLERANCE = {"float32": 1e-5, "bfloat16": 3e-2}

_tmp_root = None


def tmp_root() -> pathlib.Path:
    global _tmp_root
    if _tmp_root is None:
        _tmp_root = tempfile.TemporaryDirectory(prefix="bare_cuda_b200_tests_")
    return pathlib.Path(_tmp_root.name)


@functools.lru_cache(maxsize=None)
def model_folder(name: str, seed: int = 7, stored: str = "bfloat16") -> pathlib.Path:
    """A model folder with random weights for tiny configuration `name`, made once per session."""
    import bare_cuda_4gib_b200.models  # noqa: F401
    from bare_cuda_4gib_b200.config import LlamaConfig
    from bare_cuda_4gib_b200.weights import write_random_model

    cfg = LlamaConfig.from_dict(TINY[name][0])
    folder = tmp_root() / f"tiny{name}-{seed}-{stored}"
    write_random_model(folder, cfg, seed, getattr(torch, stored))
    return folder


@functools.lru_cache(maxsize=None)
def plain_model(folder: pathlib.Path) -> pl.PlainModel:
    return pl.read_model_folder(folder)


_plain_cache: Dict[Tuple, torch.Tensor] = {}


def plain_logits(folder: pathlib.Path, ids: Sequence[int]) -> torch.Tensor:
    key = (str(folder), tuple(ids))
    if key not in _plain_cache:
        _plain_cache[key] = pl.forward_logits(plain_model(folder), list(ids))
    return _plain_cache[key]


def random_ids(rng: random.Random, n: int, vocab: int) -> List[int]:
    return [rng.randrange(vocab) for _ in range(n)]


def row_error(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).abs().max() / want.abs().max())


# ----------------------------------------------------------------------------- traces


def trace_whole(requests: Dict[str, List[int]]) -> List[dict]:
    """Each request alone and whole: one step, every place wanted."""
    return [{"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]}
            for i, (rid, ids) in enumerate(requests.items())]


def trace_decode_tail(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of a request in one step, the last `tail` tokens one by one."""
    steps, n = [], 0
    for rid, ids in requests.items():
        head = max(1, len(ids) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": ids[:head], "want": [head - 1]}], "end": []})
        n += 1
        for p in range(head, len(ids)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [ids[p]], "want": [0]}],
                          "end": [rid] if p == len(ids) - 1 else []})
            n += 1
        if head == len(ids):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests: Dict[str, List[int]], rng: random.Random) -> List[dict]:
    """Portions of changing size, down to two tokens, every place wanted."""
    sizes = [7, 2, 16, 3, 2, 5, 33, 2, 11, 64, 4]
    steps, n = [], 0
    for rid, ids in requests.items():
        p, k = 0, rng.randrange(len(sizes))
        while p < len(ids):
            size = min(sizes[k % len(sizes)], len(ids) - p)
            k += 1
            steps.append({"step": n, "entries": [{"id": rid, "tokens": ids[p: p + size], "want": list(range(size))}],
                          "end": [rid] if p + size == len(ids) else []})
            p += size
            n += 1
    return steps


def trace_mixed(requests: Dict[str, List[int]], rng: random.Random, live: int = 4, prompt_part: float = 0.6,
                budget_tokens: int = None, page: int = 64) -> List[dict]:
    """Up to `live` requests at a time: prompt portions of some beside single tokens of others.
    A request's first `prompt_part` goes in portions, the rest one token a step; requests may sit
    a step out.  New requests start as soon as one ends, so pages are used again; with
    `budget_tokens`, a request starts only while the live requests' page-rounded final lengths fit."""
    waiting = list(requests.items())
    active = []   # [rid, ids, fed, prompt_len]
    steps, n = [], 0
    rounded = lambda k: -(-k // page) * page
    while waiting or active:
        while waiting and len(active) < live:
            if budget_tokens is not None:
                held = sum(rounded(len(a[1])) for a in active)
                if held + rounded(len(waiting[0][1])) > budget_tokens:
                    break
            rid, ids = waiting.pop(0)
            active.append([rid, ids, 0, max(1, int(len(ids) * prompt_part))])
        entries, end = [], []
        for a in active:
            rid, ids, fed, plen = a
            if len(active) > 1 and rng.random() < 0.2:
                continue  # sits this step out
            if fed < plen:
                size = min(rng.choice([2, 3, 5, 8, 13, 21]), plen - fed)
            else:
                size = 1
            entries.append({"id": rid, "tokens": ids[fed: fed + size], "want": list(range(size))})
            a[2] += size
            if a[2] == len(ids):
                end.append(rid)
        active = [a for a in active if a[2] < len(a[1])]
        if entries:
            steps.append({"step": n, "entries": entries, "end": end})
            n += 1
    return steps


def peak_tokens(steps: List[dict], page: int) -> int:
    """Most tokens live requests hold at any time, each rounded up to a page."""
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-v // page) * page for v in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


# ----------------------------------------------------------------------------- replay


class Replayer:
    """Runs trace steps through the engine's model, cache manager and step function in-process
    (the same objects bin/trace_run drives) and collects logits by (request, position)."""

    def __init__(self, folder, dtype: str, page_tokens: int, max_tokens: int, max_live: int = 8,
                 shuffle_seed=None, **runner_options):
        from bare_cuda_4gib_b200.cache.manager import CacheManager
        from bare_cuda_4gib_b200.engine.model import load_model
        from bare_cuda_4gib_b200.engine.step import StepRunner

        capacity = -(-max_tokens // page_tokens) * page_tokens
        self.model, self.config = load_model(folder, dtype, "cuda")
        self.cache = CacheManager(self.model.cache_demands(), page_tokens=page_tokens, max_seqs=max_live,
                                  max_tokens=capacity, num_pages=capacity // page_tokens,
                                  dtype=self.model.dtype, device="cuda")
        if shuffle_seed is not None:
            for g in self.cache.groups:
                g.pool.shuffle_free_list(shuffle_seed)
        self.runner = StepRunner(self.model, self.cache, max_step_tokens=capacity, max_batch_seqs=max_live,
                                 **runner_options)
        self.slots, self.fed = {}, {}

    def run(self, steps: List[dict]) -> Dict[Tuple[str, int], torch.Tensor]:
        from bare_cuda_4gib_b200.engine.step import StepEntry

        out = {}
        for s in steps:
            entries = []
            for e in s["entries"]:
                if e["id"] not in self.slots:
                    self.slots[e["id"]] = self.cache.acquire_slot()
                    self.fed[e["id"]] = 0
                entries.append(StepEntry(self.slots[e["id"]], e["tokens"], e["want"]))
            logits = self.runner.step(entries)
            self.cache.check_consistency()
            row = 0
            for e in s["entries"]:
                for w in e["want"]:
                    out[(e["id"], self.fed[e["id"]] + w)] = logits[row].float().cpu()
                    row += 1
                self.fed[e["id"]] += len(e["tokens"])
            for rid in s["end"]:
                self.cache.release_slot(self.slots.pop(rid))
                self.fed.pop(rid)
        return out


def check_against_plain(folder, requests: Dict[str, List[int]], got: Dict[Tuple[str, int], torch.Tensor],
                        dtype: str, expect_all: bool = True) -> float:
    worst = 0.0
    for rid, ids in requests.items():
        want = plain_logits(folder, ids)
        places = [p for (r, p) in got if r == rid]
        if expect_all:
            assert sorted(places) == list(range(len(ids))), f"request {rid}: places {sorted(places)}"
        for p in places:
            err = row_error(got[(rid, p)], want[p])
            assert err <= TOLERANCE[dtype], (
                f"request {rid} position {p} of {len(ids)}: error {err:.3e} > {TOLERANCE[dtype]:.0e}")
            worst = max(worst, err)
    return worst
