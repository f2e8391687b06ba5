"""The engine at the layer sizes of real Llama checkpoints (two layers, a small odd vocabulary,
random weights) against the plain implementation: one long prompt portion that takes the
many-token kernels (tokens on the tensor-core rows, the tensor-memory attention), then single
decoded tokens, then a second request in small portions beside them."""

import functools
import random

import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

SHAPES = {
    "tinyllama": dict(num_hidden_layers=2, vocab_size=2003),
    "llama2-7b": dict(num_hidden_layers=2, vocab_size=1999),
    "llama3-8b": dict(num_hidden_layers=2, vocab_size=2001),
}


@functools.lru_cache(maxsize=None)
def _folder(preset):
    from bare_cuda_4gib_b200.models.presets import preset_config
    from bare_cuda_4gib_b200.weights import write_random_model

    cfg = preset_config(preset, **SHAPES[preset])
    folder = H.tmp_root() / f"shape-{preset}"
    write_random_model(folder, cfg, 21, torch.bfloat16, "cuda")
    return folder, cfg


def _trace(ids_a, ids_b, head):
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ids_a[:head], "want": [0, 1, head // 2, head - 1]}], "end": []}]
    p, q, n = head, 0, 1
    portions = [5, 2, 64, 3, 130]
    while p < len(ids_a) or q < len(ids_b):
        entries = []
        if p < len(ids_a):
            entries.append({"id": "a", "tokens": [ids_a[p]], "want": [0]})
            p += 1
        if q < len(ids_b):
            size = min(portions[(n - 1) % len(portions)], len(ids_b) - q)
            entries.append({"id": "b", "tokens": ids_b[q: q + size], "want": [size - 1]})
            q += size
        steps.append({"step": n, "entries": entries, "end": []})
        n += 1
    steps[-1]["end"] = ["a", "b"]
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("preset", list(SHAPES))
def test_real_layer_sizes(preset, dtype):
    folder, cfg = _folder(preset)
    rng = random.Random(13)
    ids_a = H.random_ids(rng, 300 + 12, cfg.vocab_size)
    ids_b = H.random_ids(rng, 204, cfg.vocab_size)
    steps = _trace(ids_a, ids_b, 300)
    got = H.Replayer(folder, dtype, 64, H.peak_tokens(steps, 64), shuffle_seed=2).run(steps)
    worst = H.check_against_plain(folder, {"a": ids_a, "b": ids_b}, got, dtype, expect_all=False)
    print(f"{preset} {dtype}: worst row error {worst:.3e}")
