"""The command line tools end to end on a tiny random model: `llm-infer` against the plain
implementation's greedy decode, `llm-bench` and `llm-kernel-bench` for their tables, `llm-ppl` against
the plain implementation's perplexity, `llm-batch-check` and `llm-devinfo`."""

import os
import pathlib
import subprocess
import sys

import pytest

import helpers as H
import plain_llama as pl

pytestmark = pytest.mark.gpu

ROOT = pathlib.Path(__file__).resolve().parents[1]


def _run(tool, *args):
    env = dict(os.environ, PYTHONDONTWRITEBYTECODE="1")
    done = subprocess.run([sys.executable, str(ROOT / "bin" / tool), *map(str, args)], capture_output=True, text=True,
                          env=env, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    return done.stdout


def test_llm_infer_prints_the_plain_greedy_tokens():
    folder = H.model_folder("A")
    prompt = [5, 17, 3, 200, 9, 41]
    out = _run("llm-infer", "--model", folder, "--prompt", ",".join(map(str, prompt)), "--tokens", 12, "--dtype", "float32")
    lines = dict(line.split(":", 1) for line in out.splitlines() if line.startswith(("prompt:", "generated:")))
    assert [int(t) for t in lines["prompt"].split()] == prompt
    assert [int(t) for t in lines["generated"].split()] == pl.greedy_decode(H.plain_model(folder), prompt, 12)
    assert out.splitlines()[0].startswith("[llm] 2 layers, hidden 64, vocab 256")


def test_llm_infer_refuses_a_prompt_without_ids():
    done = subprocess.run([sys.executable, str(ROOT / "bin" / "llm-infer"), "--model", str(H.model_folder("A")),
                           "--prompt", ",,"], capture_output=True, text=True, timeout=600)
    assert done.returncode == 1 and "no token ids" in done.stderr


def test_llm_bench_tables():
    folder = H.model_folder("B")
    out = _run("llm-bench", "--model", folder, "--prompt-len", 9, "--tokens", 5, "--runs", 2, "--warmup", 1,
               "--batch", 3, "--kernels")
    for row in ("TTFT", "TPOT (all)", "TPOT (1st)", "TPOT (last)", "E2E latency", "TPS (decode)", "TPS (e2e)",
                "TPS batch (dec)", "TPS batch (e2e)", "per-kernel breakdown"):
        assert row in out, row
    assert "prompt 9 tokens, generate 5 tokens, 3 sequences decoded together | 1 warmup + 2 measured runs" in out
    # exactly one prompt source, at least two tokens
    bad = subprocess.run([sys.executable, str(ROOT / "bin" / "llm-bench"), "--model", str(folder), "--tokens", "1",
                          "--prompt-len", "4"], capture_output=True, text=True, timeout=600)
    assert bad.returncode == 1


def test_llm_kernel_bench_reports_a_roofline_fraction():
    import json
    out = _run("llm-kernel-bench", "gemv", "--tokens", 4, "--out", 256, "--in", 96, "--form", "swiglu", "--norm",
               "--iters", 3, "--warmup", 1)
    line = json.loads([l for l in out.splitlines() if l.startswith("{")][-1])
    assert line["us"] > 0 and 0 < line["hbm_frac"] < 1.5


def _ids_file(name, n, vocab, seed):
    import random

    import numpy as np
    path = H.tmp_root() / name
    np.asarray(H.random_ids(random.Random(seed), n, vocab), dtype="<i4").tofile(path)
    return path


def test_llm_ppl_matches_the_plain_implementation():
    import math

    import torch
    folder = H.model_folder("A")
    ctx, windows, vocab = 33, 3, 256
    ids_path = _ids_file("ppl.ids", 120, vocab, 5)
    out = _run("llm-ppl", "--model", folder, "--ids", ids_path, "--ctx", ctx, "--windows", windows, "--dtype", "float32")
    assert f"120 ids, {windows} windows of {ctx} (BOS + {ctx - 1}), {windows * (ctx - 1)} predictions" in out
    import numpy as np
    text = np.fromfile(ids_path, dtype="<i4").tolist()
    nll = 0.0
    for w in range(windows):
        window = [1] + text[w * (ctx - 1): (w + 1) * (ctx - 1)]
        logp = torch.log_softmax(H.plain_logits(folder, window).double(), dim=1)
        nll -= float(sum(logp[t, window[t + 1]] for t in range(ctx - 1)))
    want = math.exp(nll / (windows * (ctx - 1)))
    got = float([l for l in out.splitlines() if l.startswith("perplexity")][0].split()[1])
    assert abs(got - want) <= 2e-4 * want, (got, want)
    assert f"tokens scored {windows * (ctx - 1)}" in out


def test_llm_batch_check_passes_and_reports_every_prompt():
    import torch

    from bare_cuda_4gib_b200.models.presets import preset_config
    from bare_cuda_4gib_b200.weights import write_random_model
    folder = H.tmp_root() / "batch-check-model"
    cfg = preset_config("tinyB", max_position_embeddings=512)
    write_random_model(folder, cfg, 3, torch.bfloat16)
    ids_path = _ids_file("check.ids", 600, cfg.vocab_size, 9)
    for dtype in ("float32", "bfloat16"):
        out = _run("llm-batch-check", "--model", folder, "--ids", ids_path, "--tokens", 9, "--batch", 3,
                   "--spacing", 40, "--dtype", dtype)
        assert "8 prompts of 6-301 tokens, 9 new tokens each, 3 decoding at once" in out
        assert sum(line.startswith("prompt ") for line in out.splitlines()) == 8
        assert "PASS: batched decode agrees with decoding alone" in out and "0 diverge" in out
    short = subprocess.run([sys.executable, str(ROOT / "bin" / "llm-batch-check"), "--model", str(folder), "--ids",
                            str(ids_path), "--tokens", "4"], capture_output=True, text=True, timeout=600)
    assert short.returncode == 1 and "too few for prompt" in short.stderr


def test_llm_devinfo_lines():
    log = H.tmp_root() / "devinfo.log"
    kv = _run("llm-devinfo", "--kv", "--out", log)
    assert kv.startswith('name="') and " sms=" in kv and " free_post_mib=" in kv
    assert log.read_text().strip().endswith(kv.strip())
    long_form = _run("llm-devinfo")
    assert "=> allocatable budget" in long_form and "SMs" in long_form
