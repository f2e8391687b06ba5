"""The command line tools end to end on a tiny random model: `llm-infer` against the plain
implementation's greedy decode, `llm-bench` and `llm-kernel-bench` for their tables."""

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
