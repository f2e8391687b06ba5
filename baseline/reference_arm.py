"""The reference arm of the benchmark: cuongvng/bare-cuda-4gib itself, unmodified, built with its
own CMake files for sm_100 and run through its own `llm-bench` program.

Nothing of this repository's engine is imported here.  The steps:

1. `ensure_built()` - `baseline/_ref/src` is a plain copy of the reference tree; it is configured
   with `cmake -G Ninja -DLLM_CUDA_ARCH=100 -DCMAKE_BUILD_TYPE=Release` into `baseline/_ref/build`
   and the target `llm-bench` is built (bench/CMakeLists.txt of the reference).
2. `write_model()` - a random-weight `.llmbin` of the wanted layer sizes, written by the
   reference's own `RefModel(binformat.ModelConfig(...)).write()`
   (tools/references/reference_forward.py:284-343, tools/convert/binformat.py:27-52), in a
   child process so that this module does not need torch.
3. `run_bench()` - `llm-bench --model F --prompt-len P --tokens T --batch B --runs R --warmup W`
   (bench/src/bench_main.cc:258-390); its table is parsed: the row `TPS batch (dec)` is decoded
   tokens a second of the whole batch, wall clock from the last sequence's first token to the last
   token, every token handed to a host callback; `TPS batch (e2e)` counts the prompt pass too.

Every failure is returned as one line of text (the last line the failing program printed), which
the caller prints as the arm's `unavailable` reason.
"""

from __future__ import annotations

import os
import pathlib
import re
import shutil
import subprocess
import sys
from typing import Dict, Optional, Tuple

HERE = pathlib.Path(__file__).resolve().parent
REF = HERE / "_ref"
SRC = REF / "src"
BUILD = REF / "build"
BENCH_BIN = BUILD / "bin" / "llm-bench"
UPSTREAM = pathlib.Path(os.environ.get("BARE_CUDA_REFERENCE_SOURCE", "/root/reference"))

_WRITER = r"""
import sys, pathlib
tools = pathlib.Path(sys.argv[1])
sys.path.insert(0, str(tools / "references"))
sys.path.insert(0, str(tools / "convert"))
import torch
import binformat
import reference_forward as rf
vals = [int(v) for v in sys.argv[3:11]] + [float(sys.argv[11]), float(sys.argv[12])]
torch.manual_seed(0)
config = binformat.ModelConfig(*vals)
rf.RefModel(config).write(sys.argv[2])
"""


class ReferenceUnavailable(RuntimeError):
    pass


def _last_line(text: str) -> str:
    lines = [l.strip() for l in text.splitlines() if l.strip()]
    return lines[-1][:300] if lines else "(no output)"


def _run(cmd, what: str, timeout: int, cwd=None) -> str:
    try:
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout, cwd=cwd)
    except FileNotFoundError as e:
        raise ReferenceUnavailable(f"{what}: {e}") from None
    except subprocess.TimeoutExpired:
        raise ReferenceUnavailable(f"{what}: no result after {timeout} s") from None
    if p.returncode != 0:
        raise ReferenceUnavailable(f"{what} failed (exit {p.returncode}): {_last_line(p.stdout)}")
    return p.stdout


def ensure_source() -> None:
    if (SRC / "CMakeLists.txt").exists():
        return
    if not (UPSTREAM / "CMakeLists.txt").exists():
        raise ReferenceUnavailable(f"no copy of the reference under {SRC} and none at {UPSTREAM}")
    REF.mkdir(parents=True, exist_ok=True)
    shutil.copytree(UPSTREAM, SRC)


def ensure_built(verbose: bool = True) -> pathlib.Path:
    """Builds the reference's llm-bench if it is not there yet; returns its path."""
    if BENCH_BIN.exists():
        return BENCH_BIN
    ensure_source()
    cmake = shutil.which("cmake")
    if cmake is None:
        raise ReferenceUnavailable("cmake not found: the reference cannot be built")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if verbose:
        print("[reference arm] configuring and building the reference for sm_100 ...", file=sys.stderr, flush=True)
    _run([cmake, "-S", str(SRC), "-B", str(BUILD), "-G", "Ninja", "-DLLM_CUDA_ARCH=100", "-DCMAKE_BUILD_TYPE=Release",
          f"-DCMAKE_CUDA_COMPILER={nvcc}"], "cmake configure of the reference", 600)
    _run([cmake, "--build", str(BUILD), "--target", "llm-bench"], "cmake build of the reference's llm-bench", 1800)
    if not BENCH_BIN.exists():
        raise ReferenceUnavailable("the reference built without an llm-bench binary")
    return BENCH_BIN


def write_model(path, *, vocab: int, hidden: int, layers: int, heads: int, kv_heads: int, head_dim: int,
                intermediate: int, max_seq_len: int, rope_theta: float, eps: float) -> None:
    """A random-weight .llmbin of these sizes, written by the reference's own RefModel."""
    ensure_source()
    args = [str(v) for v in (vocab, hidden, layers, heads, kv_heads, head_dim, intermediate, max_seq_len,
                             rope_theta, eps)]
    _run([sys.executable, "-c", _WRITER, str(SRC / "tools"), str(path), *args],
         "writing random weights with the reference's RefModel", 1800)


_ROW = re.compile(r"^\s*(TTFT|TPOT \(all\)|E2E latency|TPS \(decode\)|TPS \(e2e\)|TPS batch \(dec\)|TPS batch \(e2e\))"
                  r"\s+\S+\s+([-0-9.eE+]+)\s+([-0-9.eE+]+)\s+([-0-9.eE+]+)\s+([-0-9.eE+]+)\s+([-0-9.eE+]+)\s+([-0-9.eE+]+)")


def parse_table(text: str) -> Dict[str, Dict[str, float]]:
    """llm-bench's table rows -> {row name: {mean, p50, p90, p99, min, max}}."""
    out = {}
    for line in text.splitlines():
        m = _ROW.match(line)
        if m:
            keys = ("mean", "p50", "p90", "p99", "min", "max")
            out[m.group(1)] = {k: float(m.group(i + 2)) for i, k in enumerate(keys)}
    return out


def run_bench(model_path, *, prompt_len: int, tokens: int, batch: int, runs: int, warmup: int,
              timeout: int = 1500) -> Tuple[Dict[str, Dict[str, float]], str]:
    exe = ensure_built()
    text = _run([str(exe), "--model", str(model_path), "--prompt-len", str(prompt_len), "--tokens", str(tokens),
                 "--batch", str(batch), "--runs", str(runs), "--warmup", str(warmup)], "the reference's llm-bench", timeout)
    table = parse_table(text)
    if "TPS batch (dec)" not in table:
        raise ReferenceUnavailable(f"llm-bench printed no 'TPS batch (dec)' row: {_last_line(text)}")
    return table, text


if __name__ == "__main__":
    print(ensure_built())
