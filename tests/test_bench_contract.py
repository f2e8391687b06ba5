"""What `bench.py` promises without a GPU: more than one GPU is refused with one line and exit code 2
(the reference arm says `unavailable` and exits with 0), and the reference arm reads the table that the reference's `llm-bench` prints
(cuongvng/bare-cuda-4gib bench/src/bench_main.cc:371-390: name, unit, mean, p50, p90, p99, min, max)."""

import json
import pathlib
import subprocess
import sys

ROOT = pathlib.Path(__file__).resolve().parents[1]


def _bench(*args):
    run = subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=300)
    lines = [l for l in run.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    return run.returncode, json.loads(lines[0])


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    code, record = _bench("--gpus", "2")
    assert code == 2
    assert record["n_gpus"] == 2 and "one GPU" in record["error"]


def test_the_reference_arm_on_more_than_one_gpu_is_unavailable():
    code, record = _bench("--gpus", "2", "--impl", "reference")
    assert code == 0
    assert record["impl"] == "reference" and "one GPU" in record["unavailable"]


def test_reference_arm_reads_the_reference_tools_table():
    sys.path.insert(0, str(ROOT))
    from baseline import reference_arm

    text = """
  model: /tmp/m.llmbin  prompt_len 2027  tokens 21  batch 8
  metric          unit        mean        p50        p90        p99        min        max
  TTFT            ms        452.10     452.00     453.90     454.20     450.80     454.20
  TPOT (all)      ms         42.41      42.39      42.50      42.61      42.30      42.61
  TPS batch (dec) tok/s     188.70     188.73     188.79     188.79     188.66     188.79
  some other line
"""
    table = reference_arm.parse_table(text)
    assert set(table) == {"TTFT", "TPOT (all)", "TPS batch (dec)"}
    assert table["TPS batch (dec)"] == {"mean": 188.70, "p50": 188.73, "p90": 188.79, "p99": 188.79, "min": 188.66,
                                        "max": 188.79}
    assert table["TTFT"]["p50"] == 452.0
