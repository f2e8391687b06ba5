"""The command line tools refuse what they cannot run with one line and exit status 1 (no GPU
needed: a folder without a model fails before, or instead of, any work on a device)."""

import pathlib
import subprocess
import sys

import numpy as np
import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("tool,extra", [("llm-ppl", ["--ctx", "33"]),
                                        ("llm-batch-check", ["--spacing", "40", "--tokens", "4"])])
def test_tools_report_a_folder_without_a_model(tmp_path, tool, extra):
    ids = tmp_path / "text.ids"
    np.arange(700, dtype="<i4").tofile(ids)
    done = subprocess.run([sys.executable, str(ROOT / "bin" / tool), "--model", str(tmp_path), "--ids", str(ids), *extra],
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 1
    assert done.stderr.strip().splitlines()[-1].startswith("[llm] ")


def test_ppl_refuses_a_text_shorter_than_one_window(tmp_path):
    ids = tmp_path / "short.ids"
    np.arange(10, dtype="<i4").tofile(ids)
    done = subprocess.run([sys.executable, str(ROOT / "bin" / "llm-ppl"), "--model", str(tmp_path), "--ids", str(ids)],
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 1 and "less than one window of 511" in done.stderr
