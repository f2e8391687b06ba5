"""bin/trace_run as a user runs it: a subprocess fed JSON lines, logits files compared with the
plain implementation; the same trace in float32 and bfloat16, with pages used again."""

import json
import pathlib
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_subprocess(dtype, tmp_path):
    name = "B"
    folder = H.model_folder(name)
    vocab = H.TINY[name][0]["vocab_size"]
    rng = random.Random(31)
    requests = {f"q{i}": H.random_ids(rng, n, vocab) for i, n in enumerate([70, 5, 130, 33, 64, 97])}
    steps = H.trace_mixed(requests, random.Random(2), live=4, budget_tokens=320, page=64)
    steps.append({"step": len(steps), "entries": [], "end": []})            # a step that brings nothing
    peak = H.peak_tokens(steps, 64)
    assert peak <= 320
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                           "--out", str(out), "--max-tokens", str(peak)],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", text=True, capture_output=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    fed = {r: 0 for r in requests}
    got = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        path = out / f"{s['step']}.f32"
        if not wanted:
            assert not path.exists()
            continue
        data = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
        row = 0
        for e in s["entries"]:
            for w in e["want"]:
                got[(e["id"], fed[e["id"]] + w)] = torch.from_numpy(data[row].copy())
                row += 1
            fed[e["id"]] += len(e["tokens"])
    H.check_against_plain(folder, requests, got, dtype)
