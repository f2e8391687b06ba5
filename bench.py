#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens a second at a batch and context, prefill
tokens a second at 2,048 tokens, each beside its roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of the TinyLlama-1.1B shape with random weights (seeded
uniform-random token ids stand in for text), a batch of 8 and a context of 2,048 positions.  A
"step" is one decode step: every live request gets one token.  One JSON line is printed:

* `value`: decoded tokens a second, timed on the device with CUDA events around K steps of the
  engine's step function plus the sampling kernels (token ids pre-chosen, nothing read back).
* `e2e`: the same through the Python entry point (scheduler, host token lists in and out): each
  step uploads its metadata from pinned memory and reads the sampled ids back.
* `prefill`: one request of 2,048 tokens in one step, logits for its last place; `frac` = the
  step's FLOPs / time / the bf16 peak.
* `roofline`: bytes the decode step has to read (every weight once, the cache of the live
  requests) / its time, against the measured copy bandwidth.
* `points`: decode at batch 1 and 64.

The peaks come from MEASURED_PEAKS.json beside this file when present, else from the fallback
measurement (6.65 TB/s, 1.59 PFLOP/s).  The weights (2.2 GB) and the cache exceed the 126 MB L2,
so every step's inputs are larger than L2 and no flush is needed between timed iterations.
With --gpus above 1 it prints one line that says so and exits with 2: the engine runs on one GPU.
"""

from __future__ import annotations

import argparse
import json
import pathlib
import random
import statistics
import subprocess
import sys
import tempfile
import threading

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
PUBLISHED_B1_FP16_TOK_S = 77.3   # the reference's README, RTX 3050 Laptop, real weights, batch 1


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    hbm, tflops, source = FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            hbm = float(d.get("hbm_gbs", hbm))
            tflops = float(d.get("bf16_tflops", tflops))
            source = "measured"
        except (ValueError, OSError):
            pass
    return hbm, tflops, source


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.samples:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons)}


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--preset", default="tinyllama")
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the preset has (0 = all)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--no-graphs", action="store_true")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "cuongvng/bare-cuda-4gib is a CMake/CUDA C++ project without setup.py or pyproject.toml: "
                          "pip cannot install it offline, and it builds for sm_86 against its own .llmbin weights"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": f"this engine runs on one GPU; --gpus {args.gpus} is not supported", "n_gpus": args.gpus}))
        return 2
    warmup = max(3, args.warmup)

    import torch

    from bare_cuda_4gib_b200.engine.engine import LLMEngine
    from bare_cuda_4gib_b200.engine.scheduler import Request
    from bare_cuda_4gib_b200.engine.step import StepEntry
    from bare_cuda_4gib_b200.kernels import gemm, lib as K
    from bare_cuda_4gib_b200.models.presets import PRESETS, preset_config
    from bare_cuda_4gib_b200.weights.random_init import write_random_model

    full_layers = PRESETS[args.preset]["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg = preset_config(args.preset, num_hidden_layers=layers)
    hbm_gbs, bf16_tflops, peak_source = peaks()
    tmp = tempfile.TemporaryDirectory(prefix="bench_model_")
    write_random_model(tmp.name, cfg, seed=0, dtype=torch.bfloat16, device="cuda")
    context = args.context
    max_batch = max(args.batch, 1 if args.no_points else 64)
    engine = LLMEngine(tmp.name, max_tokens=context, max_seqs=max_batch, dtype="bfloat16", page_tokens=64,
                       max_step_tokens=2048 + max_batch, use_cuda_graphs=not args.no_graphs)
    runner, cache, vocab = engine.runner, engine.cache, cfg.vocab_size
    rng = random.Random(0)
    d, nkv, nh, H, I = cfg.head_dim, cfg.num_key_value_heads, cfg.num_attention_heads, cfg.hidden_size, cfg.intermediate_size
    layer_params = (nh + 2 * nkv) * d * H + nh * d * H + 3 * H * I
    weight_bytes = 2 * (layers * (layer_params + 2 * H) + H + vocab * H)     # every weight once, lm_head included
    kv_bytes_per_token = layers * 2 * nkv * d * 2

    def fill(batch, cached):
        """Puts `cached` random tokens of `batch` requests into the cache through the step function."""
        slots = [cache.acquire_slot() for _ in range(batch)]
        chunk = 2048
        for slot in slots:
            fed = 0
            while fed < cached:
                n = min(chunk, cached - fed)
                runner.step([StepEntry(slot, [rng.randrange(vocab) for _ in range(n)], [])])
                fed += n
        return slots


    def decode_steps(slots, n):
        for _ in range(n):
            runner.step([StepEntry(s, [rng.randrange(vocab)], [0]) for s in slots])   # ends with the rows' argmax

    def measure_decode(batch, steps, warm):
        cached = context - steps - warm - 1
        slots = fill(batch, cached)
        decode_steps(slots, warm)
        torch.cuda.synchronize()
        launches0 = K.LAUNCHES[0]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        decode_steps(slots, steps)
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        launches = K.LAUNCHES[0] - launches0
        for s in slots:
            cache.release_slot(s)
        gemm.check_errors()
        mean_ctx = cached + warm + (steps + 1) / 2
        bytes_per_step = weight_bytes + kv_bytes_per_token * mean_ctx * batch
        return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launches,
                "gbs": bytes_per_step / (ms / steps / 1e3) / 1e9}

    def measure_prefill(tokens, reps=5):
        best = None
        for i in range(reps + 2):
            slot = cache.acquire_slot()
            ids = [rng.randrange(vocab) for _ in range(tokens)]
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            runner.step([StepEntry(slot, ids, [tokens - 1])])
            end.record()
            torch.cuda.synchronize()
            cache.release_slot(slot)
            if i >= 2:
                ms = start.elapsed_time(end)
                best = ms if best is None else min(best, ms)
        flops = 2.0 * tokens * layers * layer_params + 2.0 * vocab * H \
            + layers * 4.0 * nh * d * tokens * (tokens + 1) / 2
        return {"value": tokens / (best / 1e3), "tokens": tokens, "ms": best,
                "frac": flops / (best / 1e3) / (bf16_tflops * 1e12), "tflops": flops / (best / 1e3) / 1e12}

    def measure_e2e(batch, steps, warm):
        """The scheduler's loop: host token lists in, sampled ids out, every step."""
        # prompts are prefilled one a step, so the first request is `batch` tokens ahead of the last:
        # leave room for all of them to decode through the timed steps before any reaches the context's end
        cached = context - steps - warm - batch - 2
        sched = engine.scheduler
        for i in range(batch):
            sched.submit(Request(id=i, prompt=[rng.randrange(vocab) for _ in range(cached)],
                                 max_new_tokens=steps + warm + 64))
        while any(l.generated == 0 for l in list(sched.running) + list(sched.waiting)):
            sched.step()
        for _ in range(warm - 1):
            sched.step()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        produced = 0
        for _ in range(steps):
            produced += sum(1 for e in sched.step() if e.token >= 0)
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        for rid in range(batch):
            sched.cancel(rid)
        h2d = runner.metadata_bytes(batch, batch)
        return {"value": produced / (ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4 * batch}

    clocks = ClockSampler()
    clocks.start()
    main_run = measure_decode(args.batch, args.steps, warmup)
    clock_summary = clocks.summary()
    clocks.stop()
    e2e = measure_e2e(args.batch, args.steps, warmup)
    prefill = measure_prefill(min(2048, context))
    points = {}
    if not args.no_points:
        for b in (1, 64):
            r = measure_decode(b, args.steps, warmup)
            points[f"decode_b{b}"] = r["tok_s"]
            points[f"decode_b{b}_hbm_frac"] = r["gbs"] / hbm_gbs
    line = {
        "metric": "decode tokens/s (TinyLlama-1.1B shape, bf16, batch 8, context 2048)",
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: seeded random weights, uniform random token ids",
        "impl": "ours",
        "config": {"model": f"{args.preset} shape (LlamaForCausalLM)", "layers": layers,
                   "layers_of_config": full_layers, "hidden": H, "heads": nh, "kv_heads": nkv, "head_dim": d,
                   "intermediate": I, "vocab": vocab, "global_batch": args.batch, "seq_len": context,
                   "page_tokens": 64, "parallelism": "single GPU", "l2": "inputs larger than L2 (weights 2.2 GB)",
                   "peaks": peak_source, "cuda_graphs": not args.no_graphs},
        "e2e": e2e,
        "gpu_launches": main_run["launches"],
        "clocks": clock_summary,
        "prefill": {k: prefill[k] for k in ("value", "tokens", "ms", "frac")},
        "roofline": {"bound": "hbm", "achieved": main_run["gbs"], "peak": hbm_gbs, "unit": "GB/s",
                     "frac": main_run["gbs"] / hbm_gbs},
        "points": points,
        "vs_published_b1_fp16_rtx3050": (points.get("decode_b1") / PUBLISHED_B1_FP16_TOK_S) if points else None,
    }
    print(json.dumps(line))
    tmp.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
