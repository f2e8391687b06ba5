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
* `points`: decode at batch 1 and 64, and - unless --no-shapes - decode at batch 8 and the
  2,048-token prefill at the Llama-2-7B and Llama-3-8B layer sizes with all their 32 layers
  (random weights generated straight on the device).

Every timed region is repeated (--repeats, default 5); the figure reported is the median and
`*_min` / `*_max` give the spread.  `--impl reference` runs cuongvng/bare-cuda-4gib itself, built
unmodified with its own CMake files for sm_100, through its own `llm-bench` program on a random
model of the same sizes (see baseline/reference_arm.py), and prints the same keys.

The peaks come from MEASURED_PEAKS.json beside this file when present, else from the fallback
measurement (6.65 TB/s, 1.59 PFLOP/s).  The weights (2.2 GB) and the cache exceed the 126 MB L2,
so every step's inputs are larger than L2 and no flush is needed between timed iterations.
Between putting the prompts into the cache (40 ms of tensor-core work at the power cap) and the
decode steps the device rests for 100 ms (`config.pause_after_prompts_ms`): right after that burst
the same decode steps ran 3 to 5 % slower for some tens of milliseconds, and the decode figures
are those of steady decoding.
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
import time

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


def reference_main(args) -> int:
    """The reference arm: nothing of this repository's engine is imported."""
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_arm as ref

    from_presets = {
        "tinyllama": dict(vocab=32000, hidden=2048, layers=22, heads=32, kv_heads=4, head_dim=64, intermediate=5632,
                          rope_theta=10000.0, eps=1e-5),
    }
    if args.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "the reference runs on one GPU"}))
        return 0
    if args.preset not in from_presets:
        print(json.dumps({"impl": "reference", "unavailable": f"the reference arm is set up for the tinyllama shape, not {args.preset}"}))
        return 0
    shape = dict(from_presets[args.preset])
    if args.layers:
        shape["layers"] = args.layers
    context, steps, batch = args.context, args.steps, args.batch
    prompt_len = context - steps - 1            # decode steps then run over the same contexts as the repo arm's
    try:
        ref.ensure_built()
        with tempfile.TemporaryDirectory(prefix="bench_reference_") as tmp:
            model = pathlib.Path(tmp) / "model.llmbin"
            ref.write_model(model, max_seq_len=context + 8, **shape)
            clocks = ClockSampler()
            clocks.start()
            table, _text = ref.run_bench(model, prompt_len=prompt_len, tokens=steps + 1, batch=batch,
                                         runs=args.repeats, warmup=1)
            clock_summary = clocks.summary()
            clocks.stop()
            single, _ = ref.run_bench(model, prompt_len=min(2048, context) - 1, tokens=2, batch=1, runs=3, warmup=1)
    except ref.ReferenceUnavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e)}))
        return 0
    dec, whole = table["TPS batch (dec)"], table["TPS batch (e2e)"]
    ttft_ms = single["TTFT"]["p50"]
    line = {
        "metric": f"decode tokens/s ({args.preset} shape, batch {batch}, context {context})",
        "value": dec["p50"], "value_min": dec["min"], "value_max": dec["max"], "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": 1, "repeats": args.repeats, "ms_per_step": batch / dec["p50"] * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16 weights, fp32 math", "data": "synthetic: the reference's own RefModel random weights, its synthetic prompt",
        "impl": "reference",
        "config": {"model": f"{args.preset} shape (.llmbin)", "layers": shape["layers"],
                   "layers_of_config": from_presets[args.preset]["layers"], "hidden": shape["hidden"],
                   "heads": shape["heads"], "kv_heads": shape["kv_heads"], "head_dim": shape["head_dim"],
                   "intermediate": shape["intermediate"], "vocab": shape["vocab"], "global_batch": batch,
                   "seq_len": context, "prompt_len": prompt_len, "page_tokens": 64, "parallelism": "single GPU",
                   "l2": "inputs larger than L2", "program": "llm-bench, built with -DLLM_CUDA_ARCH=100"},
        # the reference times with the host's clock around its public generate_batch call, every token handed
        # to a host callback: its decode figure is an end-to-end figure already
        "e2e": {"value": dec["p50"], "unit": "tokens/s", "how": "TPS batch (dec): wall clock, host callback per token"},
        "request_tok_s_with_prefill": whole["p50"],
        "clocks": clock_summary,
        "prefill": {"value": (min(2048, context) - 1) / (ttft_ms / 1e3), "tokens": min(2048, context) - 1, "ms": ttft_ms},
    }
    print(json.dumps(line))
    return 0


SETTLE_SECONDS = 0.1      # pause between putting the prompts into the cache and the decode steps (see Bench.settle)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--prefill-tokens", type=int, default=2048, help="tokens of the timed prefill step (the contract's figure is 2,048)")
    ap.add_argument("--preset", default="tinyllama")
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the preset has (0 = all)")
    ap.add_argument("--repeats", type=int, default=5, help="times every timed region is run (the median is reported)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--no-shapes", action="store_true", help="skip the Llama-2-7B / Llama-3-8B points")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--only", default="", choices=["", "prefill", "decode"],
                    help="profiling aid: run just the prefill step or just the decode steps and print their time")
    args = ap.parse_args()
    args.repeats = max(1, args.repeats)

    if args.impl == "reference":
        return reference_main(args)
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

    hbm_gbs, bf16_tflops, peak_source = peaks()
    context = args.context
    rng = random.Random(0)
    median = statistics.median

    class Bench:
        """One engine with seeded random weights (generated on the device) and its measurements."""

        def __init__(self, preset, layers, max_batch):
            self.full_layers = PRESETS[preset]["num_hidden_layers"]
            self.layers = layers or self.full_layers
            self.cfg = cfg = preset_config(preset, num_hidden_layers=self.layers)
            self.engine = LLMEngine(None, max_tokens=context, max_seqs=max_batch, dtype="bfloat16", page_tokens=64,
                                    max_step_tokens=2048 + max_batch, use_cuda_graphs=not args.no_graphs,
                                    random=(cfg, 0))
            self.runner, self.cache, self.vocab = self.engine.runner, self.engine.cache, cfg.vocab_size
            d, nkv, nh, H, I = (cfg.head_dim, cfg.num_key_value_heads, cfg.num_attention_heads, cfg.hidden_size,
                                cfg.intermediate_size)
            self.layer_params = (nh + 2 * nkv) * d * H + nh * d * H + 3 * H * I
            # every weight once, lm_head included (the embedding table is read by row only)
            self.weight_bytes = 2 * (self.layers * (self.layer_params + 2 * H) + H + self.vocab * H)
            self.kv_bytes_per_token = self.layers * 2 * nkv * d * 2

        def settle(self):
            """After the prompts are in the cache: lets the device finish and rest for a moment.  The prefill of
            the benchmark's prompts is 40 ms of tensor-core work at the power cap, and for some tens of
            milliseconds afterwards the same decode steps ran 3 to 5 % slower (0.83 against 0.79 ms; with a
            pause of 50 ms or of 500 ms alike 0.79): the decode figures are those of steady decoding."""
            torch.cuda.synchronize()
            time.sleep(SETTLE_SECONDS)

        def fill(self, batch, cached):
            """Puts `cached` random tokens of `batch` requests into the cache through the step function."""
            slots = [self.cache.acquire_slot() for _ in range(batch)]
            for slot in slots:
                fed = 0
                while fed < cached:
                    n = min(2048, cached - fed)
                    self.runner.step([StepEntry(slot, [rng.randrange(self.vocab) for _ in range(n)], [])])
                    fed += n
            self.settle()
            return slots

        def decode_steps(self, slots, n):
            for _ in range(n):     # ends with the rows' argmax
                self.runner.step([StepEntry(s, [rng.randrange(self.vocab)], [0]) for s in slots])

        def decode_once(self, batch, steps, warm):
            cached = context - steps - warm - 1
            slots = self.fill(batch, cached)
            self.decode_steps(slots, warm)
            torch.cuda.synchronize()
            launches0 = K.LAUNCHES[0]
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            self.decode_steps(slots, steps)
            end.record()
            torch.cuda.synchronize()
            ms = start.elapsed_time(end)
            launches = K.LAUNCHES[0] - launches0
            for s in slots:
                self.cache.release_slot(s)
            gemm.check_errors()
            mean_ctx = cached + warm + (steps + 1) / 2
            bytes_per_step = self.weight_bytes + self.kv_bytes_per_token * mean_ctx * batch
            return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launches,
                    "gbs": bytes_per_step / (ms / steps / 1e3) / 1e9}

        def decode(self, batch, steps, warm, repeats):
            runs = sorted((self.decode_once(batch, steps, warm) for _ in range(repeats)), key=lambda r: r["tok_s"])
            mid = dict(runs[(len(runs) - 1) // 2])          # the median run (the lower middle of an even count)
            mid["tok_s_min"], mid["tok_s_max"] = runs[0]["tok_s"], runs[-1]["tok_s"]
            return mid

        def prefill(self, tokens, repeats):
            times = []
            for i in range(repeats + 2):
                slot = self.cache.acquire_slot()
                ids = [rng.randrange(self.vocab) for _ in range(tokens)]
                torch.cuda.synchronize()
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                self.runner.step([StepEntry(slot, ids, [tokens - 1])])
                end.record()
                torch.cuda.synchronize()
                self.cache.release_slot(slot)
                if i >= 2:
                    times.append(start.elapsed_time(end))
            gemm.check_errors()
            cfg = self.cfg
            flops = 2.0 * tokens * self.layers * self.layer_params + 2.0 * self.vocab * cfg.hidden_size \
                + self.layers * 4.0 * cfg.num_attention_heads * cfg.head_dim * tokens * (tokens + 1) / 2
            ms = median(times)
            return {"value": tokens / (ms / 1e3), "tokens": tokens, "ms": ms, "ms_min": min(times), "ms_max": max(times),
                    "frac": flops / (ms / 1e3) / (bf16_tflops * 1e12)}

        def e2e_once(self, batch, steps, warm):
            """The scheduler's loop: host token lists in, sampled ids out, every step."""
            # prompts are prefilled one a step, so the first request is `batch` tokens ahead of the last:
            # leave room for all of them to decode through the timed steps before any reaches the context's end
            cached = context - steps - warm - batch - 2
            sched = self.engine.scheduler
            for i in range(batch):
                sched.submit(Request(id=i, prompt=[rng.randrange(self.vocab) for _ in range(cached)],
                                     max_new_tokens=steps + warm + 64))
            while any(l.generated == 0 for l in list(sched.running) + list(sched.waiting)):
                sched.step()
            self.settle()
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
            while not sched.idle:
                sched.step()
            return produced / (ms / 1e3)

        def e2e(self, batch, steps, warm, repeats):
            values = sorted(self.e2e_once(batch, steps, warm) for _ in range(repeats))
            return {"value": values[(len(values) - 1) // 2], "value_min": values[0], "value_max": values[-1],
                    "unit": "tokens/s", "h2d_bytes_per_step": self.runner.metadata_bytes(batch, batch),
                    "d2h_bytes_per_step": 4 * batch}

        def close(self):
            self.engine = self.runner = self.cache = None
            import gc
            gc.collect()
            torch.cuda.empty_cache()

    max_batch = max(args.batch, 1 if args.no_points else 64)
    bench = Bench(args.preset, args.layers, max_batch)
    cfg = bench.cfg
    if args.only:      # a short run for a profiler: one kind of step, nothing else
        if args.only == "prefill":
            r = bench.prefill(min(args.prefill_tokens, context), args.repeats)
        else:
            r = bench.decode(args.batch, args.steps, warmup, args.repeats)
        print(json.dumps({"only": args.only, "layers": bench.layers, "batch": args.batch, **r}))
        return 0
    clocks = ClockSampler()
    clocks.start()
    main_run = bench.decode(args.batch, args.steps, warmup, args.repeats)
    clock_summary = clocks.summary()
    clocks.stop()
    e2e = bench.e2e(args.batch, args.steps, warmup, args.repeats)
    prefill = bench.prefill(min(args.prefill_tokens, context), args.repeats)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            r = bench.decode(b, args.steps, warmup, args.repeats)
            points[f"decode_b{b}"] = r["tok_s"]
            points[f"decode_b{b}_min"], points[f"decode_b{b}_max"] = r["tok_s_min"], r["tok_s_max"]
            points[f"decode_b{b}_hbm_frac"] = r["gbs"] / hbm_gbs
    weights_gb = bench.weight_bytes / 1e9
    bench.close()
    if not args.no_shapes:
        for preset in ("llama2-7b", "llama3-8b"):
            key = preset.replace("-", "_")
            other = Bench(preset, 0, 8)
            r = other.decode(8, args.steps, warmup, max(3, args.repeats // 2))
            pf = other.prefill(min(2048, context), 3)
            points[f"{key}_decode_b8"] = r["tok_s"]
            points[f"{key}_decode_b8_hbm_frac"] = r["gbs"] / hbm_gbs
            points[f"{key}_prefill_tok_s"] = pf["value"]
            points[f"{key}_prefill_frac"] = pf["frac"]
            points[f"{key}_layers"], points[f"{key}_layers_of_config"] = other.layers, other.full_layers
            other.close()
    line = {
        "metric": f"decode tokens/s ({args.preset} shape, bf16, batch {args.batch}, context {context})",
        "value": main_run["tok_s"], "value_min": main_run["tok_s_min"], "value_max": main_run["tok_s_max"],
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup, "repeats": args.repeats,
        "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: seeded random weights, uniform random token ids",
        "impl": "ours",
        "config": {"model": f"{args.preset} shape (LlamaForCausalLM)", "layers": bench.layers,
                   "layers_of_config": bench.full_layers, "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size,
                   "vocab": cfg.vocab_size, "global_batch": args.batch, "seq_len": context,
                   "page_tokens": 64, "parallelism": "single GPU",
                   "l2": f"inputs larger than L2 (weights {weights_gb:.1f} GB read every step)",
                   "peaks": peak_source, "cuda_graphs": not args.no_graphs, "repeats": args.repeats,
                   "pause_after_prompts_ms": int(SETTLE_SECONDS * 1000)},
        "e2e": e2e,
        "gpu_launches": main_run["launches"],
        "clocks": clock_summary,
        "prefill": {k: prefill[k] for k in ("value", "tokens", "ms", "ms_min", "ms_max", "frac")},
        "roofline": {"bound": "hbm", "achieved": main_run["gbs"], "peak": hbm_gbs, "unit": "GB/s",
                     "frac": main_run["gbs"] / hbm_gbs},
        "points": points,
        "vs_published_b1_fp16_rtx3050": (points.get("decode_b1") / PUBLISHED_B1_FP16_TOK_S)
        if "decode_b1" in points and args.preset == "tinyllama" else None,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
