"""`llm-bench`: latency and throughput of whole requests through the engine's entry point.

    bin/llm-bench --model DIR (--prompt 1,15043,3186 | --prompt-len 512) [--tokens 32] [--runs 20]
                  [--warmup 2] [--batch N] [--kernels]

The options have the names, defaults and meanings of cuongvng/bare-cuda-4gib's tool
(bench/src/bench_main.cc:63-78,259-301): `--prompt-len N` makes a synthetic prompt (BOS, then
100 + (i * 7919) mod (vocab - 100), bench_main.cc:96-103); `--batch N` decodes N copies of the
prompt together; at least two tokens so that the time per output token has a sample.  The table
is the reference's too (bench_main.cc:371-390): TTFT, TPOT (all gaps, each sequence's first and
last), end-to-end latency, tokens a second per sequence in decode and end to end, and for a
batch the whole batch's rates; mean, nearest-rank p50 / p90 / p99, min, max.  `--kernels` adds a
breakdown of one request by kernel: launches, device time and its share (that request runs
without CUDA graphs and with an event pair around every launch, so its own wall time says
nothing).  Added here: `--random NAME` (write random weights of that preset into --model
first), `--dtype`, `--page-tokens`.  What it reports is the engine as a user meets it; the
fractions of roofline come from `bench.py` and `llm-kernel-bench`.
"""

from __future__ import annotations

import argparse
import math
import sys
import time


def synthetic_prompt(length: int, vocab: int):
    return [1] + [100 + (i * 7919) % (vocab - 100) for i in range(1, length)]


def percentile(samples, p):
    """Nearest rank: the smallest sample with at least p% of the samples at or below it."""
    ordered = sorted(samples)
    rank = math.ceil(p / 100.0 * len(ordered))
    return ordered[max(rank, 1) - 1]


def print_row(name, unit, samples):
    mean = sum(samples) / len(samples)
    print(f"  {name:<15s} {unit:<5s} {mean:10.2f} {percentile(samples, 50):10.2f} {percentile(samples, 90):10.2f} "
          f"{percentile(samples, 99):10.2f} {min(samples):10.2f} {max(samples):10.2f}")


def run_once(engine, prompt, tokens, batch):
    """One request (batch 0) or `batch` copies decoded together; per sequence the arrival time of every token."""
    import torch
    n = max(batch, 1)
    stamps = [[] for _ in range(n)]
    torch.cuda.synchronize()
    start = time.perf_counter()
    engine.generate_batch([prompt] * n, tokens, on_token=lambda seq, index, token: stamps[seq].append(time.perf_counter()))
    return start, stamps


def kernel_report(engine_factory, prompt, tokens, batch):
    """Device time of one request by kernel: every launcher call between two CUDA events."""
    import torch
    from ..kernels import attention, gemm, gemv
    from ..kernels import lib as K

    records = {}

    def timed(module, name, label):
        inner = getattr(module, name)

        def wrapper(*args, **kwargs):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = inner(*args, **kwargs)
            b.record()
            records.setdefault(label, []).append((a, b))
            return out

        setattr(module, name, wrapper)
        return inner

    saved = []
    for module, name, label in [(K, "embed_gather", "embedding"), (K, "add_rmsnorm", "add + rmsnorm"),
                                (K, "rope_cache_write", "rotation + cache"), (K, "swiglu", "swiglu"),
                                (K, "argmax_rows", "argmax"), (K, "sample_rows", "sampling"),
                                (K, "matmul_plain", "matmul (plain)"), (K, "attention_plain", "attention (plain)"),
                                (gemm, "run", "matmul (tcgen05)"), (gemv, "run", "few-token product"),
                                (attention, "run", "attention")]:
        saved.append((module, name, timed(module, name, label)))
    try:
        engine = engine_factory(False)
        torch.cuda.synchronize()
        wall = time.perf_counter()
        engine.generate_batch([prompt] * max(batch, 1), tokens)
        torch.cuda.synchronize()
        wall = (time.perf_counter() - wall) * 1e3
    finally:
        for module, name, inner in saved:
            setattr(module, name, inner)
    rows = [(label, len(pairs), sum(a.elapsed_time(b) for a, b in pairs)) for label, pairs in records.items()]
    total = sum(ms for _, _, ms in rows)
    print(f"\nper-kernel breakdown of one profiled request ({wall:.0f} ms wall with an event pair around every "
          f"launch, {total:.1f} ms on device)\n")
    print(f"  {'kernel':<20s} {'calls':>7s} {'ms':>9s} {'%':>6s}")
    for label, calls, ms in sorted(rows, key=lambda r: -r[2]):
        print(f"  {label:<20s} {calls:7d} {ms:9.2f} {100.0 * ms / total:6.1f}")
    print("\n  'matmul (tcgen05)' on few rows includes the kernels that add its partial results")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="llm-bench", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="model folder (config.json + model.safetensors)")
    ap.add_argument("--prompt", default="", help="comma-separated int32 token ids (offline-tokenized)")
    ap.add_argument("--prompt-len", type=int, default=0, help="use a synthetic prompt of N ids instead")
    ap.add_argument("--tokens", type=int, default=32, help="tokens to generate per request (default 32)")
    ap.add_argument("--runs", type=int, default=20, help="measured requests (default 20)")
    ap.add_argument("--warmup", type=int, default=2, help="unmeasured requests first (default 2)")
    ap.add_argument("--batch", type=int, default=0, help="decode N copies of the prompt together")
    ap.add_argument("--kernels", action="store_true", help="add a per-kernel breakdown of one profiled request")
    ap.add_argument("--random", default=None, help="write random weights of this preset into --model first")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--page-tokens", type=int, default=64)
    args = ap.parse_args(argv)
    if (not args.prompt) == (args.prompt_len <= 0) or args.tokens < 2 or args.runs < 1 or args.warmup < 0 or args.batch < 0:
        ap.print_usage(sys.stderr)
        print("exactly one of --prompt and --prompt-len; at least two tokens, one run", file=sys.stderr)
        return 1

    import torch
    from ..engine.engine import LLMEngine
    from .infer import parse_ids

    if args.random:
        from ..models.presets import preset_config
        from ..weights.random_init import write_random_model
        write_random_model(args.model, preset_config(args.random), 0)
    prompt = parse_ids(args.prompt) if args.prompt else None
    prompt_tokens = len(prompt) if prompt else args.prompt_len
    if prompt_tokens <= 0:
        print("[llm] empty prompt", file=sys.stderr)
        return 1
    free_before = torch.cuda.mem_get_info()[0]

    def make_engine(graphs=True):
        return LLMEngine(args.model, max_tokens=prompt_tokens + args.tokens, max_seqs=max(args.batch, 1),
                         dtype=args.dtype, page_tokens=args.page_tokens, use_cuda_graphs=graphs)

    load_start = time.perf_counter()
    engine = make_engine()
    torch.cuda.synchronize()
    load_ms = (time.perf_counter() - load_start) * 1e3
    if prompt is None:
        prompt = synthetic_prompt(args.prompt_len, engine.config.vocab_size)
    mib = 1024.0 * 1024.0
    print(f"model      {args.model}")
    print(f"request    prompt {prompt_tokens} tokens, generate {args.tokens} tokens"
          + (f", {args.batch} sequences decoded together" if args.batch else "")
          + f" | {args.warmup} warmup + {args.runs} measured runs")
    print(f"load       {load_ms:.0f} ms (file read, upload and kernel libraries, excluded below)")
    print(f"vram       {(free_before - torch.cuda.mem_get_info()[0]) / mib:.1f} MiB measured | "
          f"{engine.model.weight_bytes() / mib:.1f} weights + {sum(g.bytes for g in engine.cache.groups) / mib:.1f} kv cache accounted")
    print(engine.summary() + "\n")

    for _ in range(args.warmup):
        run_once(engine, prompt, args.tokens, args.batch)
    ttft, e2e, tps_decode, tps_e2e, tpot_all, tpot_first, tpot_last, batch_decode, batch_e2e = ([] for _ in range(9))
    for _ in range(args.runs):
        start, stamps = run_once(engine, prompt, args.tokens, args.batch)
        for s in stamps:
            first, last = (s[0] - start) * 1e3, (s[-1] - start) * 1e3
            gaps = [(b - a) * 1e3 for a, b in zip(s, s[1:])]
            ttft.append(first)
            e2e.append(last)
            tps_decode.append((args.tokens - 1) / ((last - first) / 1e3))
            tps_e2e.append(args.tokens / (last / 1e3))
            tpot_all.extend(gaps)
            tpot_first.append(gaps[0])
            tpot_last.append(gaps[-1])
        if args.batch:
            last_first, last = max(s[0] for s in stamps), max(s[-1] for s in stamps)
            batch_decode.append(args.batch * (args.tokens - 1) / (last - last_first))
            batch_e2e.append(args.batch * args.tokens / (last - start))
    print(f"  {'metric':<15s} {'unit':<5s} {'mean':>10s} {'p50':>10s} {'p90':>10s} {'p99':>10s} {'min':>10s} {'max':>10s}")
    print_row("TTFT", "ms", ttft)
    print_row("TPOT (all)", "ms", tpot_all)
    print_row("TPOT (1st)", "ms", tpot_first)
    print_row("TPOT (last)", "ms", tpot_last)
    print_row("E2E latency", "ms", e2e)
    print_row("TPS (decode)", "tok/s", tps_decode)
    print_row("TPS (e2e)", "tok/s", tps_e2e)
    if args.batch:
        print_row("TPS batch (dec)", "tok/s", batch_decode)
        print_row("TPS batch (e2e)", "tok/s", batch_e2e)
        print("\n  rows above the batch rows are per sequence; batch rows are whole-batch rates")
    print("\n  tokens reach the caller one step late while the scheduler runs a step ahead; the gaps between them are the steps'")
    if args.kernels:
        kernel_report(make_engine, prompt, args.tokens, args.batch)
    if args.runs < 100:
        print(f"\n  note: p99 over {args.runs} runs is the max sample; use --runs 100+ for a real tail")
    return 0


if __name__ == "__main__":
    sys.exit(main())
