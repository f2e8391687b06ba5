"""Trace replay: feeds given token ids through a model step by step and writes logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

It samples nothing and owns no forward pass, cache or loader: it drives the engine's own model,
step function and cache manager, the ones that generation uses.  For a step in which something
is wanted it writes OUT/<step>.f32 (little-endian float32, [wanted, vocab], in the order of the
entries and of `want`), prints `done <step>` after every step, and exits 0 when its input ends.
The cache pool is made for `--max-tokens` positions (each live request's count rounded up to a
page), so pages are used again as requests end.
"""

from __future__ import annotations

import argparse
import json
import pathlib
import sys



def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the logits files are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (rounded up per request to a page)")
    ap.add_argument("--page-tokens", type=int, default=64, help="positions per cache page (default 64)")
    ap.add_argument("--max-live", type=int, default=8, help="request slots (default 8)")
    args = ap.parse_args(argv)

    import torch

    from ..cache.manager import CacheManager
    from ..engine.model import load_model
    from ..engine.step import StepEntry, StepRunner

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; the engine has no CPU path", file=sys.stderr)
        return 1
    out_dir = pathlib.Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    page = args.page_tokens
    capacity = -(-args.max_tokens // page) * page
    model, _config = load_model(args.model, args.dtype, "cuda")
    cache = CacheManager(model.cache_demands(), page_tokens=page, max_seqs=args.max_live,
                         max_tokens=capacity, num_pages=capacity // page, dtype=model.dtype, device="cuda")
    runner = StepRunner(model, cache, max_step_tokens=capacity, max_batch_seqs=args.max_live)
    slots = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for e in record.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = cache.acquire_slot()
            entries.append(StepEntry(slots[rid], e["tokens"], e.get("want", [])))
        if entries:
            logits = runner.step(entries)
            if logits is not None:
                data = logits.detach().to("cpu", torch.float32).contiguous().numpy()
                data.astype("<f4").tofile(out_dir / f"{step}.f32")
            else:
                torch.cuda.synchronize()
        for rid in record.get("end", []):
            if rid in slots:
                cache.release_slot(slots.pop(rid))
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
