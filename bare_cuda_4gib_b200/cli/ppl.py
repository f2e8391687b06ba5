"""`llm-ppl`: perplexity of a model over an offline-tokenized text.

    bin/llm-ppl --model DIR --ids FILE [--ctx 512] [--windows 0]

Options and arithmetic are those of cuongvng/bare-cuda-4gib's tool (bench/src/ppl_main.cc:27-34,
84-127): `--ids` is a flat file of little-endian int32 token ids; it is cut into non-overlapping
windows of `--ctx` tokens, a BOS id (1) and then ctx - 1 text ids; each window is one fresh
request whose logits at every position score the id that follows, so a window yields ctx - 1
predictions; `--windows N` evaluates only the first N (0: all full windows).  The negative
log-likelihood is taken in double from the float32 logits (ppl_main.cc:53-58) and the
perplexity is exp(mean).  Added here: `--dtype`, `--page-tokens`, and `--random NAME`, which
first writes random weights of that preset into `--model` (the perplexity of random weights is
about the vocabulary size: a smoke check, not a quality figure).
"""

from __future__ import annotations

import argparse
import math
import sys
import time

BOS_ID = 1      # ppl_main.cc:24


def read_ids(path: str):
    import numpy as np
    return np.fromfile(path, dtype="<i4").tolist()


def window_nll(logits, targets) -> float:
    """Sum over the rows of -log softmax(row)[target], in double."""
    import torch
    rows = logits.double()
    top = rows.max(dim=1, keepdim=True).values
    log_norm = top.squeeze(1) + torch.log(torch.exp(rows - top).sum(dim=1))
    picked = rows[torch.arange(rows.shape[0]), torch.tensor(targets)]
    return float((log_norm - picked).sum())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="llm-ppl", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="model folder (config.json + model.safetensors)")
    ap.add_argument("--ids", required=True, help="flat little-endian int32 token ids")
    ap.add_argument("--ctx", type=int, default=512, help="window length in tokens, BOS included (default 512)")
    ap.add_argument("--windows", type=int, default=0, help="evaluate only the first N windows (default: all full windows)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--page-tokens", type=int, default=64)
    ap.add_argument("--random", default=None, help="write random weights of this preset into --model first")
    args = ap.parse_args(argv)
    if args.ctx < 2:
        ap.print_usage(sys.stderr)
        return 1

    text = read_ids(args.ids)
    stride = args.ctx - 1
    windows = len(text) // stride
    if args.windows > 0:
        windows = min(windows, args.windows)
    if windows == 0:
        print(f"[llm] {len(text)} ids is less than one window of {stride}", file=sys.stderr)
        return 1

    from ..engine.engine import LLMEngine
    from ..errors import EngineError
    if args.random:
        from ..models.presets import preset_config
        from ..weights.random_init import write_random_model
        write_random_model(args.model, preset_config(args.random), 0)
    try:
        engine = LLMEngine(args.model, max_tokens=args.ctx, max_seqs=1, dtype=args.dtype, page_tokens=args.page_tokens)
    except EngineError as e:
        print(f"[llm] {e}", file=sys.stderr)
        return 1
    vocab = engine.vocab_size
    bad = [t for t in text[: windows * stride] if not 0 <= t < vocab]
    if bad:
        print(f"[llm] token id {bad[0]} is outside the vocabulary of {vocab}", file=sys.stderr)
        return 1
    print(f"[llm] {len(text)} ids, {windows} windows of {args.ctx} (BOS + {stride}), {windows * stride} predictions")

    start = time.perf_counter()
    total_nll, scored = 0.0, 0
    for w in range(windows):
        window = [BOS_ID] + text[w * stride: (w + 1) * stride]
        logits = engine.score(window)
        # position t predicts window[t + 1]; the last position has nothing to score
        total_nll += window_nll(logits[:-1], window[1:])
        scored += stride
        if (w + 1) % 50 == 0 or w + 1 == windows:
            print(f"  window {w + 1:4d}/{windows}  running ppl {math.exp(total_nll / scored):.4f}", flush=True)
    seconds = time.perf_counter() - start
    mean_nll = total_nll / scored
    print(f"tokens scored {scored}\nmean nll      {mean_nll:.6f}\nperplexity    {math.exp(mean_nll):.4f}\n"
          f"time          {seconds:.1f} s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
