"""`llm-batch-check`: batched decode against one-at-a-time decode.

    bin/llm-batch-check --model DIR --ids FILE [--tokens 64] [--batch 4] [--tol 0.01]

The check and its options are those of cuongvng/bare-cuda-4gib's tool
(bench/src/batch_check_main.cc:26-40,86-149): eight prompts are cut from an offline-tokenized
text (a flat file of little-endian int32 ids) at spacings of 1,000 ids, with 5, 17, 64, 120, 300,
8, 200 and 37 text ids after a BOS id (1): mixed lengths and more prompts than `--batch` slots,
so queueing and retiring run too.  Each prompt is decoded greedily alone, then all together
with `--batch` sequences decoding at once.  Alone and batched steps run different kernels that
sum in different orders, so a near-tie between the two best logits may break the other way: a
divergence is scored from one fresh pass over the shared prefix (a third, neutral path) and
only a gap between the two candidates' logits above `--tol` fails.  Exit status 1 on failure.
Added here: `--dtype`, `--page-tokens`, `--random NAME` (write random weights of that preset
into `--model` first) and `--spacing` (the reference's 1,000; smaller for short id files).
"""

from __future__ import annotations

import argparse
import sys

BOS_ID = 1                                              # batch_check_main.cc:25
PROMPT_LENGTHS = (5, 17, 64, 120, 300, 8, 200, 37)      # text ids, BOS added (batch_check_main.cc:26)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="llm-batch-check", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="model folder (config.json + model.safetensors)")
    ap.add_argument("--ids", required=True, help="flat little-endian int32 token ids")
    ap.add_argument("--tokens", type=int, default=64, help="tokens to generate per prompt (default 64)")
    ap.add_argument("--batch", type=int, default=4, help="sequences decoded at once (default 4)")
    ap.add_argument("--tol", type=float, default=0.01,
                    help="largest logit gap a divergence may have and still pass (default 0.01)")
    ap.add_argument("--spacing", type=int, default=1000, help="ids between the starts of two prompts' slices")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--page-tokens", type=int, default=64)
    ap.add_argument("--random", default=None, help="write random weights of this preset into --model first")
    args = ap.parse_args(argv)
    if args.tokens <= 0 or args.batch <= 0 or args.spacing <= 0:
        ap.print_usage(sys.stderr)
        return 1

    from .ppl import read_ids
    text = read_ids(args.ids)
    prompts = []
    for p, length in enumerate(PROMPT_LENGTHS):
        start = p * args.spacing
        if start + length > len(text):
            print(f"[llm] {args.ids} has {len(text)} ids, too few for prompt {p}", file=sys.stderr)
            return 1
        prompts.append([BOS_ID] + text[start: start + length])
    longest = max(len(p) for p in prompts)

    from ..engine.engine import LLMEngine
    from ..errors import EngineError
    if args.random:
        from ..models.presets import preset_config
        from ..weights.random_init import write_random_model
        write_random_model(args.model, preset_config(args.random), 0)
    try:
        engine = LLMEngine(args.model, max_tokens=longest + args.tokens, max_seqs=args.batch, dtype=args.dtype,
                           page_tokens=args.page_tokens)
    except EngineError as e:
        print(f"[llm] {e}", file=sys.stderr)
        return 1
    print(f"model      {args.model}")
    print(f"check      {len(prompts)} prompts of {len(prompts[0])}-{longest} tokens, {args.tokens} new tokens each, "
          f"{args.batch} decoding at once")
    print(f"kv pool    {engine.kv_pages} pages | max batch {engine.max_seqs} at {engine.max_tokens} tokens per sequence\n")

    alone = [engine.generate(prompt, args.tokens) for prompt in prompts]
    together = engine.generate_batch(prompts, args.tokens)

    exact = near_ties = failures = 0
    for p, prompt in enumerate(prompts):
        step = next((i for i, (a, b) in enumerate(zip(alone[p], together[p])) if a != b), None)
        if step is None and len(alone[p]) == len(together[p]):
            exact += 1
            print(f"prompt {p}  {len(prompt):3d} tokens  match, {len(alone[p])} ids identical")
            continue
        if step is None:     # one run is a prefix of the other: cannot happen without stop ids
            failures += 1
            print(f"prompt {p}  {len(prompt):3d} tokens  DIVERGES: {len(alone[p])} ids alone, {len(together[p])} batched")
            continue
        # score both candidates from one fresh pass over the shared prefix
        row = engine.score(prompt + alone[p][:step])[-1]
        one, other = alone[p][step], together[p][step]
        gap = abs(float(row[one]) - float(row[other]))
        tie = gap <= args.tol
        near_ties += tie
        failures += not tie
        print(f"prompt {p}  {len(prompt):3d} tokens  {'near-tie' if tie else 'DIVERGES'} at step {step}: "
              f"alone {one}, batched {other}, logit gap {gap:.5f}")

    print(f"\n{exact} match, {near_ties} split on a near-tie (gap <= {args.tol:.3g}), {failures} diverge")
    if failures:
        print("FAIL: batched decode disagrees with decoding alone beyond rounding")
        return 1
    print("PASS: batched decode agrees with decoding alone")
    return 0


if __name__ == "__main__":
    sys.exit(main())
