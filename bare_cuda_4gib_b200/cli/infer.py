"""`llm-infer`: token ids in, generated token ids out.

    bin/llm-infer --model DIR --prompt 1,15043,3186 [--tokens 16] [--max-seq 0]

The options `--model`, `--prompt`, `--tokens` and `--max-seq` have the names and meanings of
cuongvng/bare-cuda-4gib's tool (bench/src/main.cc:18-27,45-94): ids are pre-tokenized (there is
no tokenizer in the engine), `--tokens` defaults to 16, `--max-seq` 0 means prompt + tokens.
It prints a model summary line, `prompt:` and `generated:`.  Added here: `--dtype`, the sampling
options of the Python entry point, cache sizing, and `--random NAME` which writes a model
folder with random weights (seed `--weights-seed`) into `--model` first.
"""

from __future__ import annotations

import argparse
import sys


def parse_ids(text: str):
    return [int(piece) for piece in text.split(",") if piece.strip()]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="llm-infer", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="model folder (config.json + model.safetensors)")
    ap.add_argument("--prompt", required=True, help="comma-separated int32 token ids (offline-tokenized)")
    ap.add_argument("--tokens", type=int, default=16, help="number of tokens to generate (default 16)")
    ap.add_argument("--max-seq", type=int, default=0, help="cache size in tokens; must cover prompt + generated")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--temperature", type=float, default=0.0, help="0 is greedy")
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--seed", type=int, default=-1, help="sampling seed; -1 draws one")
    ap.add_argument("--page-tokens", type=int, default=64)
    ap.add_argument("--kv-pages", type=int, default=0, help="0 fits the pool to the request")
    ap.add_argument("--random", default=None, help="write random weights of this preset into --model first")
    ap.add_argument("--weights-seed", type=int, default=0)
    args = ap.parse_args(argv)

    prompt = parse_ids(args.prompt)
    if not prompt:
        print("[llm] no token ids parsed from --prompt", file=sys.stderr)
        return 1
    from ..engine.engine import LLMEngine
    from ..sampling.params import SamplingParams

    if args.random:
        from ..models.presets import preset_config
        from ..weights.random_init import write_random_model
        write_random_model(args.model, preset_config(args.random), args.weights_seed)
    max_seq = args.max_seq if args.max_seq > 0 else len(prompt) + args.tokens
    engine = LLMEngine(args.model, max_tokens=max_seq, max_seqs=1, kv_pages=args.kv_pages, dtype=args.dtype,
                       page_tokens=args.page_tokens)
    print(engine.summary())
    sampling = SamplingParams(args.temperature, args.top_p, args.top_k, args.seed)
    generated = engine.generate(prompt, args.tokens, sampling=sampling)
    print("prompt:    " + " ".join(str(t) for t in prompt))
    print("generated: " + " ".join(str(t) for t in generated))
    return 0


if __name__ == "__main__":
    sys.exit(main())
