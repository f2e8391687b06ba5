"""Writes tests/golden/refmodel_tiny.npz: a tiny random model of the reference's own torch
model (`RefModel`, tools/references/reference_forward.py:285-391 of cuongvng/bare-cuda-4gib),
its whole-prompt logits and its cacheless greedy ids.

Usage:  python tests/golden/make_golden.py <path to a checkout of cuongvng/bare-cuda-4gib>

`RefModel` runs on the CPU with torch and numpy only.  Two models are written, shaped like the
two tiny test configurations (different head counts and groups, sizes that are no power of two,
layers, vocabulary, eps and rope base).  tests/test_plain_vs_golden.py feeds the same weights to
tests/plain_llama.py and compares; that anchors the plain implementation's formulas on the
reference's code, and everything else in the suite on the plain implementation.
"""

import pathlib
import sys

import numpy as np
import torch


def main() -> None:
    if len(sys.argv) != 2:
        print(__doc__)
        sys.exit(2)
    root = pathlib.Path(sys.argv[1])
    sys.path.insert(0, str(root / "tools" / "references"))
    sys.path.insert(0, str(root / "tools" / "convert"))
    import binformat
    import reference_forward as rf

    shapes = {
        "a": dict(vocab_size=256, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2,
                  head_dim=16, intermediate_size=176, max_seq_len=128, rope_theta=10000.0,
                  rms_norm_eps=1e-5),
        "b": dict(vocab_size=320, hidden_size=96, num_layers=3, num_heads=3, num_kv_heads=1,
                  head_dim=32, intermediate_size=256, max_seq_len=256, rope_theta=500000.0,
                  rms_norm_eps=1e-6),
    }
    out = {}
    torch.manual_seed(rf.SEED)
    for tag, shape in shapes.items():
        cfg = binformat.ModelConfig(**shape)
        model = rf.RefModel(cfg)
        prompt = torch.randint(0, cfg.vocab_size, (23 if tag == "a" else 41,))
        logits = model.forward(prompt)
        greedy = model.greedy_decode(prompt, 24)
        for key, value in shape.items():
            out[f"{tag}.config.{key}"] = np.asarray(value)
        out[f"{tag}.prompt"] = prompt.numpy().astype(np.int32)
        out[f"{tag}.logits"] = logits.numpy().astype(np.float32)
        out[f"{tag}.greedy"] = greedy.numpy().astype(np.int32)
        # weights are FP16-rounded FP32 values: store them as float16 without loss
        out[f"{tag}.tok_embeddings"] = model.tok_embeddings.numpy().astype(np.float16)
        out[f"{tag}.output_norm"] = model.output_norm.numpy().astype(np.float16)
        out[f"{tag}.lm_head"] = model.lm_head.numpy().astype(np.float16)
        for i, layer in enumerate(model.layers):
            for name, t in layer.items():
                out[f"{tag}.layers.{i}.{name}"] = t.numpy().astype(np.float16)
    target = pathlib.Path(__file__).resolve().parent / "refmodel_tiny.npz"
    np.savez_compressed(target, **out)
    print(f"wrote {target} ({target.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
