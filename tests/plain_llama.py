"""Plain, slow Llama decoder for the tests: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite.  It shares no code with the package under test:
it reads model folders with the `safetensors` library (the package has its own reader), keeps
every tensor as a float64 torch tensor on the CPU and recomputes the whole sequence for every
answer.  Each function restates one formula of cuongvng/bare-cuda-4gib and cites where that
project computes it (paths are relative to that project's root).

Precision.  Weights are used exactly as stored (a bfloat16 value widens exactly).  Sums run in
float64, so this is the truth that the 32-bit engine is measured against.  Two things follow
the reference in 32-bit on purpose, because they are part of the definition rather than of
the rounding: the rotation angle `float(pos) * inv_freq` (a product of two float32 numbers,
rounded to float32: engine/kernels/rope.cu:44-47) and the inverse frequencies themselves
(tools/references/reference_forward.py:91).

`round_to` (None or torch.bfloat16) makes the function round activations at the places where
an engine that stores activations in that type would: it is only used to explain bfloat16
differences, never to loosen a comparison.
"""

from __future__ import annotations

import json
import math
import pathlib
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- model folder


@dataclass
class PlainLayer:
    input_norm: torch.Tensor
    wq: torch.Tensor
    wk: torch.Tensor
    wv: torch.Tensor
    wo: torch.Tensor
    post_norm: torch.Tensor
    w_gate: torch.Tensor
    w_up: torch.Tensor
    w_down: torch.Tensor
    window: Optional[int] = None  # keys older than pos - window + 1 are masked; None = all keys


@dataclass
class PlainModel:
    vocab_size: int
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate_size: int
    rope_theta: float
    rms_norm_eps: float
    embed: torch.Tensor
    final_norm: torch.Tensor
    lm_head: torch.Tensor
    layers: List[PlainLayer] = field(default_factory=list)
    # order in which layers run: (layer index, index of the earlier run whose keys and values
    # this run reads instead of its own, or None)
    order: Optional[List[tuple]] = None


def read_model_folder(folder) -> PlainModel:
    """Reads config.json + model.safetensors with the HF tensor names.

    The reference gets these names renamed offline (tools/convert/convert_weights.py:68-83:
    model.embed_tokens.weight, model.norm.weight, lm_head.weight,
    model.layers.{i}.input_layernorm / self_attn.{q,k,v,o}_proj / post_attention_layernorm /
    mlp.{gate,up,down}_proj) and its config numbers from the HF keys
    (tools/convert/convert_weights.py:35-46; head_dim = hidden_size // num_attention_heads at :41).
    """
    from safetensors import safe_open

    folder = pathlib.Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    tensors: Dict[str, torch.Tensor] = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            tensors[name] = f.get_tensor(name).to(F64)

    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    d = cfg.get("head_dim") or cfg["hidden_size"] // nh
    embed = tensors["model.embed_tokens.weight"]
    tied = cfg.get("tie_word_embeddings", False) or "lm_head.weight" not in tensors
    model = PlainModel(
        vocab_size=cfg["vocab_size"],
        hidden_size=cfg["hidden_size"],
        num_heads=nh,
        num_kv_heads=nkv,
        head_dim=d,
        intermediate_size=cfg["intermediate_size"],
        rope_theta=float(cfg.get("rope_theta", 10000.0)),
        rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-5)),
        embed=embed,
        final_norm=tensors["model.norm.weight"],
        lm_head=embed if tied else tensors["lm_head.weight"],
    )
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        model.layers.append(
            PlainLayer(
                input_norm=tensors[p + "input_layernorm.weight"],
                wq=tensors[p + "self_attn.q_proj.weight"],
                wk=tensors[p + "self_attn.k_proj.weight"],
                wv=tensors[p + "self_attn.v_proj.weight"],
                wo=tensors[p + "self_attn.o_proj.weight"],
                post_norm=tensors[p + "post_attention_layernorm.weight"],
                w_gate=tensors[p + "mlp.gate_proj.weight"],
                w_up=tensors[p + "mlp.up_proj.weight"],
                w_down=tensors[p + "mlp.down_proj.weight"],
            )
        )
    return model


# ----------------------------------------------------------------------------- parts


def _round(x: torch.Tensor, round_to) -> torch.Tensor:
    return x if round_to is None else x.to(round_to).to(F64)


def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """x[t, :] = E[ids[t], :]; no scale, no position term (engine/kernels/embedding_lookup.cu:22-30)."""
    return table[ids.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w: eps inside the root, on the mean; the weight multiplied
    last; no bias and no 1 + w (engine/kernels/rmsnorm.cu:26-40;
    tools/references/reference_forward.py:84-86)."""
    scale = torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return x * scale * weight


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """y = x W^T, W stored [out, in], no bias (engine/include/llm/kernels.h:48-57;
    engine/kernels/gemm_tiled.cuh:36-96)."""
    return x @ weight.t()


def rope_inverse_frequencies(head_dim: int, theta: float) -> torch.Tensor:
    """inv_freq[p] = 1 / theta^(2p / d) for p in [0, d/2), in float32
    (tools/references/reference_forward.py:91; engine/kernels/rope.cu:44)."""
    half = head_dim // 2
    return 1.0 / (theta ** (torch.arange(half, dtype=torch.float32) * 2.0 / head_dim))


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotary position encoding with the rotate_half pairing (p with p + d/2), in place of x
    [T, heads, d]: lo' = lo cos - hi sin, hi' = hi cos + lo sin; the angle is the float32
    product float(pos) * inv_freq (engine/kernels/rope.cu:44-53;
    tools/references/reference_forward.py:96-104)."""
    d = x.shape[-1]
    half = d // 2
    inv = rope_inverse_frequencies(d, theta)
    angles = (positions.to(torch.float32).unsqueeze(-1) * inv).to(F64)  # float32 product, widened
    cos = torch.cos(angles).unsqueeze(1)
    sin = torch.sin(angles).unsqueeze(1)
    lo, hi = x[..., :half], x[..., half:]
    return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], dim=-1)


def attention_scores(q: torch.Tensor, k: torch.Tensor, window: Optional[int] = None) -> torch.Tensor:
    """S[h, i, j] = (q[i, h] . k[j, h // g]) / sqrt(d), -inf for j > i (and, with a window, for
    j <= i - window); scale applied after the dot product
    (engine/kernels/attention_qk.cu:25,34-35,49-68; tools/references/reference_forward.py:118-120)."""
    t, nh, d = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    kv_index = torch.div(torch.arange(nh), group, rounding_mode="floor")
    scores = torch.einsum("ihd,jhd->hij", q, k[:, kv_index, :]) * (1.0 / math.sqrt(d))
    i = torch.arange(t).unsqueeze(1)
    j = torch.arange(t).unsqueeze(0)
    mask = j > i
    if window is not None:
        mask = mask | (j <= i - window)
    return scores.masked_fill(mask, float("-inf"))


def softmax_rows(scores: torch.Tensor) -> torch.Tensor:
    """Row softmax with the maximum subtracted; masked entries become exactly 0
    (engine/kernels/softmax.cu:28-42)."""
    return torch.softmax(scores, dim=-1)


def attention_values(probs: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """O[i, h, :] = sum_j P[h, i, j] v[j, h // g, :] (engine/kernels/attention_av.cu:24-44)."""
    nh = probs.shape[0]
    nkv = v.shape[1]
    kv_index = torch.div(torch.arange(nh), nh // nkv, rounding_mode="floor")
    return torch.einsum("hij,jhd->ihd", probs, v[:, kv_index, :])


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up with silu(g) = g / (1 + exp(-g)) (engine/kernels/swiglu.cu:22-23)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def attention_mixer(m: PlainModel, layer: PlainLayer, h: torch.Tensor, positions: torch.Tensor,
                    round_to=None, kv_from=None):
    """q, k, v projections, rotation of q and k, causal attention, output projection
    (engine/src/model.cpp:540-572).  Returns (projected output, (k, v) as cached)."""
    t = h.shape[0]
    q = _round(linear(h, layer.wq), round_to).view(t, m.num_heads, m.head_dim)
    q = _round(rope(q, positions, m.rope_theta), round_to)
    if kv_from is None:
        k = _round(linear(h, layer.wk), round_to).view(t, m.num_kv_heads, m.head_dim)
        v = _round(linear(h, layer.wv), round_to).view(t, m.num_kv_heads, m.head_dim)
        k = _round(rope(k, positions, m.rope_theta), round_to)
    else:
        k, v = kv_from
    probs = softmax_rows(attention_scores(q, k, layer.window))
    out = _round(attention_values(probs, v), round_to).reshape(t, m.num_heads * m.head_dim)
    return linear(out, layer.wo), (k, v)


def feed_forward(layer: PlainLayer, h: torch.Tensor, round_to=None) -> torch.Tensor:
    """down(silu(gate(h)) * up(h)), no biases (engine/src/model.cpp:589-598)."""
    act = _round(swiglu(linear(h, layer.w_gate), linear(h, layer.w_up)), round_to)
    return linear(act, layer.w_down)


def decoder_block(m: PlainModel, layer: PlainLayer, x: torch.Tensor, positions: torch.Tensor,
                  round_to=None, kv_from=None):
    """Pre-norm residual block: x += mixer(norm(x)); x += ffn(norm(x))
    (engine/src/model.cpp:526-604; tools/references/reference_forward.py:365-378)."""
    h = _round(rms_norm(x, layer.input_norm, m.rms_norm_eps), round_to)
    mixed, kv = attention_mixer(m, layer, h, positions, round_to, kv_from)
    x = x + mixed
    h = _round(rms_norm(x, layer.post_norm, m.rms_norm_eps), round_to)
    x = x + feed_forward(layer, h, round_to)
    return x, kv


def output_head(m: PlainModel, x: torch.Tensor, round_to=None) -> torch.Tensor:
    """logits = rms_norm(x, final_norm) lm_head^T (engine/src/model.cpp:608-615)."""
    return linear(_round(rms_norm(x, m.final_norm, m.rms_norm_eps), round_to), m.lm_head)


def forward_logits(m: PlainModel, ids: Sequence[int], round_to=None) -> torch.Tensor:
    """Whole-sequence forward without a cache; logits [T, vocab] in float64
    (tools/references/reference_forward.py:358-380)."""
    ids_t = torch.as_tensor(list(ids), dtype=torch.long)
    positions = torch.arange(ids_t.shape[0])
    x = embedding(m.embed, ids_t)
    order = m.order if m.order is not None else [(i, None) for i in range(len(m.layers))]
    kvs = []
    for layer_index, source in order:
        kv_from = None if source is None else kvs[source]
        x, kv = decoder_block(m, m.layers[layer_index], x, positions, round_to, kv_from)
        kvs.append(kv)
    return output_head(m, x, round_to)


def greedy_decode(m: PlainModel, prompt: Sequence[int], steps: int, round_to=None) -> List[int]:
    """Argmax decoding with no cache: every step re-runs the whole sequence; the lowest index
    wins a tie (tools/references/reference_forward.py:382-391; engine/kernels/logits_argmax.cu:36-64)."""
    ids = list(prompt)
    out = []
    for _ in range(steps):
        nxt = int(torch.argmax(forward_logits(m, ids, round_to)[-1]))
        out.append(nxt)
        ids.append(nxt)
    return out


# ----------------------------------------------------------------------------- sampling


def sampling_weights(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """Unnormalised softmax weights exp((l - max) / T) (engine/src/sampler.cpp:38-46)."""
    lg = logits.to(F64)
    return torch.exp((lg - lg.max()) / temperature)


def kept_token_set(logits: torch.Tensor, temperature: float, top_k: int, top_p: float) -> List[int]:
    """Token ids that survive top-k then top-p, likeliest first, lower id first on ties; top-p is
    measured on the top-k set renormalised: the smallest prefix whose mass reaches top_p
    (engine/src/sampler.cpp:48-93)."""
    w = sampling_weights(logits, temperature)
    vocab = w.shape[0]
    k = min(top_k, vocab) if top_k > 0 else vocab
    order = sorted(range(vocab), key=lambda i: (-float(w[i]), i))[:k]
    if top_p >= 1.0:
        return order
    total = sum(float(w[i]) for i in order)
    cum = 0.0
    for n, i in enumerate(order):
        cum += float(w[i])
        if cum >= top_p * total:
            return order[: n + 1]
    return order


def inverse_cdf_pick(weights: Sequence[float], ids: Sequence[int], u: float) -> int:
    """Walks the kept ids in order, subtracting weights from u * total; the first id that takes
    the target below zero is drawn, the last one if rounding leaves it short
    (engine/src/sampler.cpp:52-58,96-103)."""
    target = u * float(sum(weights))
    for w, i in zip(weights, ids):
        target -= float(w)
        if target < 0.0:
            return int(i)
    return int(ids[-1])
