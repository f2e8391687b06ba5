"""The plain implementation against the reference's own torch model (see golden/make_golden.py)."""

import pathlib

import numpy as np
import pytest
import torch

import plain_llama as pl

GOLDEN = pathlib.Path(__file__).resolve().parent / "golden" / "refmodel_tiny.npz"


def _model(data, tag) -> pl.PlainModel:
    cfg = {k.split(".")[-1]: data[k].item() for k in data.files if k.startswith(f"{tag}.config.")}
    t = lambda name: torch.from_numpy(data[f"{tag}.{name}"].astype(np.float64))
    m = pl.PlainModel(
        vocab_size=cfg["vocab_size"], hidden_size=cfg["hidden_size"], num_heads=cfg["num_heads"],
        num_kv_heads=cfg["num_kv_heads"], head_dim=cfg["head_dim"],
        intermediate_size=cfg["intermediate_size"], rope_theta=float(cfg["rope_theta"]),
        rms_norm_eps=float(cfg["rms_norm_eps"]), embed=t("tok_embeddings"),
        final_norm=t("output_norm"), lm_head=t("lm_head"))
    for i in range(cfg["num_layers"]):
        g = lambda name: t(f"layers.{i}.{name}")
        m.layers.append(pl.PlainLayer(
            input_norm=g("attn_norm"), wq=g("wq"), wk=g("wk"), wv=g("wv"), wo=g("wo"),
            post_norm=g("ffn_norm"), w_gate=g("gate_proj"), w_up=g("up_proj"), w_down=g("down_proj")))
    return m


@pytest.mark.parametrize("tag", ["a", "b"])
def test_plain_matches_reference_model(tag):
    data = np.load(GOLDEN)
    m = _model(data, tag)
    prompt = data[f"{tag}.prompt"].tolist()
    want = torch.from_numpy(data[f"{tag}.logits"]).double()
    got = pl.forward_logits(m, prompt)
    # the reference model runs in float32: its own rounding is the only difference
    err = (got - want).abs().max().item() / want.abs().max().item()
    assert err < 2e-6, err
    steps = len(data[f"{tag}.greedy"])
    assert pl.greedy_decode(m, prompt, steps) == data[f"{tag}.greedy"].tolist()
