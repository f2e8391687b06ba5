"""Configuration, registry and weight binding (no GPU)."""

import json

import pytest
import torch

import helpers as H


def _cfg(**over):
    d = dict(H.TINY_A)
    d.update(over)
    return d


def test_config_reads_the_architectures_own_keys():
    from bare_cuda_4gib_b200.config import LlamaConfig
    c = LlamaConfig.from_dict(H.TINY_B)
    assert (c.vocab_size, c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads,
            c.head_dim, c.intermediate_size, c.rope_theta, c.rms_norm_eps, c.tie_word_embeddings) == \
           (320, 96, 3, 3, 1, 32, 256, 500000.0, 1e-6, True)
    # defaults of the reference's converter: kv heads = heads, head_dim = hidden / heads, theta, eps
    d = _cfg()
    for k in ("num_key_value_heads", "head_dim", "rope_theta", "rms_norm_eps", "max_position_embeddings"):
        d.pop(k)
    c = LlamaConfig.from_dict(d)
    assert (c.num_key_value_heads, c.head_dim, c.rope_theta, c.rms_norm_eps, c.max_position_embeddings) == \
           (4, 16, 10000.0, 1e-5, 2048)
    assert LlamaConfig.from_dict(c.to_dict()) == c


@pytest.mark.parametrize("change,word", [
    (dict(vocab_size=None), "vocab_size"), (dict(num_attention_heads=5, head_dim=None), "hidden_size"),
    (dict(num_key_value_heads=3), "num_key_value_heads"), (dict(head_dim=15), "head_dim"),
    (dict(hidden_act="gelu"), "hidden_act"), (dict(rope_scaling={"type": "linear", "factor": 2}), "rope_scaling"),
    (dict(attention_bias=True), "attention_bias"), (dict(rms_norm_eps=-1.0), "rms_norm_eps"),
    (dict(num_hidden_layers=0), "num_hidden_layers"), (dict(hidden_size="64"), "hidden_size"),
])
def test_config_errors_name_the_key(change, word):
    from bare_cuda_4gib_b200.config import LlamaConfig
    from bare_cuda_4gib_b200.errors import ConfigError
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_dict(_cfg(**change))


def test_registry_resolves_by_name_and_lists_known_ones():
    import bare_cuda_4gib_b200.models  # noqa: F401
    from bare_cuda_4gib_b200.config import resolve_architecture
    from bare_cuda_4gib_b200.errors import ConfigError
    arch = resolve_architecture(H.TINY_A)
    assert arch.name == "LlamaForCausalLM"
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        resolve_architecture({"architectures": ["SomethingElse"]})
    with pytest.raises(ConfigError, match="architectures"):
        resolve_architecture({})


def test_spec_is_data_and_order_is_a_list():
    import bare_cuda_4gib_b200.models  # noqa: F401
    from bare_cuda_4gib_b200.config import LlamaConfig, resolve_architecture
    spec = resolve_architecture(H.TINY_B).build_spec(LlamaConfig.from_dict(H.TINY_B))
    assert [c.layer for c in spec.order] == [0, 1, 2] and all(c.cache_from is None for c in spec.order)
    assert spec.layers[1].mixer.kind == "attention" and spec.layers[1].ffn.kind == "swiglu"
    assert spec.layers[1].mixer.params["kv_heads"] == 1 and spec.layers[1].mixer.params["position"].params["theta"] == 500000.0
    assert spec.head.weights["weight"] == "model.embed_tokens.weight"      # tied


def test_safetensors_round_trip_matches_the_library(tmp_path):
    from safetensors import safe_open
    from bare_cuda_4gib_b200.weights import SafetensorsFile, write_safetensors
    tensors = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
               "c": torch.randn(2, 2, 2), "d": torch.randn(4).to(torch.float16)}
    path = tmp_path / "x.safetensors"
    write_safetensors(path, tensors)
    with SafetensorsFile(path) as f:
        for n, t in tensors.items():
            assert torch.equal(f.tensor(n), t) and f.entries[n].shape == tuple(t.shape)
    with safe_open(str(path), framework="pt") as f:
        for n, t in tensors.items():
            assert torch.equal(f.get_tensor(n), t)


def test_weights_keep_their_types(tmp_path):
    """bfloat16 stays bfloat16, float16 becomes bfloat16, a 32-bit tensor stays 32-bit, integers int32;
    a float32 run widens everything."""
    from bare_cuda_4gib_b200.weights import storage_dtype
    bf, f32 = torch.bfloat16, torch.float32
    assert storage_dtype(torch.bfloat16, bf) == bf and storage_dtype(torch.float16, bf) == bf
    assert storage_dtype(torch.float32, bf) == f32 and storage_dtype(torch.int64, bf) == torch.int32
    assert storage_dtype(torch.bfloat16, f32) == f32 and storage_dtype(torch.float16, f32) == f32
    from bare_cuda_4gib_b200.engine.model import load_model
    folder = H.model_folder("A", stored="float32")
    model, _ = load_model(folder, "bfloat16", "cpu")
    assert model.final_norm.tensors["weight"].dtype == f32
    model, _ = load_model(H.model_folder("A"), "bfloat16", "cpu")
    assert model.final_norm.tensors["weight"].dtype == bf


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    from bare_cuda_4gib_b200.engine.model import load_model
    from bare_cuda_4gib_b200.errors import WeightError
    from bare_cuda_4gib_b200.weights import SafetensorsFile, write_safetensors
    src = H.model_folder("A")
    with SafetensorsFile(src / "model.safetensors") as f:
        tensors = {n: f.tensor(n) for n in f.entries}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 64).to(torch.bfloat16)
    (tmp_path / "config.json").write_text((src / "config.json").read_text())
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightError) as e:
        load_model(tmp_path, "float32", "cpu")
    text = str(e.value)
    assert "missing tensors (2)" in text and "model.norm.weight" in text and "up_proj" in text
    assert "unexpected tensors (1)" in text and "inv_freq" in text
    assert "wrong shapes (1)" in text and "k_proj" in text and "[64, 64]" in text and "[32, 64]" in text


def test_tied_and_aliased_head(tmp_path):
    from bare_cuda_4gib_b200.engine.model import load_model
    from bare_cuda_4gib_b200.weights import SafetensorsFile, write_safetensors
    model, _ = load_model(H.model_folder("B"), "float32", "cpu")       # tied in config
    assert model.head.tensors["weight"].data_ptr() == model.embed.tensors["weight"].data_ptr()
    src = H.model_folder("A")                                          # untied, lm_head dropped from the file
    with SafetensorsFile(src / "model.safetensors") as f:
        tensors = {n: f.tensor(n) for n in f.entries if n != "lm_head.weight"}
    (tmp_path / "config.json").write_text((src / "config.json").read_text())
    write_safetensors(tmp_path / "model.safetensors", tensors)
    model, _ = load_model(tmp_path, "float32", "cpu")
    assert model.head.tensors["weight"].data_ptr() == model.embed.tensors["weight"].data_ptr()


def test_file_errors(tmp_path):
    from bare_cuda_4gib_b200.errors import ConfigError, WeightError
    from bare_cuda_4gib_b200.engine.model import load_model
    from bare_cuda_4gib_b200.weights import SafetensorsFile
    with pytest.raises(ConfigError, match="cannot read"):
        load_model(tmp_path, "float32", "cpu")
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_model(tmp_path, "float32", "cpu")
    (tmp_path / "config.json").write_text(json.dumps(H.TINY_A))
    with pytest.raises(WeightError, match="cannot open"):
        load_model(tmp_path, "float32", "cpu")
    bad = tmp_path / "model.safetensors"
    bad.write_bytes(b"\x01\x00")
    with pytest.raises(WeightError, match="truncated"):
        SafetensorsFile(bad)
    bad.write_bytes((10 ** 6).to_bytes(8, "little") + b"{}")
    with pytest.raises(WeightError, match="exceeds the file"):
        SafetensorsFile(bad)
    header = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    bad.write_bytes(len(header).to_bytes(8, "little") + header + b"\0" * 8)
    with pytest.raises(WeightError, match="exceeds the file"):
        SafetensorsFile(bad)
    with pytest.raises(ConfigError, match="dtype"):
        load_model(H.model_folder("A"), "float16", "cpu")


def test_random_weights_are_seeded_and_shaped():
    from bare_cuda_4gib_b200.weights import SafetensorsFile
    a1, a2, a3 = H.model_folder("A", 7), H.model_folder("A", 8), H.model_folder("A", 7, "float32")
    with SafetensorsFile(a1 / "model.safetensors") as f1, SafetensorsFile(a2 / "model.safetensors") as f2, \
            SafetensorsFile(a3 / "model.safetensors") as f3:
        w1, w2, w3 = (f.tensor("model.layers.0.mlp.down_proj.weight") for f in (f1, f2, f3))
        assert w1.shape == (64, 176) and not torch.equal(w1, w2)
        assert torch.equal(w1, w3.to(torch.bfloat16))
        assert 0.015 < float(w3.std()) < 0.025
        n = f3.tensor("model.norm.weight")
        assert abs(float(n.mean()) - 1.0) < 0.01 and float(n.std()) < 0.02
    assert json.loads((a1 / "config.json").read_text())["architectures"] == ["LlamaForCausalLM"]
