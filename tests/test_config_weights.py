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


def _as_shards(src, dst, n_shards=3, index_extra=None, drop=None):
    """Rewrites the single-file model folder `src` as `n_shards` shards plus an index in `dst`."""
    from bare_cuda_4gib_b200.weights import SafetensorsFile, write_safetensors
    with SafetensorsFile(src / "model.safetensors") as f:
        tensors = {n: f.tensor(n) for n in f.entries}
    names = sorted(tensors)
    weight_map = {}
    for i in range(n_shards):
        shard = f"model-{i + 1:05d}-of-{n_shards:05d}.safetensors"
        mine = {n: tensors[n] for n in names[i::n_shards]}
        for n in mine:
            weight_map[n] = shard
        if drop != shard:
            write_safetensors(dst / shard, mine)
    weight_map.update(index_extra or {})
    (dst / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    (dst / "config.json").write_text((src / "config.json").read_text())
    return tensors, weight_map


def test_sharded_checkpoint_loads_bit_equal_to_the_single_file(tmp_path):
    from bare_cuda_4gib_b200.engine.model import load_model
    src = H.model_folder("B")
    _as_shards(src, tmp_path, 3)
    one, _ = load_model(src, "bfloat16", "cpu")
    many, _ = load_model(tmp_path, "bfloat16", "cpu")
    a = {id(p): p for p in one.all_parts()}
    for p1, p2 in zip(one.all_parts(), many.all_parts()):
        for name in p1.tensors:
            assert torch.equal(p1.tensors[name], p2.tensors[name]), name
    for b1, b2 in zip(one.blocks, many.blocks):
        assert torch.equal(b1.mixer.qkv.weight, b2.mixer.qkv.weight) and torch.equal(b1.ffn.gate_up.weight, b2.ffn.gate_up.weight)


def test_shard_problems_are_part_of_the_one_error(tmp_path):
    from bare_cuda_4gib_b200.engine.model import load_model
    from bare_cuda_4gib_b200.errors import WeightError
    from bare_cuda_4gib_b200.weights import write_safetensors
    src = H.model_folder("A")
    missing_shard = "model-00002-of-00003.safetensors"
    tensors, weight_map = _as_shards(src, tmp_path, 3, drop=missing_shard,
                                     index_extra={"model.layers.9.ghost.weight": "model-00001-of-00003.safetensors"})
    # a tensor that two shards hold
    twice = next(n for n, s in weight_map.items() if s == "model-00001-of-00003.safetensors" and "ghost" not in n)
    third = {n: tensors[n] for n, s in weight_map.items() if s == "model-00003-of-00003.safetensors"}
    third[twice] = tensors[twice]
    write_safetensors(tmp_path / "model-00003-of-00003.safetensors", third)
    with pytest.raises(WeightError) as e:
        load_model(tmp_path, "float32", "cpu")
    text = str(e.value)
    assert text.count("do not match the model") == 1
    assert missing_shard in text and "cannot open" in text                         # the missing shard file
    assert "ghost" in text and "does not hold it" in text                          # listed in the index, absent from its shard
    assert f"'{twice}' is held by 2 shards" in text                                # present in two shards
    assert "missing tensors" in text                                               # what the lost shard held
    (tmp_path / "model.safetensors.index.json").write_text("{}")
    with pytest.raises(WeightError, match="not a usable shard index"):
        load_model(tmp_path, "float32", "cpu")


def test_duplicate_name_in_a_header_is_refused(tmp_path):
    from bare_cuda_4gib_b200.errors import WeightError
    from bare_cuda_4gib_b200.weights import SafetensorsFile
    header = ('{"t":{"dtype":"F32","shape":[2],"data_offsets":[0,8]},'
              '"t":{"dtype":"F32","shape":[2],"data_offsets":[8,16]}}').encode()
    bad = tmp_path / "model.safetensors"
    bad.write_bytes(len(header).to_bytes(8, "little") + header + b"\0" * 16)
    with pytest.raises(WeightError, match="listed twice"):
        SafetensorsFile(bad)


def test_weights_lie_in_one_arena_and_fused_matrices_are_views():
    """Every tensor at a 1,024-byte offset of one allocation; [Wq; Wk; Wv] and [Wgate; Wup] back to
    back, so the fused matrices are views; known non-parameter buffers are ignored."""
    from bare_cuda_4gib_b200.engine.model import load_model
    from bare_cuda_4gib_b200.weights.loader import ARENA_ALIGN
    model, _ = load_model(H.model_folder("A"), "bfloat16", "cpu")
    storages = set()
    for part in model.all_parts():
        for t in part.tensors.values():
            storages.add(t.untyped_storage().data_ptr())
    for block in model.blocks:
        for lin in (block.mixer.qkv, block.mixer.o, block.ffn.gate_up, block.ffn.down):
            storages.add(lin.weight.untyped_storage().data_ptr())
            assert (lin.weight.data_ptr() - lin.weight.untyped_storage().data_ptr()) % ARENA_ALIGN == 0
        assert block.mixer.qkv.weight.shape == (4 * 16 + 2 * 2 * 16, 64)
    assert len(storages) == 1


def test_rotary_buffers_of_old_exports_are_ignored(tmp_path):
    from bare_cuda_4gib_b200.engine.model import load_model
    from bare_cuda_4gib_b200.weights import SafetensorsFile, write_safetensors
    src = H.model_folder("A")
    with SafetensorsFile(src / "model.safetensors") as f:
        tensors = {n: f.tensor(n) for n in f.entries}
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    (tmp_path / "config.json").write_text((src / "config.json").read_text())
    write_safetensors(tmp_path / "model.safetensors", tensors)
    load_model(tmp_path, "float32", "cpu")


def test_random_model_without_a_file_equals_the_written_folder():
    from bare_cuda_4gib_b200.engine.model import load_model, random_model
    from bare_cuda_4gib_b200.config import LlamaConfig
    for name, cfg in (("A", H.TINY_A), ("B", H.TINY_B)):
        for dtype in ("bfloat16", "float32"):
            a, _ = load_model(H.model_folder(name, 5), dtype, "cpu")
            b = random_model(LlamaConfig.from_dict(cfg), 5, dtype, "cpu")
            for p1, p2 in zip(a.all_parts(), b.all_parts()):
                for n in p1.tensors:
                    assert p1.tensors[n].dtype == p2.tensors[n].dtype and torch.equal(p1.tensors[n], p2.tensors[n]), n
            assert torch.equal(a.blocks[0].mixer.qkv.weight, b.blocks[0].mixer.qkv.weight)


def test_large_tensor_goes_through_the_staging_buffer_in_pieces(tmp_path, monkeypatch):
    from bare_cuda_4gib_b200.weights import loader, write_safetensors
    from bare_cuda_4gib_b200.parts.spec import WeightSpec
    monkeypatch.setattr(loader, "STAGING_BYTES", 4096)
    t = {"w": torch.randn(300, 77).to(torch.float16), "i": torch.arange(5000, dtype=torch.int64),
         "f": torch.randn(3000)}
    write_safetensors(tmp_path / "model.safetensors", t)
    expected = {n: WeightSpec(n, tuple(x.shape)) for n, x in t.items()}
    got = loader.load_weights(tmp_path, expected, {}, (), torch.bfloat16, "cpu")
    assert got["w"].dtype == torch.bfloat16 and torch.equal(got["w"], t["w"].to(torch.bfloat16))
    assert got["i"].dtype == torch.int32 and torch.equal(got["i"], t["i"].to(torch.int32))
    assert got["f"].dtype == torch.float32 and torch.equal(got["f"], t["f"])
