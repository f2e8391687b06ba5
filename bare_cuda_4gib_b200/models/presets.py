"""Named Llama shapes for the random-weights mode of the command line tools and the benchmark.
The numbers are what the respective config.json files hold; they are data for `LlamaConfig`,
not constants of the engine."""

PRESETS = {
    "tinyA": dict(vocab_size=256, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=16, intermediate_size=176, max_position_embeddings=128,
                  rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False),
    "tinyB": dict(vocab_size=320, hidden_size=96, num_hidden_layers=3, num_attention_heads=3,
                  num_key_value_heads=1, head_dim=32, intermediate_size=256, max_position_embeddings=256,
                  rope_theta=500000.0, rms_norm_eps=1e-6, tie_word_embeddings=True),
    "tinyllama": dict(vocab_size=32000, hidden_size=2048, num_hidden_layers=22, num_attention_heads=32,
                      num_key_value_heads=4, intermediate_size=5632, max_position_embeddings=2048,
                      rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False),
    "llama2-7b": dict(vocab_size=32000, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
                      num_key_value_heads=32, intermediate_size=11008, max_position_embeddings=4096,
                      rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False),
    "llama3-8b": dict(vocab_size=128256, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
                      num_key_value_heads=8, intermediate_size=14336, max_position_embeddings=8192,
                      rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=False),
}


def preset_config(name: str, **overrides):
    from ..config.llama import LlamaConfig
    from ..errors import ConfigError

    if name not in PRESETS:
        raise ConfigError(f"unknown preset '{name}' (known: {sorted(PRESETS)})")
    d = dict(PRESETS[name], architectures=["LlamaForCausalLM"])
    d.update(overrides)
    return LlamaConfig.from_dict(d)
