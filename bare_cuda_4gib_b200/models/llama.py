"""The Llama dense decoder laid out as parts: every layer is a pre-norm block of grouped-query
attention with rotary positions and a SwiGLU feed-forward; layers run once each, in order
(cuongvng/bare-cuda-4gib engine/src/model.cpp:526-615).  Tensor names are the Hugging Face ones
that the reference's converter renames offline (tools/convert/convert_weights.py:68-83).
"""

from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        position = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta})
        layers.append(LayerSpec(
            mixer_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                                {"weight": p + "input_layernorm.weight"}),
            mixer=PartSpec("attention",
                           {"hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
                            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                            "window": None, "position": position},
                           {"q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
                            "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight"}),
            ffn_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                              {"weight": p + "post_attention_layernorm.weight"}),
            ffn=PartSpec("swiglu", {"hidden": cfg.hidden_size, "intermediate": cfg.intermediate_size},
                         {"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
                          "down": p + "mlp.down_proj.weight"}),
            block="prenorm"))
    sizes = {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size}
    embed_name = "model.embed_tokens.weight"
    tied = cfg.tie_word_embeddings
    return ModelSpec(
        architecture=LlamaConfig.ARCHITECTURE,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embed=PartSpec("table", sizes, {"weight": embed_name}),
        layers=layers,
        order=[LayerCall(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                            {"weight": "model.norm.weight"}),
        head=PartSpec("linear", sizes, {"weight": embed_name if tied else "lm_head.weight"}),
        # a checkpoint without lm_head.weight shares the embedding table
        aliases={} if tied else {"lm_head.weight": embed_name},
        # buffers that older exports store beside the parameters, and the head of a tied model
        ignorable=("*.rotary_emb.inv_freq",) + (("lm_head.weight",) if tied else ()),
    )


register_architecture(LlamaConfig.ARCHITECTURE, LlamaConfig, llama_spec)
