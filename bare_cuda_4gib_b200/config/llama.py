"""Typed configuration of the Llama dense decoder, read from the keys of a Hugging Face
`config.json`.

cuongvng/bare-cuda-4gib carries the same ten numbers in its model-file header
(engine/include/llm/config.h:24-35), filled offline from these keys
(tools/convert/convert_weights.py:35-46: num_key_value_heads defaults to num_attention_heads,
head_dim = hidden_size // num_attention_heads, max_position_embeddings defaults to 2048,
rope_theta to 10000.0, rms_norm_eps to 1e-5).  No size and no constant that config.json gives
is written anywhere else in the package.
"""

from __future__ import annotations

import math
from dataclasses import asdict, dataclass
from typing import Any, Dict, List, Optional

from ..errors import ConfigError


def _require(d: Dict[str, Any], key: str, kind=int):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    value = d[key]
    if kind is int and (isinstance(value, bool) or not isinstance(value, int)):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {value!r}")
    if kind is float and (isinstance(value, bool) or not isinstance(value, (int, float))):
        raise ConfigError(f"config.json: '{key}' must be a number, got {value!r}")
    return kind(value)


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    max_position_embeddings: int = 2048
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    tie_word_embeddings: bool = False
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[Any] = None
    torch_dtype: str = "bfloat16"
    architectures: tuple = ("LlamaForCausalLM",)

    ARCHITECTURE = "LlamaForCausalLM"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LlamaConfig":
        nh = _require(d, "num_attention_heads")
        hidden = _require(d, "hidden_size")
        nkv = d.get("num_key_value_heads")
        nkv = nh if nkv is None else _require(d, "num_key_value_heads")
        if nh <= 0:
            raise ConfigError(f"config.json: 'num_attention_heads' must be positive, got {nh}")
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % nh:
                raise ConfigError(f"config.json: 'hidden_size' {hidden} is not a multiple of "
                                  f"'num_attention_heads' {nh} and no 'head_dim' is given")
            head_dim = hidden // nh
        else:
            head_dim = _require(d, "head_dim")
        if d.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"config.json: 'hidden_act' {d['hidden_act']!r} is not supported "
                              "(the Llama feed-forward gates with 'silu')")
        if d.get("rope_scaling") not in (None, {}):
            raise ConfigError("config.json: 'rope_scaling' is set; scaled rotary positions are not supported")
        for key in ("attention_bias", "mlp_bias"):
            if d.get(key, False):
                raise ConfigError(f"config.json: '{key}' is true; projections with a bias are not supported")
        cfg = cls(
            vocab_size=_require(d, "vocab_size"),
            hidden_size=hidden,
            num_hidden_layers=_require(d, "num_hidden_layers"),
            num_attention_heads=nh,
            num_key_value_heads=nkv,
            head_dim=head_dim,
            intermediate_size=_require(d, "intermediate_size"),
            max_position_embeddings=int(d.get("max_position_embeddings", 2048) or 2048),
            rope_theta=float(d.get("rope_theta", 10000.0) or 10000.0),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-5) or 1e-5),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            bos_token_id=d.get("bos_token_id"),
            eos_token_id=d.get("eos_token_id"),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
            architectures=tuple(d.get("architectures") or (cls.ARCHITECTURE,)),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for key in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "head_dim", "intermediate_size", "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"config.json: '{key}' must be positive, got {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"config.json: 'num_attention_heads' {self.num_attention_heads} is not a "
                              f"multiple of 'num_key_value_heads' {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: 'head_dim' {self.head_dim} must be even for rotary positions")
        if not (self.rope_theta > 0 and math.isfinite(self.rope_theta)):
            raise ConfigError(f"config.json: 'rope_theta' must be a positive number, got {self.rope_theta}")
        if not (self.rms_norm_eps > 0 and math.isfinite(self.rms_norm_eps)):
            raise ConfigError(f"config.json: 'rms_norm_eps' must be a positive number, got {self.rms_norm_eps}")

    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration is read back from."""
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        d["model_type"] = "llama"
        d["hidden_act"] = "silu"
        return d

    @property
    def stop_ids(self) -> List[int]:
        if self.eos_token_id is None:
            return []
        if isinstance(self.eos_token_id, (list, tuple)):
            return [int(t) for t in self.eos_token_id]
        return [int(self.eos_token_id)]
