"""Typed model configuration read from an architecture's own ``config.json`` keys.

Every size and constant the model uses comes from here; nothing is hard-wired in
the parts or kernels.  Parity: qwen3_runtime/models/qwen3.py:19-59 (field set,
required keys, rejections).
"""

from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any, Mapping


class ConfigError(ValueError):
    """A ``config.json`` that this engine cannot run, with the reason."""


def _require(raw: Mapping[str, Any], key: str) -> Any:
    if key not in raw:
        raise ConfigError(f"config.json is missing required key {key!r}")
    return raw[key]


@dataclass(frozen=True)
class Qwen3Config:
    """Hyper-parameters of a Qwen3 dense decoder (qwen3_runtime/models/qwen3.py:19-31)."""

    # what a pinned config.json is compared on (qwen3_runtime/utils/loader.py:20-30)
    pin_fields = ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
                  "intermediate_size", "vocab_size", "rope_theta", "tie_word_embeddings")

    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool

    architecture = "Qwen3ForCausalLM"

    def __post_init__(self) -> None:
        for name in (
            "vocab_size",
            "hidden_size",
            "num_hidden_layers",
            "num_attention_heads",
            "num_key_value_heads",
            "head_dim",
            "intermediate_size",
            "max_position_embeddings",
        ):
            if int(getattr(self, name)) < 1:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)!r}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads={self.num_key_value_heads}"
            )
        if self.head_dim % 2:
            raise ConfigError(f"head_dim={self.head_dim} must be even for rotary pairs")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps!r}")
        if not self.rope_theta > 0:
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta!r}")

    @classmethod
    def from_hf_config(cls, raw: Mapping[str, Any]) -> "Qwen3Config":
        """Parse and validate the Hugging Face keys (qwen3_runtime/models/qwen3.py:33-59)."""
        arch = raw.get("architectures") or []
        if cls.architecture not in arch:
            raise ConfigError(f"unsupported architectures: {list(arch)}")
        if raw.get("hidden_act") != "silu":
            raise ConfigError(f"unsupported hidden_act: {raw.get('hidden_act')!r}")
        if raw.get("use_sliding_window"):
            raise ConfigError("use_sliding_window=true is not part of Qwen3 dense as served here")
        if raw.get("rope_scaling") not in (None, {}):
            raise ConfigError(f"unsupported rope_scaling: {raw.get('rope_scaling')!r}")
        if raw.get("attention_bias"):
            raise ConfigError("attention_bias=true is not supported (Qwen3 dense has no qkv bias)")
        hidden = int(_require(raw, "hidden_size"))
        heads = int(_require(raw, "num_attention_heads"))
        head_dim = int(raw.get("head_dim") or hidden // heads)
        return cls(
            vocab_size=int(_require(raw, "vocab_size")),
            hidden_size=hidden,
            num_hidden_layers=int(_require(raw, "num_hidden_layers")),
            num_attention_heads=heads,
            num_key_value_heads=int(_require(raw, "num_key_value_heads")),
            head_dim=head_dim,
            intermediate_size=int(_require(raw, "intermediate_size")),
            rms_norm_eps=float(_require(raw, "rms_norm_eps")),
            rope_theta=float(_require(raw, "rope_theta")),
            max_position_embeddings=int(_require(raw, "max_position_embeddings")),
            tie_word_embeddings=bool(_require(raw, "tie_word_embeddings")),
        )

    def to_hf_config(self) -> dict[str, Any]:
        """The ``config.json`` dictionary that :meth:`from_hf_config` reads back."""
        out = asdict(self)
        out.update(
            architectures=[self.architecture],
            model_type="qwen3",
            hidden_act="silu",
            attention_bias=False,
            use_sliding_window=False,
            rope_scaling=None,
        )
        return out
