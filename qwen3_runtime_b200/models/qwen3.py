"""Qwen3 dense expressed as data for the generic decoder.

Pre-norm blocks of GQA attention (per-head RMSNorm on q and k before NeoX RoPE)
and a SwiGLU feed-forward, RMSNorm everywhere with one eps, tied or untied head.
Parity: qwen3_runtime/models/qwen3.py:62-266 (structure) and
qwen3_runtime/utils/loader.py:33-54 (tensor names).
"""

from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..config.registry import register_architecture
from ..config.spec import ModelSpec, PartSpec


def qwen3_spec(cfg: Qwen3Config) -> ModelSpec:
    position = PartSpec(
        "rope_neox",
        dict(rotary_dim=cfg.head_dim, theta=cfg.rope_theta, max_positions=cfg.max_position_embeddings),
    )
    mixer = PartSpec(
        "paged_attention",
        dict(
            hidden_size=cfg.hidden_size,
            num_heads=cfg.num_attention_heads,
            num_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim,
            qk_norm_eps=cfg.rms_norm_eps,
            position=position,
            window=None,
        ),
    )
    feed_forward = PartSpec(
        "gated_mlp",
        dict(hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size, activation="silu"),
    )
    norm = PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps))
    block = PartSpec(
        "pre_norm",
        dict(
            mixer=mixer,
            feed_forward=feed_forward,
            mixer_norm=norm,
            feed_forward_norm=norm,
            mixer_prefix="self_attn.",
            feed_forward_prefix="mlp.",
            mixer_norm_prefix="input_layernorm.",
            feed_forward_norm_prefix="post_attention_layernorm.",
        ),
    )
    n = cfg.num_hidden_layers
    return ModelSpec(
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        blocks=tuple(block for _ in range(n)),
        order=ModelSpec.sequential_order(n),
        final_norm=norm,
        tie_word_embeddings=cfg.tie_word_embeddings,
    )


def tiny_qwen3_config() -> Qwen3Config:
    """The sizes of the reference's built-in tiny model (qwen3_runtime/llm.py:168-181), with a
    head size the attention kernels accept."""
    return Qwen3Config(vocab_size=32, hidden_size=32, num_hidden_layers=2, num_attention_heads=2,
                       num_key_value_heads=1, head_dim=16, intermediate_size=64, rms_norm_eps=1e-6,
                       rope_theta=10000.0, max_position_embeddings=128, tie_word_embeddings=True)


register_architecture(Qwen3Config.architecture, Qwen3Config, qwen3_spec, tiny_config=tiny_qwen3_config)
