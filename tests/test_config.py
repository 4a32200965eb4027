import json

import pytest

from qwen3_runtime_b200.config import (
    ConfigError, EngineConfig, LayerRun, ModelSpec, PartSpec, Qwen3Config, load_config,
    register_architecture, registered_architectures, resolve_architecture, unregister_architecture,
)
from helpers import TINY


def _raw(**over):
    raw = TINY["B"]["config"].to_hf_config()
    raw.update(over)
    return raw


def test_round_trip_through_config_json(tmp_path):
    for spec in TINY.values():
        cfg = spec["config"]
        (tmp_path / "config.json").write_text(json.dumps(cfg.to_hf_config()))
        arch, got = load_config(tmp_path)
        assert arch.name == "Qwen3ForCausalLM" and got == cfg


def test_head_dim_defaults_to_hidden_over_heads():
    raw = _raw()
    del raw["head_dim"]
    assert Qwen3Config.from_hf_config(raw).head_dim == raw["hidden_size"] // raw["num_attention_heads"]


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                                 "num_key_value_heads", "intermediate_size", "rms_norm_eps", "rope_theta",
                                 "max_position_embeddings", "tie_word_embeddings"])
def test_required_keys(key):
    raw = _raw()
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_hf_config(raw)


@pytest.mark.parametrize("over", [dict(architectures=["LlamaForCausalLM"]), dict(hidden_act="gelu"),
                                  dict(use_sliding_window=True), dict(rope_scaling={"type": "yarn"}),
                                  dict(attention_bias=True), dict(num_key_value_heads=3), dict(head_dim=15)])
def test_rejections(over):
    with pytest.raises(ConfigError):
        Qwen3Config.from_hf_config(_raw(**over))


def test_registry_names_and_extension():
    assert "Qwen3ForCausalLM" in registered_architectures()
    with pytest.raises(ConfigError, match="unsupported architectures"):
        resolve_architecture({"architectures": ["Nope"]})
    register_architecture("ToyForCausalLM", Qwen3Config, lambda cfg: None)
    try:
        assert resolve_architecture({"architectures": ["ToyForCausalLM"]}).name == "ToyForCausalLM"
        with pytest.raises(ValueError):
            register_architecture("ToyForCausalLM", Qwen3Config, lambda cfg: None)
    finally:
        unregister_architecture("ToyForCausalLM")


def test_spec_carries_every_size_from_config():
    from qwen3_runtime_b200.models.qwen3 import qwen3_spec

    for spec in TINY.values():
        cfg = spec["config"]
        ms = qwen3_spec(cfg)
        assert len(ms.blocks) == cfg.num_hidden_layers and ms.vocab_size == cfg.vocab_size
        mixer = ms.blocks[0]["mixer"]
        assert (mixer["num_heads"], mixer["num_kv_heads"], mixer["head_dim"]) == (
            cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim)
        assert mixer["qk_norm_eps"] == cfg.rms_norm_eps and mixer["position"]["theta"] == cfg.rope_theta
        assert ms.blocks[0]["feed_forward"]["intermediate_size"] == cfg.intermediate_size
        assert ms.final_norm["eps"] == cfg.rms_norm_eps and ms.tie_word_embeddings == cfg.tie_word_embeddings


def test_run_order_is_checked():
    norm = PartSpec("rmsnorm", dict(size=8, eps=1e-6))
    blocks = (PartSpec("pre_norm"), PartSpec("pre_norm"))
    ok = ModelSpec(10, 8, blocks, (LayerRun(0, 0), LayerRun(1, 1), LayerRun(0, 2), LayerRun(1, 0, writes=False)), norm, True)
    assert len(ok.order) == 4
    with pytest.raises(ValueError, match="written by two"):
        ModelSpec(10, 8, blocks, (LayerRun(0, 0), LayerRun(1, 0)), norm, True)
    with pytest.raises(ValueError, match="before any entry writes"):
        ModelSpec(10, 8, blocks, (LayerRun(0, 1, writes=False),), norm, True)
    with pytest.raises(ValueError, match="names block"):
        ModelSpec(10, 8, blocks, (LayerRun(2, 0),), norm, True)


def test_engine_config():
    assert EngineConfig(dtype="bf16").dtype == "bfloat16" and EngineConfig(dtype="fp32").dtype == "float32"
    for bad in (dict(block_size=0), dict(max_num_seqs=0), dict(max_num_batched_tokens=0), dict(dtype="fp16"),
                dict(num_kv_blocks=0)):
        with pytest.raises(ValueError):
            EngineConfig(**bad)


def test_pinned_config_refuses_another_model(tmp_path):
    """A deployment may pin the model it expects (a config.json); a folder with another model is
    refused before a weight is read, with every differing size in the message; sizes that do
    not shape tensors or arithmetic (context length, eps) may differ."""
    cfg = TINY["B"]["config"]
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_hf_config()))
    pin = tmp_path / "pin.json"
    pin.write_text(json.dumps({**cfg.to_hf_config(), "max_position_embeddings": 77, "rms_norm_eps": 1e-3}))
    assert load_config(tmp_path, pin)[1] == cfg
    pin.write_text(json.dumps(_raw(num_hidden_layers=cfg.num_hidden_layers + 1, rope_theta=123.0)))
    with pytest.raises(ConfigError) as err:
        load_config(tmp_path, pin)
    assert "num_hidden_layers" in str(err.value) and "rope_theta" in str(err.value) and "vocab_size" not in str(err.value)
