import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from emulated_ops import TorchOps
from helpers import TINY, make_model_dir
from qwen3_runtime_b200.engine.factory import load_model
from qwen3_runtime_b200.weights import WeightError, expected_tensors_for, random_state


def test_random_model_is_a_function_of_config_and_seed(tmp_path):
    cfg = TINY["A"]["config"]
    a, b, c = random_state(cfg, 5), random_state(cfg, 5), random_state(cfg, 6)
    assert list(a) == list(expected_tensors_for(cfg))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert any(not torch.equal(a[k], c[k]) for k in a)
    assert a["model.layers.0.input_layernorm.weight"].float().mean().item() == pytest.approx(1.0, abs=0.05)
    assert all(v.dtype == torch.bfloat16 for v in a.values())
    assert "lm_head.weight" not in a and "lm_head.weight" in random_state(TINY["B"]["config"], 0)


def test_folder_has_config_and_safetensors(tmp_path):
    folder = make_model_dir(tmp_path, "B")
    raw = json.loads((folder / "config.json").read_text())
    assert raw["architectures"] == ["Qwen3ForCausalLM"] and raw["num_hidden_layers"] == 3
    tensors = load_file(str(folder / "model.safetensors"))
    exp = expected_tensors_for(TINY["B"]["config"])
    assert set(tensors) == set(exp) and all(tuple(tensors[k].shape) == exp[k].shape for k in exp)


def test_placement_matrix_in_compute_dtype_vector_in_float32(tmp_path):
    for store in ("bfloat16", "float32"):
        folder = make_model_dir(tmp_path, "A", store_dtype=store)
        for dtype, td in (("bfloat16", torch.bfloat16), ("float32", torch.float32)):
            model, _cfg, _raw = load_model(folder, dtype=dtype, device="cpu", ops=TorchOps())
            blk = model.blocks[0]
            assert model.embed.dtype == td and blk.mixer.qkv_weight.dtype == td and blk.feed_forward.down_weight.dtype == td
            assert blk.mixer_norm.weight.dtype == torch.float32 and blk.mixer.q_norm_weight.dtype == torch.float32
            assert model.head is model.embed  # tied
    # a vector stored in 32-bit keeps all its bits
    folder = make_model_dir(tmp_path, "A", store_dtype="float32")
    stored = load_file(str(folder / "model.safetensors"))["model.norm.weight"]
    model, _, _ = load_model(folder, dtype="bfloat16", device="cpu", ops=TorchOps())
    assert torch.equal(model.final_norm.weight, stored)


def test_fused_weights_keep_row_order(tmp_path):
    folder = make_model_dir(tmp_path, "B")
    t = load_file(str(folder / "model.safetensors"))
    model, cfg, _ = load_model(folder, dtype="float32", device="cpu", ops=TorchOps())
    p = "model.layers.1.self_attn."
    want = torch.cat([t[p + "q_proj.weight"], t[p + "k_proj.weight"], t[p + "v_proj.weight"]]).float()
    assert torch.equal(model.blocks[1].mixer.qkv_weight, want)
    m = "model.layers.2.mlp."
    assert torch.equal(model.blocks[2].feed_forward.gate_up_weight,
                       torch.cat([t[m + "gate_proj.weight"], t[m + "up_proj.weight"]]).float())
    assert model.head is not model.embed and torch.equal(model.head, t["lm_head.weight"].float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_model_dir(tmp_path, "A")
    t = load_file(str(folder / "model.safetensors"))
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    t["model.layers.0.self_attn.o_proj.weight"] = torch.zeros(64, 32, dtype=torch.bfloat16)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()  # a tied model may carry a copy: ignored
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "config.json").write_text((folder / "config.json").read_text())
    save_file(t, str(bad / "model.safetensors"))
    with pytest.raises(WeightError) as err:
        load_model(bad, dtype="float32", device="cpu", ops=TorchOps())
    msg = str(err.value)
    assert "missing tensors (2)" in msg and "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected tensors (1)" in msg and "rotary_emb.inv_freq" in msg
    assert "wrong shapes (1)" in msg and "o_proj.weight: checkpoint [64, 32], model [64, 64]" in msg
    assert "lm_head" not in msg


def test_sharded_checkpoint_with_index(tmp_path):
    folder = make_model_dir(tmp_path, "A")
    t = load_file(str(folder / "model.safetensors"))
    names = sorted(t)
    shard = tmp_path / "sharded"
    shard.mkdir()
    (shard / "config.json").write_text((folder / "config.json").read_text())
    half = len(names) // 2
    save_file({k: t[k] for k in names[:half]}, str(shard / "model-00001-of-00002.safetensors"))
    save_file({k: t[k] for k in names[half:]}, str(shard / "model-00002-of-00002.safetensors"))
    wm = {k: "model-00001-of-00002.safetensors" for k in names[:half]}
    wm.update({k: "model-00002-of-00002.safetensors" for k in names[half:]})
    (shard / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    a, _, _ = load_model(folder, dtype="float32", device="cpu", ops=TorchOps())
    b, _, _ = load_model(shard, dtype="float32", device="cpu", ops=TorchOps())
    assert torch.equal(a.blocks[1].mixer.qkv_weight, b.blocks[1].mixer.qkv_weight)
    empty = tmp_path / "empty"
    empty.mkdir()
    (empty / "config.json").write_text((folder / "config.json").read_text())
    with pytest.raises(FileNotFoundError):
        load_model(empty, dtype="float32", device="cpu", ops=TorchOps())
