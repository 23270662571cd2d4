"""The safetensors loader and the random-weights mode (no GPU: tensors are loaded to the CPU)."""
import json

import pytest
import torch
from safetensors.torch import load_file, save_file

import tiny_models as tm
from cisr_b200.config.llama import LlamaConfig
from cisr_b200.engine.model import Model
from cisr_b200.weights import WeightError, load_model_tensors, write_random_model


def needs_of(cfg, dtype=torch.bfloat16):
    return Model(LlamaConfig.from_dict(cfg).to_spec(), dtype).tensor_needs()


def test_random_model_folder_round_trip(tmp_path):
    path = write_random_model(tmp_path / "m", tm.TINY_B, seed=5, store_dtype="bfloat16")
    assert sorted(p.name for p in path.iterdir()) == ["config.json", "model.safetensors"]
    raw = json.loads((path / "config.json").read_text())
    assert LlamaConfig.from_dict(raw) == LlamaConfig.from_dict(dict(tm.TINY_B, torch_dtype="bfloat16"))
    stored = load_file(str(path / "model.safetensors"))
    assert set(stored) == set(tm.tensor_shapes(tm.TINY_B))
    assert all(t.dtype == torch.bfloat16 for t in stored.values())
    loaded = load_model_tensors(path, needs_of(tm.TINY_B), torch.bfloat16, "cpu")
    for name, shape in tm.tensor_shapes(tm.TINY_B).items():
        assert tuple(loaded[name].shape) == shape and torch.equal(loaded[name], stored[name])
    again = write_random_model(tmp_path / "n", tm.TINY_B, seed=5, store_dtype="bfloat16")
    other = write_random_model(tmp_path / "o", tm.TINY_B, seed=6, store_dtype="bfloat16")
    name = "model.layers.1.mlp.up_proj.weight"
    assert torch.equal(load_file(str(again / "model.safetensors"))[name], stored[name])
    assert not torch.equal(load_file(str(other / "model.safetensors"))[name], stored[name])
    w = stored[name].float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(stored["model.norm.weight"].float().mean()) - 1.0) < 0.05


def test_tied_head_is_not_stored_and_is_shared():
    needs = needs_of(tm.TINY_A)
    assert needs["lm_head.weight"].alias == "model.embed_tokens.weight"
    assert "lm_head.weight" not in tm.tensor_shapes(tm.TINY_A)


def test_kept_dtypes(tmp_path):
    weights = tm.make_weights(tm.TINY_A, 1)
    path = tm.write_model_dir(tmp_path / "f32", tm.TINY_A, weights, store_dtype=torch.float32)
    as_bf16 = load_model_tensors(path, needs_of(tm.TINY_A), torch.bfloat16, "cpu")
    assert as_bf16["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16      # matrices: the compute dtype
    assert as_bf16["model.layers.0.input_layernorm.weight"].dtype == torch.float32   # stored in 32-bit: stays so
    path16 = tm.write_model_dir(tmp_path / "bf16", tm.TINY_A, weights, store_dtype=torch.bfloat16)
    as_f32 = load_model_tensors(path16, needs_of(tm.TINY_A, torch.float32), torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in as_f32.values())
    assert load_model_tensors(path16, needs_of(tm.TINY_A), torch.bfloat16, "cpu")["model.norm.weight"].dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    weights = tm.torch_weights(tm.make_weights(tm.TINY_B, 2))
    del weights["model.layers.2.mlp.down_proj.weight"], weights["lm_head.weight"]
    weights["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(96, 95)
    weights["model.layers.1.input_layernorm.weight"] = torch.zeros(97)
    weights["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    (tmp_path / "config.json").write_text(json.dumps(tm.TINY_B))
    save_file(weights, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightError) as err:
        load_model_tensors(tmp_path, needs_of(tm.TINY_B), torch.bfloat16, "cpu")
    text = str(err.value)
    assert "missing tensors (2): lm_head.weight, model.layers.2.mlp.down_proj.weight" in text
    assert "unexpected tensors (1): model.layers.0.self_attn.rotary_emb.inv_freq" in text
    assert "wrong shapes (2)" in text and "[96, 95]" in text and "[97]" in text


def test_no_checkpoint_and_duplicates(tmp_path):
    with pytest.raises(FileNotFoundError):
        load_model_tensors(tmp_path, needs_of(tm.TINY_A), torch.bfloat16, "cpu")
    weights = tm.torch_weights(tm.make_weights(tm.TINY_A, 2))
    save_file(weights, str(tmp_path / "a.safetensors"))
    save_file({"model.norm.weight": weights["model.norm.weight"]}, str(tmp_path / "b.safetensors"))
    with pytest.raises(WeightError, match="duplicate tensor model.norm.weight"):
        load_model_tensors(tmp_path, needs_of(tm.TINY_A), torch.bfloat16, "cpu")


def test_untied_model_needs_its_head(tmp_path):
    weights = tm.make_weights(tm.TINY_A, 2)                       # tied: no lm_head in the file
    tm.write_model_dir(tmp_path, dict(tm.TINY_A, tie_word_embeddings=False), weights)
    with pytest.raises(WeightError, match="missing tensors \\(1\\): lm_head.weight"):
        load_model_tensors(tmp_path, needs_of(dict(tm.TINY_A, tie_word_embeddings=False)), torch.bfloat16, "cpu")
