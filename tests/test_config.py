"""Configuration, presets, the architecture registry and the model spec (no GPU)."""
import json

import pytest

import tiny_models as tm
from cisr_b200.config import ARCHITECTURES, ModelSpec, RunEntry, architecture_for, register_architecture
from cisr_b200.config import ConfigError, LlamaConfig, preset, preset_dict, preset_names


def test_every_field_comes_from_config_json():
    cfg = LlamaConfig.from_dict(tm.TINY_B)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers) == (384, 96, 250, 3)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (3, 1, 32)
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 500000.0 and not cfg.tie_word_embeddings
    assert cfg.eos_token_ids == (5,)
    assert LlamaConfig.from_dict(cfg.to_dict()) == cfg


def test_head_dim_defaults_to_hidden_over_heads_and_may_differ():
    raw = dict(tm.TINY_A)
    del raw["head_dim"]
    assert LlamaConfig.from_dict(raw).head_dim == 16
    raw["head_dim"] = 32           # wider heads than hidden/heads: allowed, the projections are sized by it
    spec = LlamaConfig.from_dict(raw).to_spec()
    assert spec.layers[0].mixer["head_dim"] == 32


def test_eos_may_be_a_list_and_kv_heads_default_to_heads():
    raw = dict(tm.TINY_A, eos_token_id=[2, 7])
    del raw["num_key_value_heads"]
    cfg = LlamaConfig.from_dict(raw)
    assert cfg.eos_token_ids == (2, 7) and cfg.num_key_value_heads == 4


@pytest.mark.parametrize("change,word", [
    ({"model_type": "mistral"}, "llama"), ({"rope_scaling": {"type": "linear", "factor": 2}}, "rope_scaling"),
    ({"attention_bias": True}, "bias"), ({"mlp_bias": True}, "bias"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"), ({"vocab_size": 0}, "positive"),
])
def test_unsupported_options_are_refused_by_name(change, word):
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_dict(dict(tm.TINY_A, **change))


def test_missing_keys_are_listed():
    raw = dict(tm.TINY_A)
    del raw["vocab_size"], raw["intermediate_size"]
    with pytest.raises(ConfigError, match="vocab_size, intermediate_size"):
        LlamaConfig.from_dict(raw)


def test_registry_picks_by_architecture_name_then_model_type():
    assert architecture_for(tm.TINY_A).config_class is LlamaConfig
    assert architecture_for({"model_type": "llama"}).config_class is LlamaConfig
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        architecture_for({"architectures": ["NoSuchModel"], "model_type": "other"})
    with pytest.raises(ValueError, match="already registered"):
        register_architecture("LlamaForCausalLM", LlamaConfig)
    assert "LlamaForCausalLM" in ARCHITECTURES


def test_presets_are_the_measured_shapes():
    assert {"tiny-a", "tiny-b", "smollm2-135m", "smollm2-1.7b", "llama-3.1-8b"} <= set(preset_names())
    c = preset("smollm2-135m")
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (30, 576, 9, 3, 64)
    assert (c.intermediate_size, c.vocab_size, c.rope_theta, c.tie_word_embeddings) == (1536, 49152, 100000.0, True)
    assert json.dumps(preset_dict("llama-3.1-8b"))
    with pytest.raises(ConfigError, match="unknown preset"):
        preset("nope")


def test_spec_lists_layers_parts_and_run_order():
    spec = LlamaConfig.from_dict(tm.TINY_B).to_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.run] == [0, 1, 2]
    layer = spec.layers[1]
    assert layer.prefix == "model.layers.1." and layer.mixer.kind == "gqa_attention" and layer.feed_forward.kind == "swiglu"
    assert layer.mixer["position"].kind == "rotary_half" and layer.mixer["position"]["theta"] == 500000.0
    assert layer.mixer_norm["eps"] == 1e-6 and spec.head["tied_to"] is None
    assert LlamaConfig.from_dict(tm.TINY_A).to_spec().head["tied_to"] == "model.embed_tokens.weight"


def test_run_list_is_validated():
    spec = LlamaConfig.from_dict(tm.TINY_A).to_spec()

    def with_run(run):
        return ModelSpec(**{**spec.__dict__, "run": tuple(run)})

    with_run([RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(1, cache_of=1)]).validate()   # a layer twice, a shared cache
    with pytest.raises(ValueError, match="does not exist"):
        with_run([RunEntry(5)]).validate()
    with pytest.raises(ValueError, match="must run earlier"):
        with_run([RunEntry(0, cache_of=1), RunEntry(1)]).validate()
    with pytest.raises(ValueError, match="owns none"):
        with_run([RunEntry(0), RunEntry(1, cache_of=0), RunEntry(1, cache_of=1)]).validate()
