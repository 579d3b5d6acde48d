"""Configuration and registry: the reference's acceptance and refusal list
(src/qwen.ts:14-40, test/qwen.test.ts:94-100)."""
import json

import pytest

import helpers
from sprout_lm_b200.config import (ConfigError, LayerCall, ModelSpec, Qwen2Config, architecture_name, load_config,
                                   parse_config, register_architecture)


def good(**changes):
    raw = helpers.raw_config(helpers.TINY_A)
    raw.update(changes)
    return raw


def test_parses_every_key_without_defaults():
    c = parse_config(good())
    assert isinstance(c, Qwen2Config)
    assert (c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (64, 4, 2, 16)
    assert c.eos_token_ids == (255,) and c.tie_word_embeddings is True
    for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                "vocab_size", "max_position_embeddings", "rms_norm_eps", "rope_theta", "tie_word_embeddings",
                "eos_token_id"):
        raw = good()
        del raw[key]
        with pytest.raises(ConfigError):
            parse_config(raw)


def test_round_trip_and_both_tiny_configs_differ_everywhere():
    a = parse_config(helpers.raw_config(helpers.TINY_A))
    b = parse_config(helpers.raw_config(helpers.TINY_B))
    assert parse_config(a.to_dict()) == a and parse_config(b.to_dict()) == b
    for field in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "vocab_size", "rms_norm_eps", "rope_theta", "tie_word_embeddings", "head_dim"):
        assert getattr(a, field) != getattr(b, field), field
    assert b.eos_token_ids == (507, 508)


@pytest.mark.parametrize("changes", [
    {"model_type": "llama"}, {"hidden_act": "gelu"}, {"rope_scaling": {"type": "yarn"}}, {"use_sliding_window": True},
    {"quantization_config": {"bits": 4}}, {"use_mrope": True}, {"num_key_value_heads": 3}, {"rms_norm_eps": 0},
    {"eos_token_id": -1}, {"eos_token_id": []}, {"eos_token_id": 256}, {"hidden_size": 66}, {"head_dim": 32},
    {"vocab_size": 0}, {"rope_theta": float("inf")}, {"tie_word_embeddings": "yes"}, {"num_hidden_layers": 2.5},
    {"hidden_size": 4 * 7},   # head_dim 7 is odd
])
def test_refused_before_any_weight_is_read(changes):
    with pytest.raises(ConfigError):
        parse_config(good(**changes))


def test_falsy_options_are_accepted():
    parse_config(good(use_sliding_window=False, rope_scaling=None, sliding_window=None, head_dim=16,
                      layer_types=["full_attention"] * 2, torch_dtype="bfloat16"))


def test_registry_by_architecture_and_model_type():
    assert architecture_name(good()) == "Qwen2ForCausalLM"
    raw = good(architectures=None)                      # the reference's fixture has null here
    assert architecture_name(raw) == "Qwen2ForCausalLM"
    with pytest.raises(ConfigError, match="Unknown architecture"):
        architecture_name(good(architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="Unknown model_type"):
        architecture_name({"model_type": "mamba"})


def test_model_spec_is_data(tmp_path):
    spec = parse_config(good()).model_spec()
    assert isinstance(spec, ModelSpec) and len(spec.layers) == 2 and spec.cache_slots == 2
    assert [c.layer for c in spec.order] == [0, 1] and all(c.writes_cache for c in spec.order)
    layer = spec.layers[1]
    assert layer.block == "pre_norm" and layer.prefix == "model.layers.1."
    assert layer.mixer.kind == "gqa_attention" and layer.mixer.get("kv_heads") == 2
    assert layer.mixer.get("position").kind == "rope_half_split" and layer.mixer.get("position").get("theta") == 10000.0
    assert layer.feed_forward.kind == "swiglu_mlp" and layer.norms[0].get("eps") == 1e-6
    assert spec.head.get("tied_to") == "model.embed_tokens" and spec.ignorable_tensors == ("lm_head.weight",)
    # the run order may name a layer twice and let a call read another call's cache
    import dataclasses
    twice = dataclasses.replace(spec, order=(LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 0, writes_cache=False)))
    assert twice.cache_slots == 2
    with pytest.raises(ConfigError):
        dataclasses.replace(spec, order=(LayerCall(0, 0, writes_cache=False),))
    with pytest.raises(ConfigError):
        dataclasses.replace(spec, order=(LayerCall(5, 0),))


def test_generation_config_overrides_eos(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(good()))
    assert load_config(tmp_path).eos_token_ids == (255,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [3, 4, 3]}))
    assert load_config(tmp_path).eos_token_ids == (3, 4)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 999}))
    with pytest.raises(ConfigError):
        load_config(tmp_path)


def test_another_architecture_can_be_registered():
    class Other:
        @classmethod
        def from_dict(cls, raw):
            return cls()
    register_architecture("OtherForCausalLM", Other, model_types=("other",))
    assert isinstance(parse_config({"architectures": ["OtherForCausalLM"]}), Other)
    assert isinstance(parse_config({"model_type": "other"}), Other)
