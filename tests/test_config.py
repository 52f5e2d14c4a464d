"""Configuration and registry (no GPU)."""

import json

import pytest

from simple_inference_b200.config import (ConfigError, LlamaConfig, architecture_of,
                                          known_architectures, read_config)
from tests.conftest import TINY_A, TINY_B


def test_reads_every_key_of_both_tiny_configs():
    a = LlamaConfig.from_dict(TINY_A)
    b = LlamaConfig.from_dict(TINY_B)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads,
            a.head_dim, a.intermediate_size, a.vocab_size) == (2, 64, 4, 2, 16, 160, 256)
    assert a.rope_scaling is None and a.tie_word_embeddings and a.rms_norm_eps == 1e-5
    assert a.num_kv_groups == 2 and a.eos_ids() == ()
    assert b.rope_scaling.rope_type == "llama3" and b.rope_scaling.factor == 8.0
    assert b.rope_scaling.original_max_position_embeddings == 64
    assert not b.tie_word_embeddings and b.eos_ids() == (7,) and b.num_kv_groups == 3


def test_head_dim_defaults_to_hidden_over_heads():
    d = dict(TINY_A)
    del d["head_dim"]
    assert LlamaConfig.from_dict(d).head_dim == 64 // 4


def test_missing_keys_are_all_listed():
    d = dict(TINY_A)
    for k in ("hidden_size", "rope_theta", "rms_norm_eps"):
        del d[k]
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(d)
    for k in ("hidden_size", "rope_theta", "rms_norm_eps"):
        assert k in str(e.value)


@pytest.mark.parametrize("patch", [
    {"num_key_value_heads": 3},            # 4 heads do not divide into 3 groups
    {"head_dim": 15},                      # odd head size
    {"rms_norm_eps": 0.0},
    {"vocab_size": -1},
    {"torch_dtype": "float8"},
    {"hidden_act": "gelu"},
    {"attention_bias": True},
    {"rope_scaling": {"rope_type": "llama3", "factor": 8.0}},   # llama3 keys missing
])
def test_bad_values_are_refused(patch):
    with pytest.raises(ConfigError):
        LlamaConfig.from_dict({**TINY_A, **patch})


def test_round_trip_through_json(tmp_path):
    b = LlamaConfig.from_dict(TINY_B)
    (tmp_path / "config.json").write_text(json.dumps(b.to_dict()))
    arch, again = read_config(tmp_path)
    assert arch.name == "LlamaForCausalLM" and again == b


def test_registry_names_the_architecture():
    assert "LlamaForCausalLM" in known_architectures()
    with pytest.raises(ConfigError) as e:
        architecture_of({"architectures": ["MysteryForCausalLM"]})
    assert "LlamaForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        architecture_of({})


def test_plan_carries_only_config_values():
    from simple_inference_b200.models.llama import llama_plan
    for cfg in (TINY_A, TINY_B):
        c = LlamaConfig.from_dict(cfg)
        plan = llama_plan(c)
        assert len(plan.layers) == c.num_hidden_layers and len(plan.run_order) == c.num_hidden_layers
        mixer = plan.layers[0].block.params["mixer"].params
        assert mixer["num_heads"] == c.num_attention_heads and mixer["head_dim"] == c.head_dim
        assert mixer["position"].params["theta"] == c.rope_theta
        assert plan.layers[0].block.params["mixer_norm"].params["eps"] == c.rms_norm_eps
        assert plan.tie_embeddings == c.tie_word_embeddings


def test_float16_checkpoints_are_accepted():
    # reference config.py:137-142 maps bfloat16, float16 and float32
    assert LlamaConfig.from_dict({**TINY_A, "torch_dtype": "float16"}).torch_dtype == "float16"
