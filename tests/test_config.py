"""Configuration and registry: config.json keys in, typed numbers out, clear refusals."""

from __future__ import annotations

import json

import pytest

import tiny_configs
from llmserve_triton_kernels_b200 import models  # noqa: F401  registers the architecture
from llmserve_triton_kernels_b200.config import (
    ConfigError, LlamaConfig, architecture_of, known_architectures, read_config, register_architecture,
    unregister_architecture,
)
from llmserve_triton_kernels_b200.config.presets import PRESETS


@pytest.mark.parametrize("name", ["a", "b"])
def test_tiny_configs_parse_and_differ_in_every_size(name):
    cfg = LlamaConfig.from_dict(tiny_configs.TINY[name][0])
    d = tiny_configs.TINY[name][0]
    assert cfg.head_dim == d["hidden_size"] // d["num_attention_heads"]
    assert cfg.to_dict()["architectures"] == ["LlamaForCausalLM"]
    assert LlamaConfig.from_dict(cfg.to_dict()) == cfg


def test_the_two_tiny_configs_share_no_size():
    a, b = (LlamaConfig.from_dict(tiny_configs.TINY[n][0]) for n in "ab")
    for field in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "max_position_embeddings", "rope_theta", "rms_norm_eps", "tie_word_embeddings"):
        assert getattr(a, field) != getattr(b, field), field
    assert a.head_dim != b.head_dim
    assert a.num_attention_heads // a.num_key_value_heads != b.num_attention_heads // b.num_key_value_heads


def test_defaults_follow_the_reference():
    d = {"vocab_size": 10, "hidden_size": 16, "intermediate_size": 8, "num_hidden_layers": 1, "num_attention_heads": 2}
    cfg = LlamaConfig.from_dict(d)
    assert (cfg.num_key_value_heads, cfg.max_position_embeddings, cfg.rope_theta, cfg.rms_norm_eps, cfg.tie_word_embeddings) == (
        2, 2048, 10000.0, 1e-5, False)
    assert LlamaConfig.from_dict({**d, "rope_parameters": {"rope_theta": 5e5}}).rope_theta == 5e5


@pytest.mark.parametrize(
    "patch,word",
    [({"rope_scaling": {"rope_type": "llama3", "factor": 8}}, "rope_scaling"), ({"hidden_act": "gelu"}, "hidden_act"),
     ({"attention_bias": True}, "attention_bias"), ({"head_dim": 64}, "head_dim"), ({"num_key_value_heads": 3}, "multiple"),
     ({"hidden_size": 66}, "divisible"), ({"vocab_size": 0}, "positive")],
)
def test_refusals_name_the_key(patch, word):
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_dict({**tiny_configs.TINY_A, **patch})


def test_missing_key_is_named():
    d = dict(tiny_configs.TINY_A)
    del d["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        LlamaConfig.from_dict(d)


def test_registry_chooses_by_architectures_and_lists_known_names(tmp_path):
    assert "LlamaForCausalLM" in known_architectures()
    assert architecture_of(tiny_configs.TINY_A).config_class is LlamaConfig
    with pytest.raises(KeyError, match="LlamaForCausalLM"):
        architecture_of({"architectures": ["MysteryForCausalLM"]})
    with pytest.raises(KeyError, match="architectures"):
        architecture_of({"model_type": "llama"})
    (tmp_path / "config.json").write_text(json.dumps(tiny_configs.TINY_B))
    arch, cfg = read_config(tmp_path)
    assert arch.name == "LlamaForCausalLM" and cfg.num_hidden_layers == 3
    with pytest.raises(FileNotFoundError):
        read_config(tmp_path / "nowhere")


def test_another_architecture_registers_without_touching_the_package():
    class OtherConfig(LlamaConfig):
        architecture = "OtherForCausalLM"

    from llmserve_triton_kernels_b200.models.llama import llama_plan

    register_architecture("OtherForCausalLM", OtherConfig, llama_plan)
    try:
        arch = architecture_of({**tiny_configs.TINY_A, "architectures": ["OtherForCausalLM"]})
        assert arch.config_class is OtherConfig
    finally:
        unregister_architecture("OtherForCausalLM")
    assert "OtherForCausalLM" not in known_architectures()


def test_presets_are_valid_configurations():
    for name, d in PRESETS.items():
        cfg = LlamaConfig.from_dict(d)
        assert cfg.head_dim % 2 == 0, name
    assert LlamaConfig.from_dict(PRESETS["tinyllama-1.1b"]).head_dim == 64


def test_plan_is_data_with_constants_as_parameters():
    from llmserve_triton_kernels_b200.models.llama import llama_plan

    cfg = LlamaConfig.from_dict(tiny_configs.TINY_B)
    plan = llama_plan(cfg)
    assert len(plan.layers) == 3 and [r.layer for r in plan.schedule] == [0, 1, 2]
    mixer = plan.layers[1].mixer
    assert mixer.kind == "attention" and mixer.prefix == "model.layers.1.self_attn."
    assert mixer.params["num_heads"] == 3 and mixer.params["num_kv_heads"] == 1 and mixer.params["head_dim"] == 32
    assert abs(mixer.params["scale"] - 32**-0.5) < 1e-12 and mixer.params["window"] is None
    assert mixer.params["position"].params == {"head_dim": 32, "theta": 500000.0, "max_positions": 256}
    assert plan.layers[2].ff_norm.params == {"size": 96, "eps": 1e-6}
    assert plan.head is None  # tied
