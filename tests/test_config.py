"""Configuration and registry (CPU)."""
import copy
import json

import pytest

from logssms_b200.config import ConfigError, FalconH1Config, load_model_config, make_model_config
from logssms_b200.registry import ARCHITECTURES

from tiny import TINY, TINY_A, TINY_B


def test_every_key_lands_in_the_typed_config():
    cfg = make_model_config(TINY_B)
    assert isinstance(cfg, FalconH1Config)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.vocab_size) == (3, 96, 517)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (3, 1, 32)
    assert (cfg.mamba_n_heads, cfg.mamba_d_head, cfg.mamba_d_state, cfg.mamba_n_groups, cfg.mamba_d_conv) == (6, 24, 32, 2, 3)
    assert cfg.mamba_chunk_size == 16 and cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 1e11
    assert cfg.ssm_multipliers == (0.6, 1.1, 0.9, 1.3, 0.8) and cfg.mlp_multipliers == (0.9, 1.1)
    assert cfg.mamba_rms_norm and cfg.mamba_norm_before_gate and cfg.projectors_bias and not cfg.tie_word_embeddings


@pytest.mark.parametrize("name", sorted(TINY))
def test_round_trip_through_config_json(name, tmp_path):
    cfg = make_model_config(TINY[name])
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    assert load_model_config(str(tmp_path)) == cfg


def test_defaults_follow_the_reference():
    raw = copy.deepcopy(TINY_A)
    del raw["num_key_value_heads"], raw["head_dim"], raw["tie_word_embeddings"], raw["mamba_chunk_size"]
    raw["mamba_d_ssm"] = None
    raw["mamba_expand"] = 1.0
    cfg = make_model_config(raw)
    assert cfg.num_key_value_heads == 4 and cfg.head_dim == 16 and cfg.tie_word_embeddings is False
    assert cfg.mamba_chunk_size == 128 and cfg.mamba_d_ssm == 64
    raw2 = copy.deepcopy(TINY_A)
    del raw2["rope_theta"]
    raw2["rope_parameters"] = {"rope_theta": 5e5, "partial_rotary_factor": 0.5}
    cfg2 = make_model_config(raw2)
    assert cfg2.rope_theta == 5e5 and cfg2.partial_rotary_factor == 0.5
    assert cfg2.model_spec().layers[0].mixers[0].spec.position.rotary_dim == 8


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "rms_norm_eps", "mamba_d_state",
                                 "embedding_multiplier", "ssm_multipliers", "mamba_conv_bias", "vocab_size"])
def test_missing_required_key(key):
    raw = copy.deepcopy(TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        make_model_config(raw)


@pytest.mark.parametrize("patch,match", [
    ({"hidden_act": "gelu"}, "SiLU"), ({"attention_bias": True}, "bias-free"), ({"mlp_bias": True}, "bias-free"),
    ({"attn_layer_indices": [0]}, "parallel"), ({"mamba_d_ssm": 65}, "SSM width"),
    ({"ssm_multipliers": [1.0, 1.0]}, "5 values"), ({"num_key_value_heads": 3}, "multiple"),
    ({"rope_scaling": {"rope_type": "longrope"}}, "rope_scaling"),
])
def test_what_the_engine_refuses(patch, match):
    raw = {**copy.deepcopy(TINY_A), **patch}
    with pytest.raises(ConfigError, match=match):
        make_model_config(raw)


def test_unknown_architecture_and_registry():
    with pytest.raises(ValueError, match="not supported"):
        make_model_config({**TINY_A, "architectures": ["NopeForCausalLM"]})
    with pytest.raises(ConfigError, match="architecture"):
        make_model_config({k: v for k, v in TINY_A.items() if k != "architectures"})
    assert "FalconH1ForCausalLM" in ARCHITECTURES


def test_model_spec_is_layer_by_layer():
    spec = make_model_config(TINY_B).model_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.resolved_schedule()] == [0, 1, 2]
    block = spec.layers[1]
    attn, mamba = block.mixers
    assert block.prefix == "model.layers.1." and attn.spec.kind == "attention" and mamba.spec.kind == "mamba2"
    assert (attn.in_scale, attn.out_scale, mamba.in_scale, mamba.out_scale) == (1.5, 0.8, 1.2, 0.7)
    assert attn.spec.key_scale == 0.5 and mamba.spec.conv_dim == 144 + 2 * 2 * 32
    assert block.feed_forward.activation_scale == 0.9 and block.feed_forward.output_scale == 1.1
    assert spec.embedding_multiplier == 5.0 and spec.lm_head_multiplier == 0.25


def test_import_keeps_cuda_untouched():
    import torch
    import logssms_b200  # noqa: F401
    assert not torch.cuda.is_initialized() or torch.cuda.is_available()
