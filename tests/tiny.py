"""Two tiny Falcon-H1 configurations that differ in every size and option, and helpers that
write a random model folder for them and ask the plain implementation for its logits."""
from __future__ import annotations

import copy
import os

import torch

from logssms_b200.config import make_model_config
from logssms_b200.weights import read_checkpoint, write_random_model

from plain.falcon_h1_plain import falcon_h1_logits

TINY_A = {
    "architectures": ["FalconH1ForCausalLM"], "model_type": "falcon_h1",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rms_norm_eps": 1e-5,
    "max_position_embeddings": 2048, "rope_theta": 1e4, "tie_word_embeddings": True,
    "mamba_d_ssm": 64, "mamba_n_heads": 4, "mamba_d_head": 16, "mamba_d_state": 16, "mamba_n_groups": 1,
    "mamba_d_conv": 4, "mamba_chunk_size": 8, "mamba_conv_bias": False, "mamba_proj_bias": False,
    "projectors_bias": False, "mamba_rms_norm": False, "mamba_norm_before_gate": False,
    "embedding_multiplier": 1.0, "lm_head_multiplier": 1.0, "attention_in_multiplier": 1.0,
    "attention_out_multiplier": 1.0, "key_multiplier": 1.0, "ssm_in_multiplier": 1.0, "ssm_out_multiplier": 1.0,
    "ssm_multipliers": [1.0, 1.0, 1.0, 1.0, 1.0], "mlp_multipliers": [1.0, 1.0],
    "hidden_act": "silu", "attention_bias": False, "mlp_bias": False,
}

TINY_B = {
    "architectures": ["FalconH1ForCausalLM"], "model_type": "falcon_h1",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 200, "vocab_size": 517, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 4096, "rope_theta": 1e11, "tie_word_embeddings": False,
    "mamba_d_ssm": 144, "mamba_n_heads": 6, "mamba_d_head": 24, "mamba_d_state": 32, "mamba_n_groups": 2,
    "mamba_d_conv": 3, "mamba_chunk_size": 16, "mamba_conv_bias": True, "mamba_proj_bias": True,
    "projectors_bias": True, "mamba_rms_norm": True, "mamba_norm_before_gate": True,
    "embedding_multiplier": 5.0, "lm_head_multiplier": 0.25, "attention_in_multiplier": 1.5,
    "attention_out_multiplier": 0.8, "key_multiplier": 0.5, "ssm_in_multiplier": 1.2, "ssm_out_multiplier": 0.7,
    "ssm_multipliers": [0.6, 1.1, 0.9, 1.3, 0.8], "mlp_multipliers": [0.9, 1.1],
    "hidden_act": "silu", "attention_bias": False, "mlp_bias": False,
}

# a third shape: gated norm applied AFTER the gate, partial rotation, llama3 frequency scaling
TINY_C = {
    **copy.deepcopy(TINY_B),
    "num_hidden_layers": 2, "mamba_norm_before_gate": False, "partial_rotary_factor": 0.5,
    "rope_theta": 1e5,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "num_attention_heads": 4, "num_key_value_heads": 4, "head_dim": 48, "vocab_size": 300,
}

# a fourth one with the head sizes of the released models (attention heads of 64, SSM heads of 64 with 128-token
# chunks): in bfloat16 its prompt portions run on the tcgen05 attention and chunk-scan kernels
TINY_D = {
    **copy.deepcopy(TINY_B),
    "num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
    "intermediate_size": 176, "vocab_size": 389, "rms_norm_eps": 1e-5,
    "mamba_d_ssm": 192, "mamba_n_heads": 3, "mamba_d_head": 64, "mamba_d_state": 64, "mamba_n_groups": 1,
    "mamba_d_conv": 4, "mamba_chunk_size": 128, "mamba_rms_norm": False,
}

# a fifth one with heads of 128 in both mixers (the larger released models), two KV groups of three query heads
TINY_E = {
    **copy.deepcopy(TINY_D),
    "hidden_size": 192, "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 128, "intermediate_size": 208,
    "vocab_size": 301, "mamba_d_ssm": 256, "mamba_n_heads": 2, "mamba_d_head": 128, "mamba_d_state": 128,
    "max_position_embeddings": 8192,
}

# the literal second tiny configuration of the benchmark definition (intermediate 192, vocabulary 512); TINY_B above
# is the same model with sizes that are no multiples of 8 or 16
TINY_B_LITERAL = {**copy.deepcopy(TINY_B), "intermediate_size": 192, "vocab_size": 512}

TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "Bl": TINY_B_LITERAL}


def make_model_dir(path: str, raw: dict, seed: int = 0, dtype=torch.float32, perturb: bool = True) -> str:
    """Write config.json + model.safetensors with seeded random weights into `path`."""
    return write_random_model(make_model_config(raw), str(path), seed=seed, dtype=dtype, perturb=perturb)


def plain_logits(model_dir: str, ids, dtype: str) -> torch.Tensor:
    """Logits of every position of `ids` from the plain implementation.  For the float32 engine the
    oracle computes in float64; for the bfloat16 engine in float32 with the bfloat16 rounding points."""
    import json
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    tensors = read_checkpoint(model_dir)
    if dtype == "float32":
        return falcon_h1_logits(cfg, tensors, ids, compute=torch.float64).float()
    return falcon_h1_logits(cfg, tensors, ids, compute=torch.float32, act=torch.bfloat16).float()


# tolerances, set once: largest error anywhere, relative to the largest reference logit of the comparison
TOL = {"float32": 1e-4, "bfloat16": 2e-2}


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.isfinite(got).all(), "engine produced non-finite logits"
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def random_tiny(seed: int, tensor_core_sizes: bool = False) -> dict:
    """A small configuration with every size and option drawn at random within what config.json allows: head sizes in
    steps of 16, any number of heads and groups, widths and vocabularies that are multiples of nothing in particular.
    `tensor_core_sizes` then redraws the mixers' head sizes, the state size and the chunk length among those that the
    tcgen05 prompt kernels take."""
    import random
    rng = random.Random(seed)
    kv, group = rng.randint(1, 3), rng.randint(1, 5)
    head_dim = rng.choice([16, 32, 48, 64, 80, 96, 112, 128])
    partial = rng.choice([1.0, 1.0, 0.5, 0.75])
    if int(head_dim * partial) % 2:
        partial = 1.0
    scaling = rng.choice([None, None,
                          {"rope_type": "llama3", "factor": rng.choice([2.0, 8.0]), "low_freq_factor": 1.0,
                           "high_freq_factor": 4.0, "original_max_position_embeddings": rng.choice([32, 64, 128])},
                          {"rope_type": "yarn", "factor": rng.choice([2.0, 4.0]),
                           "original_max_position_embeddings": rng.choice([64, 128])}])
    groups = rng.randint(1, 3)
    m_heads = groups * rng.randint(1, 3)
    m_head = rng.choice([8, 16, 24, 32, 40, 64, 128])
    mult = lambda: round(rng.uniform(0.5, 1.5), 3)
    raw = {
        "architectures": ["FalconH1ForCausalLM"], "model_type": "falcon_h1",
        "num_hidden_layers": rng.randint(1, 3), "hidden_size": 2 * rng.randint(24, 90),
        "num_attention_heads": kv * group, "num_key_value_heads": kv, "head_dim": head_dim,
        "intermediate_size": 2 * rng.randint(20, 130), "vocab_size": rng.randint(100, 700),
        "rms_norm_eps": rng.choice([1e-4, 1e-5, 1e-6]), "max_position_embeddings": rng.choice([1024, 2048, 4096]),
        "rope_theta": rng.choice([1e4, 1e5, 1e6, 1e11]), "partial_rotary_factor": partial, "rope_scaling": scaling,
        "tie_word_embeddings": rng.random() < 0.5,
        "mamba_d_ssm": m_heads * m_head, "mamba_n_heads": m_heads, "mamba_d_head": m_head,
        "mamba_d_state": rng.choice([8, 16, 32, 48, 64, 128, 256]), "mamba_n_groups": groups,
        "mamba_d_conv": rng.choice([2, 3, 4]), "mamba_chunk_size": rng.choice([8, 16, 32, 64, 128, 256]),
        "mamba_conv_bias": rng.random() < 0.5, "mamba_proj_bias": rng.random() < 0.5,
        "projectors_bias": rng.random() < 0.5, "mamba_rms_norm": rng.random() < 0.5,
        "mamba_norm_before_gate": rng.random() < 0.5,
        "embedding_multiplier": mult(), "lm_head_multiplier": mult(), "attention_in_multiplier": mult(),
        "attention_out_multiplier": mult(), "key_multiplier": mult(), "ssm_in_multiplier": mult(),
        "ssm_out_multiplier": mult(), "ssm_multipliers": [mult() for _ in range(5)],
        "mlp_multipliers": [mult(), mult()],
        "hidden_act": "silu", "attention_bias": False, "mlp_bias": False,
    }
    if tensor_core_sizes:
        rng = random.Random(1000 + seed)
        raw["head_dim"] = rng.choice([64, 128])
        raw["partial_rotary_factor"] = rng.choice([1.0, 0.5])
        raw["mamba_d_head"] = rng.choice([64, 128])
        raw["mamba_d_ssm"] = raw["mamba_n_heads"] * raw["mamba_d_head"]
        raw["mamba_d_state"] = rng.choice([64, 128, 192, 256])
        raw["mamba_chunk_size"] = rng.choice([128, 256])
        raw["max_position_embeddings"] = 4096
    return raw


# four of them as configurations of the replay tests (heads of 96 / 112 / 128 / 64, groups of 3 / 1 / 5 / 5 query heads,
# SSM heads of 128 / 8 / 16 / 128, state sizes 48 / 256 / 256 / 32, conv kernels of 2 to 4 taps)
TINY.update({f"R{seed}": random_tiny(seed) for seed in (5, 10, 11, 14)})
# and one for the long replays: 9 query heads of 128 on 3 KV heads with half of each head rotated, 4 SSM heads of 128
# with a state of 192, chunks of 256 (run as 128), a conv of 3 taps
TINY["T5"] = random_tiny(5, tensor_core_sizes=True)
