"""Typed configuration of the Falcon-H1 parallel-hybrid decoder.

Every field is a config.json key of the architecture; defaults and refusals
follow the reference (python/logssms/models/falcon_h1.py:88-119 for the Falcon-H1
keys, python/logssms/models/config.py:85-126 for the common ones).  One addition:
`mamba_chunk_size` is read (the reference ignores it and scans in chunks of 64,
python/logssms/layers/linear_attention_backend/mamba2.py:56).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Mapping

from .base import ConfigError, require
from .specs import (AttentionSpec, BlockSpec, GatedMLPSpec, Mamba2Spec, MixerSlot, ModelSpec, NormSpec,
                    RopeSpec)

ARCHITECTURE = "FalconH1ForCausalLM"


@dataclass(frozen=True)
class FalconH1Config:
    # common decoder keys
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    max_position_embeddings: int
    rope_theta: float
    rope_scaling: tuple[tuple[str, Any], ...] | None
    partial_rotary_factor: float
    tie_word_embeddings: bool
    # Mamba2 mixer
    mamba_d_ssm: int
    mamba_n_heads: int
    mamba_d_head: int
    mamba_d_state: int
    mamba_n_groups: int
    mamba_d_conv: int
    mamba_chunk_size: int
    mamba_conv_bias: bool
    mamba_proj_bias: bool
    projectors_bias: bool
    mamba_rms_norm: bool
    mamba_norm_before_gate: bool
    # muP constants
    embedding_multiplier: float
    lm_head_multiplier: float
    attention_in_multiplier: float
    attention_out_multiplier: float
    key_multiplier: float
    ssm_in_multiplier: float
    ssm_out_multiplier: float
    ssm_multipliers: tuple[float, float, float, float, float]
    mlp_multipliers: tuple[float, float]
    torch_dtype: str = "bfloat16"
    architectures: tuple[str, ...] = (ARCHITECTURE,)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "FalconH1Config":
        hidden = require(raw, "hidden_size", int)
        heads = require(raw, "num_attention_heads", int)
        head_dim = int(raw.get("head_dim") or hidden // heads)
        rope_scaling = raw.get("rope_scaling") or None
        rope_params = raw.get("rope_parameters") or {}
        rope_theta = (raw.get("rope_theta") or rope_params.get("rope_theta")
                      or (rope_scaling.get("rope_theta") if rope_scaling else None))
        if rope_theta is None:
            raise ConfigError("config.json lacks required key 'rope_theta'")
        partial = float(rope_params.get("partial_rotary_factor", raw.get("partial_rotary_factor", 1.0)))

        n_heads = require(raw, "mamba_n_heads", int)
        d_head = require(raw, "mamba_d_head", int)
        inner = raw.get("mamba_d_ssm") or int(require(raw, "mamba_expand", float) * hidden)
        if inner != n_heads * d_head:
            raise ConfigError("Falcon-H1 SSM width must equal mamba_n_heads * mamba_d_head")
        if raw.get("hidden_act", "silu") != "silu" or raw.get("attention_bias", False) or raw.get("mlp_bias", False):
            raise ConfigError("Falcon-H1 currently requires SiLU and bias-free attention/MLP")
        if raw.get("attn_layer_indices") is not None:
            raise ConfigError("Falcon-H1 currently requires parallel Attention/Mamba2 at every layer")

        ssm_mult = tuple(float(v) for v in require(raw, "ssm_multipliers"))
        mlp_mult = tuple(float(v) for v in require(raw, "mlp_multipliers"))
        if len(ssm_mult) != 5:
            raise ConfigError(f"ssm_multipliers needs 5 values (z, x, B, C, dt), got {len(ssm_mult)}")
        if len(mlp_mult) != 2:
            raise ConfigError(f"mlp_multipliers needs 2 values (gate, output), got {len(mlp_mult)}")
        if rope_scaling is not None:
            rope_type = rope_scaling.get("rope_type", rope_scaling.get("type", "default"))
            if rope_type not in ("default", "llama3", "yarn"):
                raise ConfigError(f"Unsupported rope_scaling = {rope_scaling!r}")
            rope_scaling = tuple(sorted({**rope_scaling, "rope_type": rope_type}.items()))

        cfg = cls(
            num_hidden_layers=require(raw, "num_hidden_layers", int),
            hidden_size=hidden,
            num_attention_heads=heads,
            num_key_value_heads=int(raw.get("num_key_value_heads") or heads),
            head_dim=head_dim,
            intermediate_size=require(raw, "intermediate_size", int),
            vocab_size=require(raw, "vocab_size", int),
            rms_norm_eps=require(raw, "rms_norm_eps", float),
            max_position_embeddings=require(raw, "max_position_embeddings", int),
            rope_theta=float(rope_theta),
            rope_scaling=rope_scaling,
            partial_rotary_factor=partial,
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            mamba_d_ssm=int(inner),
            mamba_n_heads=n_heads,
            mamba_d_head=d_head,
            mamba_d_state=require(raw, "mamba_d_state", int),
            mamba_n_groups=require(raw, "mamba_n_groups", int),
            mamba_d_conv=require(raw, "mamba_d_conv", int),
            mamba_chunk_size=int(raw.get("mamba_chunk_size") or 128),
            mamba_conv_bias=bool(require(raw, "mamba_conv_bias")),
            mamba_proj_bias=bool(require(raw, "mamba_proj_bias")),
            projectors_bias=bool(require(raw, "projectors_bias")),
            mamba_rms_norm=bool(require(raw, "mamba_rms_norm")),
            mamba_norm_before_gate=bool(require(raw, "mamba_norm_before_gate")),
            embedding_multiplier=require(raw, "embedding_multiplier", float),
            lm_head_multiplier=require(raw, "lm_head_multiplier", float),
            attention_in_multiplier=require(raw, "attention_in_multiplier", float),
            attention_out_multiplier=require(raw, "attention_out_multiplier", float),
            key_multiplier=require(raw, "key_multiplier", float),
            ssm_in_multiplier=require(raw, "ssm_in_multiplier", float),
            ssm_out_multiplier=require(raw, "ssm_out_multiplier", float),
            ssm_multipliers=ssm_mult,
            mlp_multipliers=mlp_mult,
            torch_dtype=str(raw.get("torch_dtype") or raw.get("dtype") or "bfloat16"),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        def positive(name):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        for name in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
                     "head_dim", "intermediate_size", "vocab_size", "mamba_n_heads", "mamba_d_head",
                     "mamba_d_state", "mamba_n_groups", "mamba_d_conv", "mamba_chunk_size",
                     "max_position_embeddings"):
            positive(name)
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.mamba_n_heads % self.mamba_n_groups:
            raise ConfigError("mamba_n_heads must be a multiple of mamba_n_groups")
        rotary = int(self.head_dim * self.partial_rotary_factor)
        if rotary <= 0 or rotary % 2 or rotary > self.head_dim:
            raise ConfigError(f"rotary_dim {rotary} must be even and within head_dim {self.head_dim}")
        if self.rms_norm_eps <= 0:
            raise ConfigError("rms_norm_eps must be positive")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict[str, Any]:
        """config.json content that `from_dict` reads back to an equal config."""
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        d["model_type"] = "falcon_h1"
        d["rope_scaling"] = dict(self.rope_scaling) if self.rope_scaling else None
        d["ssm_multipliers"] = list(self.ssm_multipliers)
        d["mlp_multipliers"] = list(self.mlp_multipliers)
        d.update(hidden_act="silu", attention_bias=False, mlp_bias=False)
        return d

    # ------------------------------------------------------------------ as parts
    def model_spec(self) -> ModelSpec:
        eps = self.rms_norm_eps
        rope = RopeSpec(
            head_dim=self.head_dim,
            rotary_dim=int(self.head_dim * self.partial_rotary_factor),
            theta=self.rope_theta,
            max_position=self.max_position_embeddings,
            scaling=self.rope_scaling,
        )
        attention = AttentionSpec(
            hidden_size=self.hidden_size, num_heads=self.num_attention_heads,
            num_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
            position=rope, key_scale=self.key_multiplier,
        )
        mamba = Mamba2Spec(
            hidden_size=self.hidden_size, num_heads=self.mamba_n_heads, head_dim=self.mamba_d_head,
            state_dim=self.mamba_d_state, num_groups=self.mamba_n_groups, conv_kernel=self.mamba_d_conv,
            conv_bias=self.mamba_conv_bias, proj_bias=self.mamba_proj_bias, out_bias=self.projectors_bias,
            gated_norm=self.mamba_rms_norm, norm_before_gate=self.mamba_norm_before_gate, norm_eps=eps,
            multipliers=self.ssm_multipliers, chunk_size=self.mamba_chunk_size,
        )
        mlp = GatedMLPSpec(
            hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
            activation_scale=self.mlp_multipliers[0], output_scale=self.mlp_multipliers[1],
        )
        norm = NormSpec(self.hidden_size, eps)
        layers = tuple(
            BlockSpec(
                prefix=f"model.layers.{i}.",
                mixers=(
                    MixerSlot(attention, "self_attn.", self.attention_in_multiplier, self.attention_out_multiplier),
                    MixerSlot(mamba, "mamba.", self.ssm_in_multiplier, self.ssm_out_multiplier),
                ),
                mixer_norm=norm, mixer_norm_name="input_layernorm.",
                feed_forward=mlp, feed_forward_name="feed_forward.",
                feed_forward_norm=norm, feed_forward_norm_name="pre_ff_layernorm.",
            )
            for i in range(self.num_hidden_layers)
        )
        return ModelSpec(
            vocab_size=self.vocab_size, hidden_size=self.hidden_size,
            embedding_name="model.embed_tokens.", embedding_multiplier=self.embedding_multiplier,
            lm_head_name="lm_head.", lm_head_multiplier=self.lm_head_multiplier,
            tie_word_embeddings=self.tie_word_embeddings,
            final_norm=norm, final_norm_name="model.final_layernorm.",
            layers=layers,
        )
