from .base import ConfigError, architecture_of, load_model_config, make_model_config, read_config_json, require
from .specs import (AttentionSpec, BlockSpec, GatedMLPSpec, Mamba2Spec, MixerSlot, ModelSpec, NormSpec,
                    RopeSpec, ScheduleEntry)
from .falcon_h1 import FalconH1Config

__all__ = [
    "ConfigError", "architecture_of", "load_model_config", "make_model_config", "read_config_json", "require",
    "AttentionSpec", "BlockSpec", "GatedMLPSpec", "Mamba2Spec", "MixerSlot", "ModelSpec", "NormSpec",
    "RopeSpec", "ScheduleEntry", "FalconH1Config",
]
