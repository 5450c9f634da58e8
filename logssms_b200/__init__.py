"""logssms_b200: a small, whole inference engine for one B200 (sm_100a)."""
from . import registry
from .config import ConfigError, FalconH1Config, load_model_config, make_model_config
from .models import build_model, register_architecture

__version__ = "0.1.0"
__all__ = ["registry", "ConfigError", "FalconH1Config", "load_model_config", "make_model_config",
           "build_model", "register_architecture"]
