"""Architectures: name in config.json -> typed config -> model built from parts."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from ..registry import ARCHITECTURES
from .decoder import DecoderModel


@dataclass(frozen=True)
class Architecture:
    """A registry entry: the typed config class (with `from_dict`, `to_dict`, `model_spec`) and the
    callable that turns a config into a model."""
    config_cls: Any
    build: Callable[..., Any]


def _build_from_spec(config, perturb_init: bool = False):
    return DecoderModel(config.model_spec(), perturb_init=perturb_init)


def register_architecture(name: str, config_cls, build=_build_from_spec, replace: bool = False) -> None:
    ARCHITECTURES.register(name, replace=replace)(Architecture(config_cls, build))


def build_model(config, perturb_init: bool = False):
    """Model (no weights yet) for a typed config; the class is chosen by the config's architecture."""
    return ARCHITECTURES.get(config.architectures[0]).build(config, perturb_init=perturb_init)


from ..config.falcon_h1 import ARCHITECTURE as _FALCON_H1, FalconH1Config  # noqa: E402

register_architecture(_FALCON_H1, FalconH1Config)

__all__ = ["Architecture", "DecoderModel", "build_model", "register_architecture"]
