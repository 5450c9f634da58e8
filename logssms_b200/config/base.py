"""Reading config.json and picking the architecture's typed config."""
from __future__ import annotations

import json
import os
from typing import Any, Mapping

from ..registry import ARCHITECTURES


class ConfigError(ValueError):
    """config.json is missing a key, or holds a value the engine refuses."""


_MISSING = object()


def require(raw: Mapping[str, Any], key: str, typ=None):
    """Fetch a key that the architecture gives no default for."""
    value = raw.get(key, _MISSING)
    if value is _MISSING or value is None:
        raise ConfigError(f"config.json lacks required key {key!r}")
    if typ is not None:
        try:
            value = typ(value)
        except (TypeError, ValueError):
            raise ConfigError(f"config.json key {key!r} = {value!r} is not a {typ.__name__}") from None
    return value


def read_config_json(model_dir: str) -> dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no config.json in {model_dir}")
    with open(path) as f:
        return json.load(f)


def architecture_of(raw: Mapping[str, Any]) -> str:
    """First entry of `architectures`, as the reference picks it
    (python/logssms/models/register.py:29-38)."""
    archs = raw.get("architectures") or (raw.get("text_config") or {}).get("architectures")
    if not archs:
        raise ConfigError("Model config does not define an architecture")
    return archs[0]


def make_model_config(raw: Mapping[str, Any]):
    """config.json mapping -> the registered architecture's typed config."""
    from .. import models  # noqa: F401  (registers the built-in architectures)
    arch = architecture_of(raw)
    entry = ARCHITECTURES.get(arch)
    return entry.config_cls.from_dict(raw)


def load_model_config(model_dir: str):
    return make_model_config(read_config_json(model_dir))
