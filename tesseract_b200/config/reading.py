"""Reading a model folder's ``config.json``: the errors every architecture's reader raises and the helpers
they share.  The typed configuration of an architecture lives beside its model (``models/``); nothing in this
package names one.

No size or constant that ``config.json`` gives is repeated anywhere else in the package: every part receives
its numbers from the typed configuration through the model description.
"""

from __future__ import annotations

import json
import os
from typing import Any, Mapping


class ConfigError(ValueError):
    """A ``config.json`` that is missing a key, has a wrong type or breaks an invariant."""


class NoArchitectureError(ConfigError):
    """``config.json`` names no architecture (src/model/mod.rs:190-202)."""


class UnsupportedArchitectureError(ConfigError):
    """``config.json`` names an architecture that no model is registered for."""


def require(data: Mapping[str, Any], key: str, kinds, what: str = "config.json"):
    """``data[key]``, which must be present, not null and of one of ``kinds`` (a bool never passes for a number)."""
    if key not in data or data[key] is None:
        raise ConfigError(f"{what}: missing required key '{key}'")
    value = data[key]
    if isinstance(value, bool) and bool not in (kinds if isinstance(kinds, tuple) else (kinds,)):
        raise ConfigError(f"{what}: key '{key}' must be {kinds}, got bool")
    if not isinstance(value, kinds):
        raise ConfigError(f"{what}: key '{key}' has type {type(value).__name__}, expected {kinds}")
    return value


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as handle:
            data = json.load(handle)
    except FileNotFoundError as exc:
        raise ConfigError(f"{path}: no such file") from exc
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: invalid JSON: {exc}") from exc
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return data
