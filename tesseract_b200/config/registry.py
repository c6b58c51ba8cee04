"""The one registry from an architecture's name to its model.

``config.json``'s ``architectures[0]`` selects the entry, as the reference's loader does
(src/model/mod.rs:91-111); a missing name and an unknown name are two distinct errors
(src/model/mod.rs:190-202).  An entry knows how to read its typed configuration and how
to turn it into an architecture-neutral :class:`ModelSpec`; everything after that is
shared.
"""

from __future__ import annotations

import importlib
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Mapping, Sequence, Tuple

from .reading import NoArchitectureError, UnsupportedArchitectureError, read_config_json
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    read_config: Callable[[Mapping[str, Any]], Any]
    build_spec: Callable[[Any], ModelSpec]
    ignorable_tensors: Callable[[Any], Iterable[str]] = lambda cfg: ()


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(architecture: Architecture) -> Architecture:
    _ARCHITECTURES[architecture.name] = architecture
    return architecture


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> List[str]:
    return sorted(_ARCHITECTURES)


PLUGIN_VARIABLE = "TESSERACT_PLUGINS"
_plugins_loaded: set = set()


def load_plugins(modules: Sequence[str] = ()) -> None:
    """Import the given modules and those named in ``$TESSERACT_PLUGINS`` (comma-separated), once each.  A plug-in
    is an ordinary Python module that registers parts and architectures when it is imported; this is how a command
    line or a replay program learns of an architecture that is not part of the package."""
    named = [m.strip() for m in os.environ.get(PLUGIN_VARIABLE, "").split(",") if m.strip()]
    for module in list(modules) + named:
        if module not in _plugins_loaded:
            importlib.import_module(module)
            _plugins_loaded.add(module)


def resolve_architecture(config: Mapping[str, Any]) -> Architecture:
    names = config.get("architectures") or []
    if not names:
        raise NoArchitectureError("config.json names no architecture ('architectures' is missing or empty)")
    first = names[0]
    if first not in _ARCHITECTURES:
        load_plugins()
    if first not in _ARCHITECTURES:
        raise UnsupportedArchitectureError(
            f"unsupported architecture {list(names)} (model_type '{config.get('model_type', '')}'); "
            f"registered: {known_architectures()}")
    return _ARCHITECTURES[first]


def load_model_description(model_dir: str) -> Tuple[Architecture, Any, ModelSpec]:
    """``(architecture entry, typed configuration, model spec)`` of a model folder."""
    raw = read_config_json(model_dir)
    architecture = resolve_architecture(raw)
    config = architecture.read_config(raw)
    return architecture, config, architecture.build_spec(config)
