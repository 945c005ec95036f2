"""One registry from the architecture name in config.json to its configuration class.

A configuration class has `from_dict(mapping)`, `to_dict()` and `plan()`; the plan
is all the rest of the engine needs.  Adding an architecture is one call of
`register_architecture`; nothing else in the framework names an architecture.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Dict, Mapping

from .qwen3 import ConfigError, Qwen3Config

_ARCHITECTURES: Dict[str, Any] = {}


def register_architecture(name: str, config_cls: Any, *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    for attr in ("from_dict", "plan"):
        if not hasattr(config_cls, attr):
            raise TypeError(f"{config_cls!r} lacks {attr}(), which a configuration class must have")
    _ARCHITECTURES[name] = config_cls


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def config_from_dict(d: Mapping[str, Any]):
    archs = d.get("architectures")
    if not archs:
        raise ConfigError("config.json has no 'architectures' entry; known: "
                          + ", ".join(known_architectures()))
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture {name!r}; known: " + ", ".join(known_architectures()))
    return _ARCHITECTURES[name].from_dict(d)


def load_config(model_dir: str | Path):
    """Read `<model_dir>/config.json` and return the typed configuration it names."""
    path = Path(model_dir)
    if path.is_dir():
        path = path / "config.json"
    if not path.exists():
        raise ConfigError(f"{path} does not exist")
    return config_from_dict(json.loads(path.read_text()))


register_architecture(Qwen3Config.architecture, Qwen3Config)
