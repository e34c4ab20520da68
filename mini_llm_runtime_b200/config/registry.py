"""One registry from an architecture's name (config.json ``architectures[0]``) to its typed
configuration and to the function that lays the model out as parts.

The reference project has no registry: it accepts ``model_type == "qwen2"`` only
(src/mini_llm_runtime/qwen_config.py:61-62).  Adding an architecture means one call of
``register_architecture``; nothing else in the package names a model.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping

from .qwen2 import Qwen2Config, qwen2_model_spec
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[Mapping[str, Any]], Any]
    model_spec: Callable[[Any], ModelSpec]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict, model_spec, *, replace: bool = False) -> Architecture:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    entry = Architecture(name, config_from_dict, model_spec)
    _ARCHITECTURES[name] = entry
    return entry


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def architecture_of(data: Mapping[str, Any]) -> Architecture:
    """Pick the registry entry that config.json's ``architectures`` names."""
    names = data.get("architectures")
    if not isinstance(names, (list, tuple)) or not names:
        raise KeyError("config.json lacks the key 'architectures' (a non-empty list); "
                       f"known architectures: {', '.join(known_architectures())}")
    name = names[0]
    if name not in _ARCHITECTURES:
        raise KeyError(f"unknown architecture {name!r}; known architectures: "
                       f"{', '.join(known_architectures())}")
    return _ARCHITECTURES[name]


def config_from_dict(data: Mapping[str, Any]):
    """Typed configuration of whatever architecture ``data`` names."""
    return architecture_of(data).config_from_dict(data)


def load_config(model_dir: str | Path):
    """Read ``<model_dir>/config.json`` (as the reference's load_qwen_config does,
    src/mini_llm_runtime/qwen_loader.py:16-27) and return ``(architecture, typed config)``."""
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json in {str(model_dir)!r}")
    with path.open("r", encoding="utf-8") as handle:
        data = json.load(handle)
    if not isinstance(data, dict):
        raise ValueError(f"{path} must hold a JSON object")
    entry = architecture_of(data)
    return entry, entry.config_from_dict(data)


register_architecture(Qwen2Config.architecture, Qwen2Config.from_dict, qwen2_model_spec)
