"""The one registry from an architecture's name (``config.json`` → ``architectures[0]``) to
how that architecture is read and built.

The reference decides this with an ``if`` chain on the name (csrc/model/model_config.cpp:34-46)
and rejects unknown names with "unsupported model architecture" (:112-115).  Here an entry holds
two callables: ``parse(raw_config_dict) -> typed config`` and ``spec(typed config) -> ModelSpec``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from .model_config import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    parse: Callable[[Mapping[str, Any]], Any]
    spec: Callable[[Any], Any]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse, spec, *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, parse, spec)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unsupported model architecture {name!r}; registered: {', '.join(sorted(_ARCHITECTURES))}"
        ) from None


def architecture_of(raw: Mapping[str, Any]) -> Architecture:
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("invalid model config: 'architectures' must be a non-empty list of names")
    return get_architecture(archs[0])


def load_model_config(model_dir: str):
    """Read ``model_dir/config.json`` and return ``(architecture entry, typed config)``."""
    raw = read_config_json(model_dir)
    arch = architecture_of(raw)
    return arch, arch.parse(raw)


def _ensure_builtin() -> None:
    # The built-in architectures register themselves on import.
    import cuinfer_b200.models  # noqa: F401
