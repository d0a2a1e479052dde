"""Reading a model folder's ``config.json``, and the helpers an architecture's typed configuration is
written with.

The reference parses the keys into one ``ModelConfig`` for all its architectures
(csrc/model/model_config.cpp:32-86) and wraps every failure as "invalid model config" / "unsupported
model architecture" (csrc/model/model_config.cpp:88-141).  Here every architecture brings a typed
configuration of its own (a frozen dataclass in its file under ``cuinfer_b200/models``); this module
only knows the file, the error class and how one key is read and checked.
"""
from __future__ import annotations

import json
import os
from typing import Any, Mapping


class ConfigError(ValueError):
    """A model or engine configuration that cannot be used; the message says why."""


_MISSING = object()


def take(raw: Mapping[str, Any], key: str, kind, default=_MISSING):
    """Read ``key`` from ``raw`` as ``kind``; a missing required key is a ConfigError."""
    if key not in raw or raw[key] is None:
        if default is _MISSING:
            raise ConfigError(f"invalid model config: required key '{key}' is missing")
        return default
    value = raw[key]
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"invalid model config: '{key}' must be a number, got {value!r}")
        return float(value)
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            raise ConfigError(f"invalid model config: '{key}' must be an integer, got {value!r}")
        return int(value)
    if kind is bool:
        if not isinstance(value, bool):
            raise ConfigError(f"invalid model config: '{key}' must be true or false, got {value!r}")
        return value
    if kind is str:
        if not isinstance(value, str):
            raise ConfigError(f"invalid model config: '{key}' must be a string, got {value!r}")
        return value
    raise AssertionError(kind)


def read_config_json(model_dir: str) -> dict[str, Any]:
    """Parse ``model_dir/config.json``; generation_config.json's eos ids override the model's
    (csrc/model/model_config.cpp:123-138)."""
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as fh:
            raw = json.load(fh)
    except OSError as exc:
        raise ConfigError(f"cannot open {path}: {exc.strerror or exc}") from exc
    except json.JSONDecodeError as exc:
        raise ConfigError(f"invalid model config {path}: {exc}") from exc
    if not isinstance(raw, dict):
        raise ConfigError(f"invalid model config {path}: top level must be an object")
    gen_path = os.path.join(model_dir, "generation_config.json")
    if os.path.exists(gen_path):
        try:
            with open(gen_path, "r", encoding="utf-8") as fh:
                gen = json.load(fh)
        except (OSError, json.JSONDecodeError) as exc:
            raise ConfigError(f"invalid generation config {gen_path}: {exc}") from exc
        if isinstance(gen, dict) and gen.get("eos_token_id") is not None:
            raw["eos_token_id"] = gen["eos_token_id"]
    return raw
