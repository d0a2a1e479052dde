"""Typed model configuration read from a model folder's ``config.json``.

The reference parses the same keys into ``ModelConfig`` (csrc/model/model_config.cpp:32-86)
and wraps every failure as "invalid model config" / "unsupported model architecture"
(csrc/model/model_config.cpp:88-141).  Here the configuration is a frozen dataclass; every
size and constant of the network comes from it and nothing in the kernels or parts repeats
one of its values.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Mapping


class ConfigError(ValueError):
    """A model or engine configuration that cannot be used; the message says why."""


_MISSING = object()


def _take(raw: Mapping[str, Any], key: str, kind, default=_MISSING):
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


@dataclass(frozen=True)
class Qwen3Config:
    """The Qwen3 dense decoder's ``config.json`` (keys as in csrc/model/model_config.cpp:32-86).

    ``head_dim`` defaults to ``hidden_size // num_attention_heads`` when the file has none
    (csrc/model/model_config.cpp:71-73).  ``eos_token_id`` may be an int, a list or absent.
    Options that the architecture fixes in code and that this engine does not build
    (sliding window, attention bias, another activation, rope scaling) are refused when a
    file switches them on, instead of being silently ignored.
    """

    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    torch_dtype: str = "bfloat16"
    eos_token_ids: tuple[int, ...] = ()
    hidden_act: str = "silu"

    ARCHITECTURE = "Qwen3ForCausalLM"

    def __post_init__(self) -> None:
        positive = (
            "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
            "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings",
        )
        for name in positive:
            if getattr(self, name) <= 0:
                raise ConfigError(f"invalid model config: '{name}' must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                "invalid model config: num_attention_heads "
                f"({self.num_attention_heads}) must be a multiple of num_key_value_heads "
                f"({self.num_key_value_heads})"
            )
        if self.head_dim % 2 != 0:
            raise ConfigError(f"invalid model config: head_dim ({self.head_dim}) must be even for rotary pairs")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError(f"invalid model config: rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"invalid model config: rope_theta must be positive, got {self.rope_theta}")
        if self.torch_dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"unsupported data type in config: {self.torch_dtype!r} (bfloat16 or float32)")
        if self.hidden_act != "silu":
            raise ConfigError(f"unsupported hidden_act {self.hidden_act!r}: this architecture's feed-forward is SiLU-gated")

    # ---- derived sizes -------------------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def max_model_len(self) -> int:
        return self.max_position_embeddings

    # ---- construction --------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen3Config":
        archs = raw.get("architectures")
        if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
            raise ConfigError("invalid model config: 'architectures' must be a non-empty list of names")
        if raw.get("use_sliding_window", False):
            raise ConfigError("unsupported option: use_sliding_window=true (this architecture attends to all keys)")
        if raw.get("attention_bias", False):
            raise ConfigError("unsupported option: attention_bias=true (projections have no bias)")
        if raw.get("rope_scaling") is not None:
            raise ConfigError("unsupported option: rope_scaling must be absent or null for this architecture")
        hidden = _take(raw, "hidden_size", int)
        heads = _take(raw, "num_attention_heads", int)
        if heads <= 0:
            raise ConfigError(f"invalid model config: 'num_attention_heads' must be positive, got {heads}")
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"invalid model config: 'eos_token_id' must be an int or a list of ints, got {eos!r}")
        return cls(
            architecture=archs[0],
            vocab_size=_take(raw, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=_take(raw, "intermediate_size", int),
            num_hidden_layers=_take(raw, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=_take(raw, "num_key_value_heads", int),
            head_dim=_take(raw, "head_dim", int, hidden // heads),
            rms_norm_eps=_take(raw, "rms_norm_eps", float),
            rope_theta=_take(raw, "rope_theta", float),
            max_position_embeddings=_take(raw, "max_position_embeddings", int),
            tie_word_embeddings=_take(raw, "tie_word_embeddings", bool),
            torch_dtype=_take(raw, "torch_dtype", str, raw.get("dtype", "bfloat16")),
            eos_token_ids=eos_ids,
            hidden_act=_take(raw, "hidden_act", str, "silu"),
        )

    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` content that reads back as this configuration."""
        out: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": self.torch_dtype,
            "hidden_act": self.hidden_act,
            "attention_bias": False,
            "use_sliding_window": False,
            "rope_scaling": None,
        }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return out


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
