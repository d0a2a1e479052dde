"""Qwen3 dense decoder as data: ``Qwen3ForCausalLM`` → a list of identical pre-norm layers.

Every layer (csrc/model/causal_lm.cpp:41-64, :138-188): RMSNorm → grouped-query attention with per-head
q/k RMSNorm (eps = rms_norm_eps, csrc/model/layers/attention.cpp:20) and rotate-half RoPE over the whole
head, scale ``head_dim ** -0.5`` (csrc/ops/paged_attention.cu:163-164), no bias, no window → RMSNorm →
SiLU-gated feed-forward.  The output head is the embedding table when ``tie_word_embeddings`` is set
(csrc/model/causal_lm.cpp:35-38).  Tensor names are the checkpoint's own (csrc/model/causal_lm.cpp:22-53,
csrc/model/layers/attention.cpp:22-40, csrc/model/layers/mlp.cpp:12-17).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ..config.model_config import ConfigError, take
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


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
        hidden = take(raw, "hidden_size", int)
        heads = take(raw, "num_attention_heads", int)
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
            vocab_size=take(raw, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=take(raw, "intermediate_size", int),
            num_hidden_layers=take(raw, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=take(raw, "num_key_value_heads", int),
            head_dim=take(raw, "head_dim", int, hidden // heads),
            rms_norm_eps=take(raw, "rms_norm_eps", float),
            rope_theta=take(raw, "rope_theta", float),
            max_position_embeddings=take(raw, "max_position_embeddings", int),
            tie_word_embeddings=take(raw, "tie_word_embeddings", bool),
            torch_dtype=take(raw, "torch_dtype", str, raw.get("dtype", "bfloat16")),
            eos_token_ids=eos_ids,
            hidden_act=take(raw, "hidden_act", str, "silu"),
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


def qwen3_spec(cfg: Qwen3Config) -> ModelSpec:
    norm = PartSpec("rmsnorm", eps=cfg.rms_norm_eps)
    position = PartSpec("rope_neox", theta=cfg.rope_theta, rotary_dim=cfg.head_dim,
                        max_positions=cfg.max_position_embeddings)
    mixer = PartSpec("attention", name="self_attn", num_heads=cfg.num_attention_heads,
                     num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, qk_norm=True,
                     qk_norm_eps=cfg.rms_norm_eps, scale=None, window=None, position=position)
    ffn = PartSpec("swiglu", name="mlp", intermediate_size=cfg.intermediate_size)
    block = PartSpec("prenorm", norm_names=("input_layernorm", "post_attention_layernorm"))
    layers = tuple(
        LayerSpec(prefix=f"model.layers.{i}", block=block, mixer=mixer, feed_forward=ffn, norm=norm)
        for i in range(cfg.num_hidden_layers)
    )
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        layers=layers,
        final_norm=norm,
        embedding_name="model.embed_tokens.weight",
        final_norm_prefix="model.norm",
        lm_head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        eos_token_ids=tuple(cfg.eos_token_ids),
    )


register_architecture(Qwen3Config.ARCHITECTURE, Qwen3Config.from_dict, qwen3_spec, replace=True)
