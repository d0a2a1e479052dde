"""Qwen3 dense decoder as data: ``Qwen3ForCausalLM`` → a list of identical pre-norm layers.

Every layer (csrc/model/causal_lm.cpp:41-64, :138-188): RMSNorm → grouped-query attention with per-head
q/k RMSNorm (eps = rms_norm_eps, csrc/model/layers/attention.cpp:20) and rotate-half RoPE over the whole
head, scale ``head_dim ** -0.5`` (csrc/ops/paged_attention.cu:163-164), no bias, no window → RMSNorm →
SiLU-gated feed-forward.  The output head is the embedding table when ``tie_word_embeddings`` is set
(csrc/model/causal_lm.cpp:35-38).  Tensor names are the checkpoint's own (csrc/model/causal_lm.cpp:22-53,
csrc/model/layers/attention.cpp:22-40, csrc/model/layers/mlp.cpp:12-17).
"""
from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


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
    )


register_architecture(Qwen3Config.ARCHITECTURE, Qwen3Config.from_dict, qwen3_spec, replace=True)
