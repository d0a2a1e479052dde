"""Causal grouped-query attention over a paged cache.

Steps, as the reference's attention layer runs them (csrc/model/layers/attention.cpp:44-105):
stacked q/k/v projection without bias; per-head RMSNorm of queries and keys with gains shared by
all heads (optional; csrc/ops/qk_norm_rope_fused.cu:88-112); position encoding of queries and keys;
write of keys and values to the request's pages; attention of every query over its request's keys
0..position read back from the pages (csrc/ops/paged_attention.cu:198-276), consecutive query heads
sharing a key/value head; output projection.

Spec: ``PartSpec("attention", num_heads, num_kv_heads, head_dim, qk_norm, qk_norm_eps, scale, window,
position=PartSpec(...))``; ``scale`` None means ``head_dim ** -0.5``; ``window`` None means all keys.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from . import attention_dispatch
from .base import Mixer
from .context import StepContext
from .linear import Linear
from .registry import MIXERS, POSITION_ENCODINGS
from .spec import PagedCacheNeed, PartSpec, TensorSpec


@MIXERS.register("attention")
class PagedAttention(Mixer):
    accepts_lazy_norm = True       # the q/k/v projection can compute the norm of its input itself

    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.num_heads = int(spec.num_heads)
        self.num_kv_heads = int(spec.num_kv_heads)
        self.head_dim = int(spec.head_dim)
        if self.num_heads % self.num_kv_heads:
            raise ValueError("attention: num_heads must be a multiple of num_kv_heads")
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.qk_norm = bool(spec.get("qk_norm", False))
        self.qk_norm_eps = float(spec.get("qk_norm_eps", 1e-6))
        scale = spec.get("scale")
        self.scale = float(scale) if scale is not None else self.head_dim ** -0.5
        window = spec.get("window")
        self.window = int(window) if window else 0
        pos_spec: PartSpec = spec.get("position") or PartSpec("none")
        self.position = POSITION_ENCODINGS.get(pos_spec.kind)(pos_spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        if self.position.rotary_dim > self.head_dim:
            raise ValueError("attention: rotary_dim exceeds head_dim")
        p = prefix
        self.qkv = Linear([f"{p}.q_proj.weight", f"{p}.k_proj.weight", f"{p}.v_proj.weight"],
                          [self.q_size, self.kv_size, self.kv_size], hidden_size, dtype)
        self.o = Linear([f"{p}.o_proj.weight"], [hidden_size], self.q_size, dtype)
        self.q_norm_weight: Optional[torch.Tensor] = None
        self.k_norm_weight: Optional[torch.Tensor] = None

    def _norm_specs(self) -> List[TensorSpec]:
        if not self.qk_norm:
            return []
        return [TensorSpec(f"{self.prefix}.q_norm.weight", (self.head_dim,), keep_stored_precision=True, init="ones"),
                TensorSpec(f"{self.prefix}.k_norm.weight", (self.head_dim,), keep_stored_precision=True, init="ones")]

    def tensors(self) -> List[TensorSpec]:
        return self.qkv.tensors() + self.o.tensors() + self._norm_specs() + self.position.tensors()

    def load(self, store) -> None:
        self.qkv.load(store)
        self.o.load(store)
        if self.qk_norm:
            qs, ks = self._norm_specs()
            self.q_norm_weight = store.get(qs)
            self.k_norm_weight = store.get(ks)
            if self.q_norm_weight.dtype != self.k_norm_weight.dtype:
                self.q_norm_weight = self.q_norm_weight.float()
                self.k_norm_weight = self.k_norm_weight.float()
        self.position.load(store)

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.qkv.weight

    def warm_after(self, weight: Optional[torch.Tensor]) -> None:
        self.o.warm_next = weight

    def cache_need(self) -> Optional[PagedCacheNeed]:
        return PagedCacheNeed(self.num_kv_heads, self.head_dim, self.window or None)

    @property
    def capturable(self) -> bool:
        return self.position.capturable

    def workspace_bytes(self, tokens: int) -> int:
        # q/k/v rows, the attention output, the projection's output
        width = 2 if self.dtype == torch.bfloat16 else 4
        return self.qkv.workspace_bytes(tokens) + tokens * self.q_size * width + self.o.workspace_bytes(tokens)

    def forward(self, x: torch.Tensor, ctx: StepContext, run: int) -> torch.Tensor:
        kv = ctx.paged_kv(run)
        qkv = self.qkv.forward(x)
        kernels.qk_norm_rope_kv_write(
            qkv, ctx.positions, kv.group.slot_mapping if kv.writes else None,
            self.q_norm_weight, self.k_norm_weight, self.qk_norm_eps,
            self.position.table(), self.position.rotary_dim,
            kv.cache if kv.writes else None, self.num_heads, self.num_kv_heads, self.head_dim)
        out = torch.empty((qkv.shape[0], self.q_size), dtype=qkv.dtype, device=qkv.device)
        attention_dispatch.paged_attention(qkv, out, kv, ctx, self.num_heads, self.num_kv_heads, self.head_dim,
                                           self.scale, self.window, warm=self.o.weight)
        return self.o.forward(out)
