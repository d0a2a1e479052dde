"""Dense SiLU-gated feed-forward: ``down( silu(gate(x)) · up(x) )``, no biases.

The reference stacks gate and up into one ``[2I, H]`` projection, gate first, applies
``g·u / (1 + exp(−g))`` in 32 bits and projects down (csrc/model/layers/mlp.cpp:8-27;
csrc/ops/swiglu.cu:23-32).  Spec: ``PartSpec("swiglu", intermediate_size=I)``.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from .base import FeedForward
from .context import StepContext
from .linear import Linear
from .registry import FEED_FORWARDS
from .spec import PartSpec, TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    accepts_lazy_norm = True       # the gate/up projection can compute the norm of its input itself

    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.intermediate_size = int(spec.intermediate_size)
        p = prefix
        self.gate_up = Linear([f"{p}.gate_proj.weight", f"{p}.up_proj.weight"],
                              [self.intermediate_size, self.intermediate_size], hidden_size, dtype)
        self.down = Linear([f"{p}.down_proj.weight"], [hidden_size], self.intermediate_size, dtype)

    def tensors(self) -> List[TensorSpec]:
        return self.gate_up.tensors() + self.down.tensors()

    def load(self, store) -> None:
        self.gate_up.load(store)
        self.down.load(store)
        self.gate_up.warm_next = self.down.weight

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.gate_up.weight

    def warm_after(self, weight: Optional[torch.Tensor]) -> None:
        self.down.warm_next = weight

    def workspace_bytes(self, tokens: int) -> int:
        return self.gate_up.workspace_bytes(tokens, silu_pair=True) + self.down.workspace_bytes(tokens)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        act = self.gate_up.forward(x, silu_pair=True)       # silu(gate) * up, fused where the kernel allows
        return self.down.forward(act)
