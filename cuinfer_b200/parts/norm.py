"""RMSNorm: ``out = x · rsqrt(mean(x²) + eps) · w`` with the squares, the mean, the rsqrt and the product
in 32 bits and one rounding at the end (csrc/ops/rms_norm.cu:43-71; eps inside the square root, the
weight multiplies directly).  Spec: ``PartSpec("rmsnorm", eps=...)``.
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from .base import Norm, ResidualStream
from .registry import NORMS
from .spec import PartSpec, TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.eps = float(spec.eps)
        self.weight: torch.Tensor | None = None

    def tensors(self) -> List[TensorSpec]:
        return [TensorSpec(f"{self.prefix}.weight", (self.hidden_size,), keep_stored_precision=True, init="ones")]

    def load(self, store) -> None:
        self.weight = store.get(self.tensors()[0])

    def fusable_rms(self):
        return (self.weight, self.eps) if self.weight is not None else None

    def add_norm(self, stream: ResidualStream) -> torch.Tensor:
        out = torch.empty(stream.residual.shape, dtype=self.dtype, device=stream.residual.device)
        kernels.add_rmsnorm(stream.residual, stream.pending, self.weight, self.eps, out)
        stream.pending = None
        return out

    def norm_rows(self, rows: torch.Tensor) -> torch.Tensor:
        out = torch.empty(rows.shape, dtype=self.dtype, device=rows.device)
        kernels.add_rmsnorm(rows, None, self.weight, self.eps, out)
        return out
