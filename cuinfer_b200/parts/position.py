"""Position encodings.

``rope_neox``: rotate-half rotary encoding over the first ``rotary_dim`` elements of a head
(csrc/model/rope_cache.cpp:15-24, :47-58; csrc/ops/qk_norm_rope_fused.cu:114-139): for i < r/2,
``f_i = 1 / theta^(2i / r)``, angle ``p · f_i``, both in 32 bits; pairs are (i, i + r/2).  The table
``[positions, r/2, (cos, sin)]`` is computed once in 32 bits on the host, as the reference does, and
handed to the kernel that applies it.  ``none``: no encoding.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import PositionEncoding
from .registry import POSITION_ENCODINGS
from .spec import PartSpec


_TABLES: dict = {}


@POSITION_ENCODINGS.register("rope_neox")
class RotaryNeox(PositionEncoding):
    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.theta = float(spec.theta)
        self.rotary_dim = int(spec.rotary_dim)
        self.max_positions = int(spec.max_positions)
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rope_neox: rotary_dim must be positive and even, got {self.rotary_dim}")
        self._table: Optional[torch.Tensor] = None
        self._device: Optional[torch.device] = None

    def host_table(self) -> torch.Tensor:
        half = self.rotary_dim // 2
        exponent = torch.arange(0, half, dtype=torch.float32) * 2.0 / float(self.rotary_dim)
        inv_freq = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), exponent)
        pos = torch.arange(self.max_positions, dtype=torch.float32)
        angle = pos[:, None] * inv_freq[None, :]
        return torch.stack((torch.cos(angle), torch.sin(angle)), dim=-1).contiguous()

    def load(self, store) -> None:
        self._device = store.device

    def table(self) -> Optional[torch.Tensor]:
        if self._table is None:
            # layers with the same constants share one table on the device
            device = torch.device(self._device or "cuda")
            key = (self.theta, self.rotary_dim, self.max_positions, str(device))
            if key not in _TABLES:
                _TABLES[key] = self.host_table().to(device)
            self._table = _TABLES[key]
        return self._table


@POSITION_ENCODINGS.register("none")
class NoPosition(PositionEncoding):
    rotary_dim = 0

    def table(self) -> Optional[torch.Tensor]:
        return None
