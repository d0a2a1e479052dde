"""Weights by tensor name, checked against what the model expects before anything is copied.

The reference looks each tensor up by its exact name with an expected dtype and shape and stops
at the first problem ("missing checkpoint tensor", "mismatched dtype/shape",
csrc/model/checkpoint.cpp:142-158).  Here the model first hands over its whole list of expected
tensors; :meth:`WeightStore.check` compares it with the checkpoint and raises ONE error that
lists every missing tensor, every unexpected tensor and every wrong shape or kind of dtype (an integer
tensor where a floating one is expected, or the other way round).

Precision rule: on a bfloat16 engine floating tensors are kept in bfloat16, except that a tensor
marked ``keep_stored_precision`` that the file stores in 32 bits stays in 32 bits; integer tables
become int32.  On a float32 engine every floating tensor is float32.
"""
from __future__ import annotations

from typing import Iterable, Sequence

import torch

from ..parts.spec import TensorSpec
from .safetensors_io import Checkpoint, WeightError


class WeightStore:
    def __init__(self, model_dir: str, dtype: torch.dtype, device: torch.device | str) -> None:
        if dtype not in (torch.bfloat16, torch.float32):
            raise WeightError(f"engine dtype must be bfloat16 or float32, got {dtype}")
        self.model_dir = model_dir
        self.dtype = dtype
        self.device = torch.device(device)
        self.checkpoint = Checkpoint(model_dir)
        self._expected: dict[str, TensorSpec] = {}

    # ---- validation ------------------------------------------------------------------
    def check(self, manifest: Iterable[TensorSpec]) -> None:
        expected: dict[str, TensorSpec] = {}
        for spec in manifest:
            expected[spec.name] = spec
        missing = [name for name in expected if name not in self.checkpoint]
        unexpected = [name for name in self.checkpoint.names() if name not in expected]
        wrong = []
        for name, spec in expected.items():
            if name in self.checkpoint:
                got = self.checkpoint.entry(name).shape
                if tuple(got) != tuple(spec.shape):
                    wrong.append(f"{name}: expected {list(spec.shape)}, got {list(got)}")
                elif self.checkpoint.entry(name).dtype.is_floating_point == spec.integer:
                    wrong.append(f"{name}: expected {'an integer' if spec.integer else 'a floating'} dtype, "
                                 f"got {self.checkpoint.entry(name).dtype}")
        if missing or unexpected or wrong:
            lines = [f"failed to load checkpoint {self.model_dir}: the tensors do not fit the model"]
            if missing:
                lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
            if unexpected:
                lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
            if wrong:
                lines.append(f"  wrong shape or dtype ({len(wrong)}): " + "; ".join(sorted(wrong)))
            raise WeightError("\n".join(lines))
        self._expected = expected

    # ---- access ----------------------------------------------------------------------
    def _target_dtype(self, stored: torch.dtype, keep_stored_precision: bool) -> torch.dtype:
        if not stored.is_floating_point:
            return torch.int32
        if self.dtype == torch.float32:
            return torch.float32
        if keep_stored_precision and stored == torch.float32:
            return torch.float32
        return torch.bfloat16

    def get(self, spec: TensorSpec) -> torch.Tensor:
        """The tensor on the engine's device, in the dtype the precision rule gives."""
        if spec.name not in self.checkpoint:
            raise WeightError(f"missing checkpoint tensor '{spec.name}' in {self.model_dir}")
        entry = self.checkpoint.entry(spec.name)
        if tuple(entry.shape) != tuple(spec.shape):
            raise WeightError(
                f"mismatched shape for '{spec.name}': expected {list(spec.shape)}, got {list(entry.shape)}"
            )
        host = self.checkpoint.tensor(spec.name)
        target = self._target_dtype(entry.dtype, spec.keep_stored_precision)
        return host.to(device=self.device, dtype=target).contiguous()

    def get_stacked(self, specs: Sequence[TensorSpec]) -> torch.Tensor:
        """Several matrices stacked along their first axis into one, the way the reference fuses
        q/k/v and gate/up projections (csrc/model/layers/linear.cpp:35-52)."""
        parts = [self.get(s) for s in specs]
        dtypes = {p.dtype for p in parts}
        if len(dtypes) != 1:
            raise WeightError(f"cannot stack tensors of different dtypes: {[s.name for s in specs]}")
        return torch.cat(parts, dim=0).contiguous()

    def close(self) -> None:
        self.checkpoint.close()
