"""Random-weights mode: write a model folder (``config.json`` + ``model.safetensors``) from a configuration
and a seed.  The reference has no such mode (it only loads checkpoints, csrc/model/checkpoint.cpp:39-178);
tests and the benchmark need models without a download.

Which tensors exist, with which shapes, comes from the architecture itself (its parts' ``tensors()``), so
the folder always fits the loader.  Matrices are N(0, std); gains are 1 or 1 + N(0, gain_std).  Every tensor
has a random stream of its own, keyed by (seed, tensor name), so values do not depend on the order of writing.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Mapping, Optional

import torch

from ..config.registry import architecture_of
from .safetensors_io import write_safetensors

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensors(config: Mapping[str, Any], seed: int, *, std: float = 0.02, gain_std: float = 0.0,
                   dtype: str = "float32", gains: Optional[Mapping[str, float]] = None) -> Dict[str, torch.Tensor]:
    """All tensors of the architecture that ``config`` (a config.json dict) names.

    ``gains`` maps a substring of a tensor name to a factor applied after drawing (tests use it to
    sharpen attention scores, e.g. ``{"q_norm": 4.0}``).
    """
    from ..parts.model import DecoderModel

    if dtype not in _TORCH_DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_TORCH_DTYPES)}")
    arch = architecture_of(config)
    typed = arch.parse(config)
    model = DecoderModel(arch.spec(typed), torch.float32)
    out: Dict[str, torch.Tensor] = {}
    for spec in model.tensors():
        gen = torch.Generator().manual_seed(_tensor_seed(seed, spec.name))
        if spec.init == "ones":
            t = torch.ones(spec.shape, dtype=torch.float32)
            if gain_std > 0:
                t += torch.randn(spec.shape, generator=gen, dtype=torch.float32) * gain_std
        else:
            t = torch.randn(spec.shape, generator=gen, dtype=torch.float32) * std
        for pattern, factor in (gains or {}).items():
            if pattern in spec.name:
                t = t * factor
        out[spec.name] = t.to(_TORCH_DTYPES[dtype])
    return out


def write_random_model(model_dir: str, config: Mapping[str, Any], seed: int, *, std: float = 0.02,
                       gain_std: float = 0.0, dtype: str = "float32",
                       gains: Optional[Mapping[str, float]] = None) -> str:
    """Write ``model_dir/config.json`` and ``model_dir/model.safetensors``; return ``model_dir``."""
    os.makedirs(model_dir, exist_ok=True)
    arch = architecture_of(config)
    typed = arch.parse(config)              # validates before anything is written
    cfg = dict(typed.to_dict()) if hasattr(typed, "to_dict") else dict(config)
    cfg["torch_dtype"] = dtype
    tensors = random_tensors(cfg, seed, std=std, gain_std=gain_std, dtype=dtype, gains=gains)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(cfg, fh, indent=1)
    return model_dir
