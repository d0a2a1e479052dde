"""Random-weights mode: write a model folder (``config.json`` + ``model.safetensors``) from a configuration
and a seed.  The reference has no such mode (it only loads checkpoints, csrc/model/checkpoint.cpp:39-178);
tests and the benchmark need models without a download.

Which tensors exist, with which shapes, comes from the architecture itself (its parts' ``tensors()``), so
the folder always fits the loader.  Matrices are N(0, std); gains are 1 or 1 + N(0, gain_std).  Every tensor
has a random stream of its own, keyed by (seed, tensor name), so values do not depend on the order of writing.

Two generators.  ``"torch"`` draws with ``torch.randn`` on the host (fast; what the tests' folders use).
``"counter"`` makes element ``i`` of a tensor a function of (seed, tensor name, i) alone, from integer hashes and
IEEE basic operations only, so that the host (numpy, here) and the device (``csrc/random_init.cu``) compute the very
same bits.  With it a folder need not hold the weights at all: ``write_random_model(..., materialize=False)`` writes
``config.json`` and ``random_weights.json`` (seed, std, ...), and the engine fills its weight tensors on the device
while loading (``DeviceRandomStore``) — 65 GB of a 32B-sized model never cross the host.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Iterable, Mapping, Optional, Sequence

import numpy as np
import torch

from ..config.registry import architecture_of
from ..parts.spec import TensorSpec
from .safetensors_io import WeightError, write_safetensors

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
RANDOM_MARKER = "random_weights.json"
GENERATOR_NAME = "counter-v1"


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def _splitmix64(x: np.ndarray) -> np.ndarray:
    x = x + np.uint64(0x9E3779B97F4A7C15)
    x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return x ^ (x >> np.uint64(31))


def counter_normal(key: int, count: int, mean: float, std: float, factor: float = 1.0, via_bf16: bool = False) -> torch.Tensor:
    """float32 [count]: ``factor * (mean + std * z(key, i))``, the host twin of ``csrc/random_init.cu``: four
    splitmix64 hashes of ``key + 4 i + j`` give twelve 21-bit integers whose sum is approximately normal
    (Irwin-Hall); ``z = (sum - (6 * 2**21 - 6)) / 2**21`` in double, the rest in the same precisions as the kernel."""
    out = np.empty(count, dtype=np.float32)
    mask = np.uint64(0x1FFFFF)
    with np.errstate(over="ignore"):
        for begin in range(0, count, 1 << 22):
            i = np.arange(begin, min(count, begin + (1 << 22)), dtype=np.uint64)
            total = np.zeros(i.shape, dtype=np.uint64)
            for j in range(4):
                h = _splitmix64(np.uint64(key & 0xFFFFFFFFFFFFFFFF) + np.uint64(4) * i + np.uint64(j))
                total += (h & mask) + ((h >> np.uint64(21)) & mask) + ((h >> np.uint64(42)) & mask)
            z = (total.astype(np.int64).astype(np.float64) - 12582906.0) / 2097152.0
            x = (float(mean) + float(std) * z).astype(np.float32) * np.float32(factor)
            out[begin:begin + x.size] = x
    t = torch.from_numpy(out)
    return t.to(torch.bfloat16).float() if via_bf16 else t


def _draw_plan(spec: TensorSpec, std: float, gain_std: float, gains: Optional[Mapping[str, float]]):
    """(mean, std, factor) of a tensor: matrices N(0, std), gains 1 + N(0, gain_std), then the factors of ``gains``."""
    mean, dev = (1.0, gain_std) if spec.init == "ones" else (0.0, std)
    factor = 1.0
    for pattern, f in (gains or {}).items():
        if pattern in spec.name:
            factor *= f
    return mean, dev, factor


def random_tensors(config: Mapping[str, Any], seed: int, *, std: float = 0.02, gain_std: float = 0.0,
                   dtype: str = "float32", gains: Optional[Mapping[str, float]] = None,
                   generator: str = "torch") -> Dict[str, torch.Tensor]:
    """All tensors of the architecture that ``config`` (a config.json dict) names.

    ``gains`` maps a substring of a tensor name to a factor applied after drawing (tests use it to
    sharpen attention scores, e.g. ``{"q_norm": 4.0}``).  ``generator``: ``"torch"`` or ``"counter"``.
    """
    from ..parts.model import DecoderModel

    if dtype not in _TORCH_DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_TORCH_DTYPES)}")
    arch = architecture_of(config)
    typed = arch.parse(config)
    model = DecoderModel(arch.spec(typed), torch.float32)
    if generator not in ("torch", "counter"):
        raise ValueError("generator must be 'torch' or 'counter'")
    out: Dict[str, torch.Tensor] = {}
    for spec in model.tensors():
        if generator == "counter":
            mean, dev, factor = _draw_plan(spec, std, gain_std, gains)
            count = int(np.prod(spec.shape)) if spec.shape else 1
            t = counter_normal(_tensor_seed(seed, spec.name), count, mean, dev, factor, via_bf16=dtype == "bfloat16")
            out[spec.name] = t.reshape(spec.shape).to(_TORCH_DTYPES[dtype])
            continue
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
                       gains: Optional[Mapping[str, float]] = None, generator: str = "torch",
                       materialize: bool = True) -> str:
    """Write ``model_dir/config.json`` and ``model_dir/model.safetensors``; return ``model_dir``.

    ``materialize=False`` (counter generator only) writes ``random_weights.json`` instead of the tensors: the engine
    then draws the same values on the device while it loads."""
    if not materialize and generator != "counter":
        raise ValueError("weights that are drawn on the device need generator='counter'")
    if dtype not in _TORCH_DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_TORCH_DTYPES)}")
    os.makedirs(model_dir, exist_ok=True)
    arch = architecture_of(config)
    typed = arch.parse(config)              # validates before anything is written
    cfg = dict(typed.to_dict()) if hasattr(typed, "to_dict") else dict(config)
    cfg["torch_dtype"] = dtype
    if materialize:
        tensors = random_tensors(cfg, seed, std=std, gain_std=gain_std, dtype=dtype, gains=gains, generator=generator)
        write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                          metadata={"format": "pt", "seed": str(seed)})
    else:
        with open(os.path.join(model_dir, RANDOM_MARKER), "w", encoding="utf-8") as fh:
            json.dump({"generator": GENERATOR_NAME, "seed": int(seed), "std": float(std), "gain_std": float(gain_std),
                       "dtype": dtype, "gains": dict(gains or {})}, fh, indent=1)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(cfg, fh, indent=1)
    return model_dir


class DeviceRandomStore:
    """The weight store of a folder that holds ``random_weights.json`` instead of tensors: same interface as
    ``WeightStore``; every tensor the model asks for is drawn on the device by ``kernels.fill_random``, bit for bit
    what ``random_tensors(..., generator="counter")`` would have written to a file."""

    def __init__(self, model_dir: str, dtype: torch.dtype, device: torch.device | str) -> None:
        if dtype not in (torch.bfloat16, torch.float32):
            raise WeightError(f"engine dtype must be bfloat16 or float32, got {dtype}")
        self.model_dir = model_dir
        self.dtype = dtype
        self.device = torch.device(device)
        path = os.path.join(model_dir, RANDOM_MARKER)
        try:
            with open(path, "r", encoding="utf-8") as fh:
                plan = json.load(fh)
            self.seed, self.std, self.gain_std = int(plan["seed"]), float(plan["std"]), float(plan["gain_std"])
            self.stored = plan["dtype"]
            self.gains = {str(k): float(v) for k, v in dict(plan.get("gains") or {}).items()}
            generator = plan["generator"]
        except (OSError, ValueError, KeyError, TypeError) as exc:
            raise WeightError(f"failed to load checkpoint {model_dir}: invalid {RANDOM_MARKER}: {exc}") from exc
        if generator != GENERATOR_NAME or self.stored not in _TORCH_DTYPES:
            raise WeightError(f"failed to load checkpoint {model_dir}: {RANDOM_MARKER} names generator {generator!r} / "
                              f"dtype {self.stored!r}; this engine draws {GENERATOR_NAME!r} in {sorted(_TORCH_DTYPES)}")
        self._expected: Dict[str, TensorSpec] = {}

    def check(self, manifest: Iterable[TensorSpec]) -> None:
        self._expected = {spec.name: spec for spec in manifest}      # whatever the model expects is what is drawn

    def get(self, spec: TensorSpec) -> torch.Tensor:
        from .. import kernels

        if spec.integer:
            raise WeightError(f"'{spec.name}' is an integer table; random weights are floating tensors only")
        if self.dtype == torch.float32 or (spec.keep_stored_precision and self.stored == "float32"):
            target = torch.float32
        else:
            target = torch.bfloat16
        out = torch.empty(tuple(spec.shape), dtype=target, device=self.device)
        mean, dev, factor = _draw_plan(spec, self.std, self.gain_std, self.gains)
        kernels.fill_random(out, _tensor_seed(self.seed, spec.name), mean, dev, factor, via_bf16=self.stored == "bfloat16")
        return out

    def get_stacked(self, specs: Sequence[TensorSpec]) -> torch.Tensor:
        rows = sum(s.shape[0] for s in specs)
        first = self.get(specs[0])
        if len(specs) == 1:
            return first
        out = torch.empty((rows, *first.shape[1:]), dtype=first.dtype, device=self.device)
        at = 0
        for i, s in enumerate(specs):
            part = first if i == 0 else self.get(s)
            out[at:at + s.shape[0]].copy_(part)
            at += s.shape[0]
        return out

    def close(self) -> None:
        pass


def open_weight_store(model_dir: str, dtype: torch.dtype, device: torch.device | str):
    """The store for a model folder: tensors from its safetensors files, or, where the folder holds
    ``random_weights.json`` and no tensors, values drawn on the device."""
    from .loader import WeightStore

    has_tensors = any(os.path.exists(os.path.join(model_dir, name)) for name in ("model.safetensors", "model.safetensors.index.json"))
    if not has_tensors and os.path.exists(os.path.join(model_dir, RANDOM_MARKER)):
        return DeviceRandomStore(model_dir, dtype, device)
    return WeightStore(model_dir, dtype, device)
