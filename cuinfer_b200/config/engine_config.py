"""Runtime knobs of the engine.

Names, defaults and range checks follow the reference's ``Config`` (csrc/engine/config.h:9-28)
and its Python mirror (cuinfer/engine.py:19-34).  Added here: ``dtype`` (the reference is
bfloat16 only), ``num_blocks`` (an explicit page count instead of a share of free memory),
``seed`` (the reference seeds its sampler from the OS, csrc/executor/sampler.cpp:12) and ``decode_run_ahead``
(launch the next decode step before the tokens of the one in flight have been read; see ``engine/core.py``).
"""
from __future__ import annotations

from dataclasses import dataclass

from .model_config import ConfigError


@dataclass(frozen=True)
class EngineConfig:
    model_path: str = ""
    gpu_memory_utilization: float = 0.8
    block_size: int = 16
    max_num_scheduled_tokens: int = 8192
    max_num_seqs: int = 256
    enable_prefix_caching: bool = False
    enable_cuda_graph: bool = True
    decode_run_ahead: bool = True
    dtype: str = "bfloat16"
    num_blocks: int | None = None
    seed: int = 0
    device: str = "cuda:0"

    def __post_init__(self) -> None:
        if not 0 < self.gpu_memory_utilization <= 0.95:
            raise ConfigError("gpu_memory_utilization must be in (0, 0.95]")
        for name in ("block_size", "max_num_scheduled_tokens", "max_num_seqs"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be greater than zero")
        if self.num_blocks is not None and self.num_blocks <= 0:
            raise ConfigError("num_blocks must be greater than zero")
        if self.dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"dtype must be 'bfloat16' or 'float32', got {self.dtype!r}")
        if self.enable_prefix_caching:
            raise ConfigError(
                "enable_prefix_caching is not built in this engine: every prompt is computed from its first token"
            )
