"""cuinfer_b200: a small, whole inference engine for the Qwen3 dense decoder on one B200 (sm_100a).

``LLM`` and ``SamplingParams`` are the Python entry point; ``python -m cuinfer_b200 generate`` is the command
line; ``bin/trace_run`` replays given token ids.  Heavy modules are imported on first use.
"""
from .config import ConfigError, EngineConfig
from .sampling.params import SamplingParams

__all__ = ["ConfigError", "EngineConfig", "LLM", "SamplingParams"]


def __getattr__(name):
    if name == "LLM":
        from .engine.llm import LLM
        return LLM
    raise AttributeError(name)
