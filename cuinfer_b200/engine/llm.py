"""The Python entry point: ``LLM(model=...).generate(prompts, sampling_params)`` on token ids.

The reference's front end talks to its engine through ``EngineClient.generate(request_id, token_ids,
{max_output_tokens, temperature, top_k, top_p, ignore_eos})`` (cuinfer/engine.py:171-200;
cuinfer/server.py:165-171) and refuses, before anything reaches the engine, an empty prompt, a prompt of
``max_model_len`` tokens or more, ``prompt + max_tokens > max_model_len`` and token ids outside the
vocabulary (cuinfer/server.py:27-45, :153-160).  The same checks are made here; the engine runs in this
process instead of a child process.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Union

from ..config import EngineConfig
from ..sampling import SamplingParams
from .. import kernels
from .core import EngineCore
from .scheduler import FinishReason


@dataclass
class GenerationResult:
    request_id: str
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: str


class LLM:
    def __init__(self, model: str, **engine_options) -> None:
        """``model``: a folder with config.json and model.safetensors.  ``engine_options`` are the fields of
        :class:`EngineConfig` (gpu_memory_utilization, block_size, max_num_scheduled_tokens, max_num_seqs,
        enable_cuda_graph, decode_run_ahead, dtype, num_blocks, seed, device)."""
        self.config = EngineConfig(model_path=model, **engine_options)
        self.engine = EngineCore(self.config)
        self._counter = 0

    def warm_up(self, batch_sizes: Sequence[int] = (1, 2, 4, 8), longest: int = 2048) -> int:
        """Record the CUDA graphs of decode steps of these batch sizes, for contexts up to ``longest`` tokens, before
        the first request needs them.  Returns how many were recorded."""
        return self.engine.runner.warm_up(batch_sizes, longest)

    def _check(self, prompt: Sequence[int], params: SamplingParams) -> None:
        n = len(prompt)
        limit = self.engine.max_model_len
        if n == 0:
            raise ValueError("prompt must hold at least one token id")
        if n >= limit:
            raise ValueError(f"prompt of {n} tokens must be shorter than max_model_len={limit}")
        if n + params.max_tokens > limit:
            raise ValueError(f"prompt ({n}) + max_tokens ({params.max_tokens}) exceeds max_model_len={limit}")
        for tok in prompt:
            if isinstance(tok, bool) or not isinstance(tok, int) or not 0 <= tok < self.engine.vocab_size:
                raise ValueError(f"token id {tok!r} is not an integer inside the vocabulary of {self.engine.vocab_size}")

    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[GenerationResult]:
        """Generate for every prompt (lists of token ids); results come back in the order of ``prompts``."""
        if isinstance(sampling_params, SamplingParams) or sampling_params is None:
            params = [sampling_params or SamplingParams()] * len(prompts)
        else:
            params = list(sampling_params)
            if len(params) != len(prompts):
                raise ValueError("one SamplingParams per prompt, or one for all")
        for prompt, p in zip(prompts, params):
            self._check(prompt, p)
        results = {}
        order = []
        for prompt, p in zip(prompts, params):
            rid = f"gen-{self._counter}"
            self._counter += 1
            order.append(rid)
            results[rid] = GenerationResult(rid, list(prompt), [], FinishReason.RUNNING.value)
            self.engine.add_request(rid, prompt, p)
        while self.engine.has_requests():
            for out in self.engine.step():
                if out.request_id in results:
                    res = results[out.request_id]
                    res.token_ids.extend(out.new_token_ids)
                    res.finish_reason = out.finish_reason.value
        kernels.check_error_flags(force=True)
        return [results[rid] for rid in order]
