"""The engine loop: scheduler → step function → sampler → scheduler, in one process.

The reference's ``EngineCore::run`` (csrc/engine/engine_core.cpp:87-108) does
``process_inputs → schedule → run_model → finish → update → send`` behind a ZeroMQ socket.  The transport
is not built here; ``add_request`` / ``abort`` / ``step`` are called directly, and ``step`` returns the
reference's per-step outputs (request id, new token ids, finish reason; csrc/engine/protocol.h:51-81).
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence

import torch

from .. import kernels
from ..config import EngineConfig
from ..sampling import Sampler, SamplingParams
from .runner import ModelRunner, StepEntry
from .scheduler import FinishReason, RequestOutput, ScheduledRequest, Scheduler


class EngineCore:
    def __init__(self, config: EngineConfig) -> None:
        self.config = config
        self.runner = ModelRunner(config.model_path, config)
        eos = getattr(self.runner.model_config, "eos_token_ids", ())
        self.scheduler = Scheduler(
            self.runner.manager, max_num_seqs=config.max_num_seqs,
            max_num_scheduled_tokens=config.max_num_scheduled_tokens,
            max_model_len=self.runner.max_model_len, eos_token_ids=eos)
        self.sampler = Sampler(config.seed, self.runner.device, config.max_num_seqs)
        self.stats: Dict[str, int] = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0}

    @property
    def vocab_size(self) -> int:
        return self.runner.vocab_size

    @property
    def max_model_len(self) -> int:
        return self.runner.max_model_len

    def add_request(self, request_id: Hashable, prompt_token_ids: Sequence[int],
                    params: Optional[SamplingParams] = None) -> None:
        params = params or SamplingParams()
        for tok in prompt_token_ids:
            if not 0 <= int(tok) < self.vocab_size:
                raise ValueError(f"token id {tok} is outside the vocabulary of {self.vocab_size}")
        self.scheduler.add_request(request_id, [int(t) for t in prompt_token_ids], params)

    def abort(self, request_ids: Sequence[Hashable]) -> None:
        self.scheduler.abort_requests(request_ids)

    def has_requests(self) -> bool:
        return self.scheduler.has_requests()

    def step(self) -> List[RequestOutput]:
        """One scheduling decision, one model step, one sample per request that reached its last token."""
        scheduled = self.scheduler.schedule()
        if not scheduled:
            return self.scheduler.update([])
        sampled = self.run(scheduled)
        self.stats["steps"] += 1
        self.stats["preemptions"] = self.scheduler.num_preemptions
        return self.scheduler.update(sampled)

    def run(self, scheduled: Sequence[ScheduledRequest]) -> List[tuple[Hashable, int]]:
        entries = [StepEntry(s.request.request_id, s.tokens, [len(s.tokens) - 1] if s.needs_sampling else [])
                   for s in scheduled]
        for s in scheduled:
            self.stats["prefill_tokens" if s.is_prefill else "decode_tokens"] += len(s.tokens)
        wanted = [s for s in scheduled if s.needs_sampling]
        if len(wanted) == len(entries) and self.runner.can_use_graph(entries):
            logits = self.runner.decode_step(entries, trusted=True)
        else:
            logits = self.runner.step(entries)
        if not wanted:
            self.runner.mark_device_end()
            return []
        ids = self.sampler.sample(
            logits, [s.request.params for s in wanted], [s.request.key for s in wanted],
            [s.request.num_output_tokens for s in wanted])
        self.runner.mark_device_end()
        host = ids.cpu().tolist()
        kernels.check_error_flags()
        return [(s.request.request_id, tok) for s, tok in zip(wanted, host)]
