"""The engine loop: scheduler → step function → sampler → scheduler, in one process.

The reference's ``EngineCore::run`` (csrc/engine/engine_core.cpp:87-108) does
``process_inputs → schedule → run_model → finish → update → send`` behind a ZeroMQ socket.  The transport
is not built here; ``add_request`` / ``abort`` / ``step`` are called directly, and ``step`` returns the
reference's per-step outputs (request id, new token ids, finish reason; csrc/engine/protocol.h:51-81).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import torch

from .. import kernels
from ..config import EngineConfig
from ..sampling import Sampler, SamplingParams
from .runner import ModelRunner, StepEntry
from .scheduler import FinishReason, RequestOutput, ScheduledRequest, Scheduler


@dataclass
class _InFlight:
    """A step that has been launched and whose sampled ids are on their way to the host."""
    requests: list                 # the requests whose next token the step samples, in row order
    ids_device: torch.Tensor       # the sampler's output
    host: torch.Tensor             # pinned copy of it
    event: torch.cuda.Event        # recorded after the copy
    all_sampled: bool              # every entry of the step sampled: the step after it is a decode step of the same rows


class EngineCore:
    """``step`` returns the outputs of one model step.  With ``decode_run_ahead`` the GPU does not wait for the host
    in between: while the ids of step N travel to the host, step N+1 is launched with its input ids taken from the
    sampler's output on the device — if nothing is waiting, every request of N is decoding and none of them ends at N
    by its length (an end-of-sequence token cannot be known yet: such a request's row of N+1 is computed and dropped).
    The host's work between two steps (scheduler, packing, sampling options: about 100 us) then overlaps the device's.
    """

    def __init__(self, config: EngineConfig) -> None:
        self.config = config
        self.runner = ModelRunner(config.model_path, config)
        eos = self.runner.spec.eos_token_ids
        self.scheduler = Scheduler(
            self.runner.manager, max_num_seqs=config.max_num_seqs,
            max_num_scheduled_tokens=config.max_num_scheduled_tokens,
            max_model_len=self.runner.max_model_len, eos_token_ids=eos)
        self.sampler = Sampler(config.seed, self.runner.device, config.max_num_seqs)
        self.stats: Dict[str, int] = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "run_ahead_steps": 0}
        self._inflight: Optional[_InFlight] = None
        self._ids_pinned = [torch.empty(max(1, config.max_num_seqs), dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._turn = 0

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
        if self._inflight is None:
            scheduled = self.scheduler.schedule()
            if not scheduled:
                return self.scheduler.update([])
            self._launch(scheduled)
            self.stats["steps"] += 1
            self.stats["preemptions"] = self.scheduler.num_preemptions
            if self._inflight is None:                   # prompt portions only: nothing was sampled
                return self.scheduler.update([])
        current = self._inflight
        self._inflight = self._run_ahead(current) if self.config.decode_run_ahead else None
        current.event.synchronize()
        tokens = current.host[:len(current.requests)].tolist()
        kernels.check_error_flags()
        live = self.scheduler.requests
        sampled = [(req.request_id, tok) for req, tok in zip(current.requests, tokens)
                   if live.get(req.request_id) is req]   # a request that ended or was aborted meanwhile drops its row
        return self.scheduler.update(sampled)

    def run(self, scheduled: Sequence[ScheduledRequest]) -> List[tuple[Hashable, int]]:
        """Launch ``scheduled`` and wait for its sampled ids (no run-ahead)."""
        self._launch(scheduled)
        current, self._inflight = self._inflight, None
        if current is None:
            return []
        current.event.synchronize()
        tokens = current.host[:len(current.requests)].tolist()
        kernels.check_error_flags()
        return [(req.request_id, tok) for req, tok in zip(current.requests, tokens)]

    # ---- launching ---------------------------------------------------------------------------------------
    def _launch(self, scheduled: Sequence[ScheduledRequest]) -> None:
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
            self._inflight = None
            return
        requests = [s.request for s in wanted]
        self._sample(logits, requests, [r.num_output_tokens for r in requests], len(wanted) == len(entries))

    def _sample(self, logits: torch.Tensor, requests: list, output_indices: List[int], all_sampled: bool) -> None:
        ids = self.sampler.sample(logits, [r.params for r in requests], [r.key for r in requests], output_indices)
        self.runner.mark_device_end()
        host = self._ids_pinned[self._turn]
        self._turn ^= 1
        host[:len(requests)].copy_(ids, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self._inflight = _InFlight(requests, ids, host, event, all_sampled)

    def _run_ahead(self, current: _InFlight) -> Optional[_InFlight]:
        """Launch the decode step after ``current`` before ``current``'s ids have been read, if that step is known
        without them.  Returns what is then in flight, or None."""
        sch = self.scheduler
        requests = current.requests
        if not current.all_sampled or sch.waiting or sch.preempted or len(requests) != len(sch.running):
            return None
        for mine, running in zip(requests, sch.running):
            if mine is not running:
                return None
            # the token on its way makes num_output_tokens + 1 outputs and len(token_ids) + 1 tokens
            if mine.num_output_tokens + 1 >= mine.params.max_tokens or len(mine.token_ids) + 1 >= sch.max_model_len:
                return None
        entries = [StepEntry(r.request_id, [0], [0]) for r in requests]       # the ids come from the device
        if not self.runner.can_use_graph(entries):
            return None
        manager = self.runner.manager
        for r in requests:
            if not manager.allocate(r.request_id, 1):
                return None                          # what was reserved stays reserved: the scheduler asks again
        for r in requests:
            r.num_computed_tokens += 1               # as the scheduler would, once the token on its way is appended
        self.stats["decode_tokens"] += len(requests)
        self.stats["steps"] += 1
        self.stats["run_ahead_steps"] += 1
        logits = self.runner.decode_step(entries, trusted=True, token_ids_device=current.ids_device)
        self._sample(logits, requests, [r.num_output_tokens + 1 for r in requests], True)
        return self._inflight
