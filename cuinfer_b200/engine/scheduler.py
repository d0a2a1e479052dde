"""Continuous batching above the step function: admit, cut prompts into portions, decode, finish, free.

Policy, as the reference's ``Scheduler`` has it (csrc/scheduler/scheduler.cpp:49-224):

* three queues: waiting (first come first served), running (in admission order), preempted (most
  recently preempted first) (scheduler.h:53-55);
* every step has a budget of ``max_num_scheduled_tokens`` shared by decoded tokens and prompt portions and
  at most ``max_num_seqs`` requests; running requests are served first, each with
  ``min(tokens not yet computed, budget left)`` (:53-61); a prompt that does not fit is cut and continues in
  the next step; only the portion that reaches the end of the prefill wants a sample (:96, :143);
* new requests are admitted after the running ones, preempted ones before waiting ones, and only in a
  step in which nothing was preempted (:110-157);
* when pages run out while a running request is served, the LAST running request is preempted: its pages
  are given back and it will later recompute its prompt plus everything it generated as one prefill; this
  repeats until the request being served fits or is itself the victim (:66-87, :134);
* after sampling: the token is appended; the request stops on an end-of-sequence id unless ``ignore_eos``
  (the id is returned), or on length when it has ``max_tokens`` outputs or ``max_model_len`` tokens
  (:162-184, :211-224).

Decided here, beyond the reference: a request that could never fit — it is alone, holds nothing others could
give back, and the pool is still too small for its next token — finishes with reason ``"capacity"`` instead
of being preempted and recomputed forever; and a prompt that the whole pool cannot hold is refused at
``add_request``.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Deque, Dict, Hashable, List, Optional, Sequence

from ..cache import CacheManager
from ..sampling.params import SamplingParams


class FinishReason(str, Enum):
    RUNNING = "running"
    STOP = "stop"            # an end-of-sequence id was sampled
    LENGTH = "length"        # max_tokens outputs or max_model_len tokens
    CAPACITY = "capacity"    # the cache pool cannot hold the request any further
    ABORT = "abort"


class RequestStatus(str, Enum):
    WAITING = "waiting"
    RUNNING = "running"
    PREEMPTED = "preempted"


@dataclass
class Request:
    request_id: Hashable
    token_ids: List[int]                       # prompt followed by every sampled token
    params: SamplingParams
    key: int = 0                               # stable number of the request, feeds the random stream
    status: RequestStatus = RequestStatus.WAITING
    num_prompt_tokens: int = 0
    num_prefill_tokens: int = 0                # prompt + outputs generated before a preemption
    num_computed_tokens: int = 0
    num_preemptions: int = 0

    @property
    def num_output_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens


@dataclass
class ScheduledRequest:
    request: Request
    is_prefill: bool
    needs_sampling: bool
    position_offset: int
    tokens: List[int]


@dataclass
class RequestOutput:
    request_id: Hashable
    new_token_ids: List[int]
    finish_reason: FinishReason


class Scheduler:
    def __init__(self, manager: CacheManager, *, max_num_seqs: int, max_num_scheduled_tokens: int,
                 max_model_len: int, eos_token_ids: Sequence[int] = ()) -> None:
        self.manager = manager
        self.max_num_seqs = max_num_seqs
        self.max_num_scheduled_tokens = max_num_scheduled_tokens
        self.max_model_len = max_model_len
        self.eos_token_ids = frozenset(eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.preempted: Deque[Request] = deque()
        self.requests: Dict[Hashable, Request] = {}
        self._next_key = 0
        self.pending_outputs: List[RequestOutput] = []   # finishes decided inside schedule()
        self.num_preemptions = 0

    # ---- requests in and out ---------------------------------------------------------------------
    def add_request(self, request_id: Hashable, prompt_token_ids: Sequence[int], params: SamplingParams) -> Request:
        if request_id in self.requests:
            raise ValueError(f"request id {request_id!r} is already in use")
        n = len(prompt_token_ids)
        if n == 0:
            raise ValueError("a prompt needs at least one token")
        if n >= self.max_model_len:
            raise ValueError(f"prompt of {n} tokens leaves no room under max_model_len={self.max_model_len}")
        pool_tokens = min(p.num_pages for p in self.manager.pools) * self.manager.page_size if self.manager.pools else n
        if n > pool_tokens:
            raise ValueError(f"prompt of {n} tokens cannot fit the cache pool of {pool_tokens} tokens")
        req = Request(request_id, list(prompt_token_ids), params, key=self._next_key, num_prompt_tokens=n,
                      num_prefill_tokens=n)
        self._next_key += 1
        self.waiting.append(req)
        self.requests[request_id] = req
        return req

    def abort_requests(self, request_ids: Sequence[Hashable]) -> None:
        for rid in request_ids:
            req = self.requests.get(rid)
            if req is not None:
                self._remove(req)

    def has_requests(self) -> bool:
        return bool(self.requests)

    def _queue_of(self, req: Request):
        return {RequestStatus.WAITING: self.waiting, RequestStatus.RUNNING: self.running,
                RequestStatus.PREEMPTED: self.preempted}[req.status]

    def _remove(self, req: Request) -> None:
        if req.request_id in self.manager:
            self.manager.release(req.request_id)
        self._queue_of(req).remove(req)
        del self.requests[req.request_id]

    # ---- one scheduling decision -------------------------------------------------------------------
    def _preempt(self, victim: Request) -> None:
        self.manager.release(victim.request_id)
        victim.num_computed_tokens = 0
        victim.status = RequestStatus.PREEMPTED
        victim.num_preemptions += 1
        self.num_preemptions += 1
        self.running.remove(victim)
        self.preempted.appendleft(victim)

    def schedule(self) -> List[ScheduledRequest]:
        scheduled: List[ScheduledRequest] = []
        budget = self.max_num_scheduled_tokens
        preempted_now = 0

        # pass 1: running requests, in admission order
        i = 0
        while i < len(self.running) and budget > 0 and len(scheduled) < self.max_num_seqs:
            req = self.running[i]
            n = min(len(req.token_ids) - req.num_computed_tokens, budget)
            assert n > 0
            allocated = False
            while True:
                if self.manager.allocate(req.request_id, n):
                    allocated = True
                    break
                victim = self.running[-1]
                if victim is req and len(self.running) == 1 and not self.preempted:
                    # alone, and still no room: recomputing would meet the same wall
                    self.pending_outputs.append(RequestOutput(req.request_id, [], FinishReason.CAPACITY))
                    self._remove(req)
                    break
                self._preempt(victim)
                preempted_now += 1
                if victim is req:
                    break
            if not allocated:
                break
            budget -= n
            start = req.num_computed_tokens
            scheduled.append(ScheduledRequest(
                request=req, is_prefill=start < req.num_prefill_tokens,
                needs_sampling=start + n >= req.num_prefill_tokens, position_offset=start,
                tokens=req.token_ids[start:start + n]))
            req.num_computed_tokens = start + n
            i += 1

        # pass 2: preempted first, then waiting; not in a step that preempted something
        if preempted_now == 0:
            while (self.preempted or self.waiting) and budget > 0 and len(scheduled) < self.max_num_seqs:
                queue = self.preempted if self.preempted else self.waiting
                req = queue[0]
                total = len(req.token_ids)
                n = min(total, budget)
                if self.manager.admit(req.request_id) is None:
                    break
                if not self.manager.allocate(req.request_id, n):
                    self.manager.release(req.request_id)
                    if not self.running and not scheduled:
                        # nothing is running that could finish and free pages: this request can never start
                        queue.popleft()
                        del self.requests[req.request_id]
                        self.pending_outputs.append(RequestOutput(req.request_id, [], FinishReason.CAPACITY))
                        continue
                    break
                queue.popleft()
                req.num_prefill_tokens = total
                budget -= n
                scheduled.append(ScheduledRequest(
                    request=req, is_prefill=True, needs_sampling=n >= total, position_offset=0,
                    tokens=req.token_ids[:n]))
                req.num_computed_tokens = n
                req.status = RequestStatus.RUNNING
                self.running.append(req)
        return scheduled

    # ---- after sampling ----------------------------------------------------------------------------------
    def finish_reason(self, req: Request, token_id: int) -> FinishReason:
        if not req.params.ignore_eos and token_id in self.eos_token_ids:
            return FinishReason.STOP
        if req.num_output_tokens >= req.params.max_tokens or len(req.token_ids) >= self.max_model_len:
            return FinishReason.LENGTH
        return FinishReason.RUNNING

    def update(self, sampled: Sequence[tuple[Hashable, int]]) -> List[RequestOutput]:
        """Append each sampled token to its request, decide whether it finished, free what finished holds."""
        outputs, self.pending_outputs = self.pending_outputs, []
        for request_id, token_id in sampled:
            req = self.requests[request_id]
            req.token_ids.append(int(token_id))
            reason = self.finish_reason(req, int(token_id))
            outputs.append(RequestOutput(request_id, [int(token_id)], reason))
            if reason != FinishReason.RUNNING:
                self._remove(req)
        return outputs
