"""Host side of sampling: one row of options and one uniform number per request, then the sampling kernel.

The reference keeps a Philox seed and a running offset on the host and draws inside its kernel
(csrc/executor/sampler.cpp:10-37).  Here the uniform number of a draw is a pure function of
(seed, request key, index of the output token), computed on the host with a 64-bit mixing function, so a
request's tokens do not depend on what else is in the batch or on how its prompt was cut.
"""
from __future__ import annotations

import struct
from typing import List, Sequence

import torch

from .. import kernels
from .params import SamplingParams

_MASK = (1 << 64) - 1


def _mix(x: int) -> int:
    """splitmix64 finaliser."""
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform(seed: int, request_key: int, output_index: int) -> float:
    """A number in [0, 1) with 24 random bits, fixed by its three arguments."""
    h = _mix(_mix(_mix(seed & _MASK) ^ (request_key & _MASK)) ^ (output_index & _MASK))
    return (h >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, seed: int, device: torch.device, max_rows: int) -> None:
        self.seed = seed
        self.device = device
        # the engine launches a step before it has waited for the one before: the options of a step are packed into a
        # pinned buffer of their own turn, reused only after the copy that read it has run
        self._hosts = [torch.empty((max(1, max_rows), 4), dtype=torch.float32, pin_memory=True) for _ in range(3)]
        self._copied: List[torch.cuda.Event | None] = [None, None, None]
        self._turn = 0
        self._host = self._hosts[0]
        self._dev = torch.empty((max(1, max_rows), 4), dtype=torch.float32, device=device)
        self._ids = torch.empty(max(1, max_rows), dtype=torch.int32, device=device)

    def _next_host(self) -> None:
        self._turn = (self._turn + 1) % len(self._hosts)
        if self._copied[self._turn] is not None:
            self._copied[self._turn].synchronize()
        self._host = self._hosts[self._turn]

    def _upload(self, rows: int) -> None:
        self._dev[:rows].copy_(self._host[:rows], non_blocking=True)
        event = self._copied[self._turn] or torch.cuda.Event()
        event.record()
        self._copied[self._turn] = event

    def pack(self, params: Sequence[SamplingParams], request_keys: Sequence[int], output_indices: Sequence[int]) -> int:
        rows = len(params)
        if rows > self._host.shape[0]:
            raise ValueError(f"{rows} rows exceed the sampler's {self._host.shape[0]}")
        raw = bytearray()
        for p, key, idx in zip(params, request_keys, output_indices):
            seed = p.seed if p.seed is not None else self.seed
            raw += struct.pack("<fiff", float(p.temperature), int(p.top_k), float(p.top_p), uniform(seed, key, idx))
        self._host.view(torch.uint8).reshape(-1)[:len(raw)] = torch.frombuffer(raw, dtype=torch.uint8)
        return rows

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], request_keys: Sequence[int],
               output_indices: Sequence[int]) -> torch.Tensor:
        """Token ids (int32, on the device) drawn from float32 ``logits[rows, vocab]``."""
        rows = len(params)
        if logits.shape[0] != rows:
            raise ValueError(f"{logits.shape[0]} logits rows for {rows} requests")
        out = self._ids[:rows]
        if all(p.greedy for p in params):
            # every row is an argmax: no options, no uniform numbers, and eight CTAs to a row
            kernels.argmax_rows(logits, out)
            return out
        self._next_host()
        self.pack(params, request_keys, output_indices)
        self._upload(rows)
        kernels.sample(logits, self._dev[:rows], out)
        return out
