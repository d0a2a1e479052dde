"""What one step hands to every part: the batch laid out flat, and where each run's cache lives.

The reference's ``ForwardBatch`` (csrc/executor/forward_batch.h:9-28) carries the same device arrays:
token ids, positions, slot mapping, prefix sums of the portions (``query_start_loc``), sequence
lengths after the step, and the block table.  Added here: a token→request map (so that kernels need
no search), one block table and slot mapping per cache group (groups have pages of their own), the
state slot of every request, and the per-run cache tensors.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch


@dataclass
class GroupView:
    """One cache group's addressing for this step."""

    page_size: int
    block_table: torch.Tensor      # [R, P] int32; -1 where a request holds no page
    slot_mapping: torch.Tensor     # [T] int32: page * page_size + offset of each token; -1 = no write


@dataclass
class PagedKV:
    """The cache of one run of a layer: ``cache[page, 0|1, kv_head, slot, d]`` with its group's addressing.

    ``writes`` is False when the run reads the cache that an earlier run filled.
    """

    cache: torch.Tensor
    group: GroupView
    writes: bool = True


@dataclass
class StepContext:
    num_tokens: int
    num_requests: int
    token_ids: torch.Tensor          # [T] int32
    positions: torch.Tensor          # [T] int32, absolute position of each token in its request
    token_request: torch.Tensor      # [T] int32, index of each token's request in this step
    query_start_loc: torch.Tensor    # [R + 1] int32
    seq_lens: torch.Tensor           # [R] int32, tokens each request holds after this step
    state_slots: torch.Tensor        # [R] int32, the fixed-size state slot of each request
    # Host copies of the small arrays, for parts that decide launches on the host.  They are None while a step is
    # captured into a CUDA graph or replayed (a decode graph keeps ``query_start_loc_host``: one token per row): only a
    # part that declares ``capturable = False`` may read them (the model then runs eagerly).  A capturable part sizes
    # its launches with ``query_lens_for_launch()``.  In a captured step, rows beyond the live requests are padding:
    # state slot -1, empty block table, and in a padded prompt step one of them holds the spare tokens.
    query_start_loc_host: Optional[List[int]] = field(default_factory=list)
    seq_lens_host: Optional[List[int]] = field(default_factory=list)
    state_slots_host: Optional[List[int]] = field(default_factory=list)
    launch_query_lens: Optional[List[int]] = None      # set for a captured step: see query_lens_for_launch
    max_query_len: int = 0
    max_seq_len: int = 0
    groups: Dict[int, GroupView] = field(default_factory=dict)
    kv: Dict[int, PagedKV] = field(default_factory=dict)          # run index -> its paged cache
    state: Dict[int, torch.Tensor] = field(default_factory=dict)  # run index -> [slots, *state shape]
    decode_only: bool = False        # every request brings exactly one token

    def query_lens_for_launch(self) -> List[int]:
        """Tokens per request as host integers, for sizing a launch (how many row tiles an attention kernel needs).
        In an eager step these are the batch's own numbers.  In a captured step they are an upper bound that holds for
        every batch the graph will replay — no request has more tokens, and no split of the step's tokens over its
        requests needs more tiles of 64 rows or more — so a kernel must find its requests' real boundaries in
        ``query_start_loc`` on the device and let CTAs that find none leave."""
        if self.launch_query_lens is not None:
            return self.launch_query_lens
        starts = self.query_start_loc_host
        return [starts[i + 1] - starts[i] for i in range(self.num_requests)]

    def paged_kv(self, run: int) -> PagedKV:
        try:
            return self.kv[run]
        except KeyError:
            raise KeyError(f"run {run} has no paged cache in this step") from None

    def run_state(self, run: int) -> torch.Tensor:
        try:
            return self.state[run]
        except KeyError:
            raise KeyError(f"run {run} has no per-request state") from None
