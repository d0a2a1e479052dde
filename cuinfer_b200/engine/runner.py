"""The step function: run the tokens a batch brings, from the cache, and return logits at the wanted places.

The reference's ``ModelRunner::run_model`` (csrc/executor/model_runner.cpp:60-92) packs the scheduled
requests into flat arrays (csrc/executor/batch_buffer.cpp:57-168: token ids, positions =
``position_offset + j``, slot mapping = ``table[pos / bs] * bs + pos % bs``, ``query_start_loc`` prefix
sums, ``seq_lens = offset + n``, block-table rows, index of each request's last token), copies them to
the device in one transfer from pinned memory, runs the model and samples.  Here the step stops at the
logits (32-bit, any number of wanted positions per entry); sampling is a separate call above it.

A batch is a list of :class:`StepEntry`: a request id, its next tokens (a whole prompt, a portion of
one, or a single decoded token) and the positions among them whose logits are wanted.  Pages for the
new tokens must have been allocated in the cache manager before the step (the scheduler or the replay
tool does that); the step records the stored tokens afterwards.
"""
from __future__ import annotations

import gc
import weakref
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache import CacheManager, CacheStorage, group_runs, page_bytes
from ..config import EngineConfig, load_model_config
from ..parts import DecoderModel, GroupView, PagedKV, StepContext
from ..weights import open_weight_store

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class StepError(RuntimeError):
    """A batch the step function cannot run; the message says which entry and why."""


@dataclass
class StepEntry:
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)   # indices into ``tokens`` whose logits are wanted


class _PinnedRing:
    """A few pinned staging buffers used in turn; a buffer is reused only after its copy has finished."""

    def __init__(self, count: int = 3) -> None:
        self._bufs: List[Optional[torch.Tensor]] = [None] * count
        self._events: List[Optional[torch.cuda.Event]] = [None] * count
        self._next = 0

    def get(self, num_ints: int) -> tuple[torch.Tensor, int]:
        i = self._next
        self._next = (self._next + 1) % len(self._bufs)
        if self._events[i] is not None:
            self._events[i].synchronize()
        buf = self._bufs[i]
        if buf is None or buf.numel() < num_ints:
            size = max(4096, 1 << (num_ints - 1).bit_length())
            buf = torch.empty(size, dtype=torch.int32, pin_memory=True)
            self._bufs[i] = buf
        return buf, i

    def mark(self, i: int) -> None:
        ev = self._events[i]
        if ev is None:
            ev = torch.cuda.Event()
            self._events[i] = ev
        ev.record()


class ModelRunner:
    def __init__(self, model_dir: str, config: EngineConfig, *, num_blocks: Optional[int] = None) -> None:
        if not torch.cuda.is_available():
            raise RuntimeError("cuinfer_b200 runs on a CUDA device only; none is visible")
        self.config = config
        self.device = torch.device(config.device)
        torch.cuda.set_device(self.device)
        self.dtype = _DTYPES[config.dtype]
        self.architecture, self.model_config = load_model_config(model_dir)
        self.spec = self.architecture.spec(self.model_config)
        self.model = DecoderModel(self.spec, self.dtype)
        store = open_weight_store(model_dir, self.dtype, self.device)
        try:
            self.model.load(store)
        finally:
            store.close()
        self.vocab_size = self.spec.vocab_size
        self.max_model_len = self.spec.max_positions
        self.page_size = config.block_size

        needs = self.model.cache_needs()
        self.groups = group_runs(needs)
        pages = num_blocks if num_blocks is not None else config.num_blocks
        if pages is None:
            pages = self._pages_from_memory()
        self.num_pages = int(pages)
        self.manager = CacheManager(self.groups, self.page_size, self.num_pages, config.max_num_seqs)
        self.storage = CacheStorage(self.groups, self.page_size, [self.num_pages] * len(self.groups),
                                    self.model.state_needs(), config.max_num_seqs, self.dtype, self.device)
        # which cache every run uses (its own, or an earlier run's)
        self._run_cache: Dict[int, tuple[int, bool]] = {}
        for run, _layer in self.model.runs():
            src = self.model.cache_source.get(run, run)
            if src in self.storage.run_cache:
                self._run_cache[run] = (src, src == run)
        self._ring = _PinnedRing()
        self._arena: Optional[torch.Tensor] = None
        self._graphs: Dict[tuple, "DecodeGraph"] = {}        # (rows bucket, context class) -> graph
        self._step_graphs: Dict[tuple, "StepGraph"] = {}     # shape of a prompt-sized step -> graph (a few, oldest dropped)
        self._step_seen: Dict[tuple, int] = {}
        self.step_graph_replays = 0
        self.step_graph_captures = 0
        self._graph_pool = None                  # the memory pool all graphs of this runner record into
        self._capture_stream: Optional[torch.cuda.Stream] = None
        self.steps_run = 0
        self.tokens_run = 0
        self.graph_steps = 0
        # when a list: (start, end) CUDA events of every step's device work are appended (the benchmark reads them)
        self.timing: Optional[list] = None
        self._timing_start: Optional[torch.cuda.Event] = None

    # ---- sizing ------------------------------------------------------------------------------------
    def page_bytes(self) -> int:
        return sum(page_bytes(g, self.page_size, self.dtype) for g in self.groups)

    def _pages_from_memory(self) -> int:
        """Pages that fit in ``gpu_memory_utilization`` of the device after the weights
        (csrc/executor/model_runner.cpp:154-163, csrc/engine/engine_core.cpp:111-128)."""
        free, total = torch.cuda.mem_get_info(self.device)
        used = total - free
        budget = int(total * self.config.gpu_memory_utilization) - used
        # room for a step's activations: qkv/gate_up/logits rows of a full token budget
        budget -= self._activation_bytes()
        per_page = max(1, self.page_bytes())
        pages = budget // per_page
        need = (self.max_model_len + self.page_size - 1) // self.page_size
        if pages < need:
            raise RuntimeError(
                f"the cache pool would hold {max(pages, 0)} pages of {self.page_size} tokens, fewer than one request of "
                f"max_model_len={self.max_model_len} needs ({need}); raise gpu_memory_utilization or give num_blocks")
        return int(pages)

    def _activation_bytes(self) -> int:
        """What a step of a full token budget allocates beside weights and cache, and what the captured steps keep
        (each graph has a pool of its own for the intermediates of its sizes); the parts say how much."""
        step = self.model.workspace_bytes(self.config.max_num_scheduled_tokens, self.config.max_num_seqs)
        if not self.config.enable_cuda_graph:
            return step
        captured = min(self.config.max_num_scheduled_tokens, self.STEP_GRAPH_MAX_TOKENS)
        # the step graphs share one pool, which grows to the largest of them; their results (logits) stay allocated
        logits = self.STEP_GRAPH_LIMIT * 64 * self.vocab_size * 4
        return step + self.model.workspace_bytes(captured, self.config.max_num_seqs) + logits

    # ---- requests ------------------------------------------------------------------------------------
    def reserve(self, request_id: Hashable, num_new_tokens: int) -> bool:
        """Admit the request if it is new and allocate pages for ``num_new_tokens`` more tokens.
        False (and nothing changed) when slots or pages are short."""
        fresh = request_id not in self.manager
        if fresh and self.manager.admit(request_id) is None:
            return False
        if not self.manager.allocate(request_id, num_new_tokens):
            if fresh:
                self.manager.release(request_id)
            return False
        return True

    def release(self, request_id: Hashable) -> None:
        if request_id in self.manager:
            self.manager.release(request_id)

    # ---- one step ----------------------------------------------------------------------------------------
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        if len(entries) > self.config.max_num_seqs:
            raise StepError(f"{len(entries)} requests in one step exceed max_num_seqs={self.config.max_num_seqs}")
        seen = set()
        total = 0
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request_id!r} brings no tokens")
            if e.request_id not in self.manager:
                raise StepError(f"request {e.request_id!r} has no pages; reserve() it before the step")
            have = self.manager.num_tokens(e.request_id)
            if have + n > self.max_model_len:
                raise StepError(f"request {e.request_id!r} would reach {have + n} tokens, beyond max_model_len={self.max_model_len}")
            if any(p > 0 for p in self.manager.pages_needed(e.request_id, n)):
                raise StepError(f"request {e.request_id!r} lacks pages for {n} more tokens; reserve() them before the step")
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"request {e.request_id!r}: wanted index {w} is outside its {n} tokens")
            for tok in e.tokens:
                if not 0 <= tok < self.vocab_size:
                    raise StepError(f"request {e.request_id!r}: token id {tok} is outside the vocabulary of {self.vocab_size}")
            total += n
        if total > self.config.max_num_scheduled_tokens:
            raise StepError(f"{total} tokens in one step exceed max_num_scheduled_tokens={self.config.max_num_scheduled_tokens}")

    def _validate_decode(self, entries: Sequence[StepEntry]) -> None:
        """The checks of ``_validate`` for a step in which every request brings one token."""
        if not entries or len(entries) > self.config.max_num_seqs:
            self._validate(entries)
        mgr = self.manager
        seen = set()
        for e in entries:
            rid = e.request_id
            tok = e.tokens[0]
            if (len(e.tokens) != 1 or rid in seen or rid not in mgr or not 0 <= tok < self.vocab_size
                    or mgr.num_tokens(rid) + 1 > self.max_model_len or any(p > 0 for p in mgr.pages_needed(rid, 1))
                    or any(w != 0 for w in e.want)):
                self._validate(entries)          # raises with the full message
                raise StepError(f"request {rid!r} cannot take part in a decode step")
            seen.add(rid)

    def build_context(self, entries: Sequence[StepEntry], table_stride: Optional[int] = None,
                      arena: Optional[torch.Tensor] = None, pad: Optional[Tuple[int, int, int]] = None):
        """Pack the batch, copy it to the device and return ``(StepContext, logits_indices tensor)``.
        ``arena``: the device buffer to copy into (a captured step's own); default: the runner's.
        ``pad = (tokens, requests, wanted rows)``: lay the batch out for that many — the sizes a captured step was
        recorded with.  The tokens beyond the batch's own belong to one more request that holds no pages and writes
        none (positions 0, 1, ...; slot -1; empty block table), further requests bring no tokens, and the wanted rows
        beyond the batch's own point at row 0; the caller drops what comes out of them."""
        mgr = self.manager
        R_live = len(entries)
        lens = [len(e.tokens) for e in entries]
        starts = [mgr.num_tokens(e.request_id) for e in entries]
        T_live = sum(lens)
        S_live = sum(len(e.want) for e in entries)
        T, R, S = pad if pad is not None else (T_live, R_live, S_live)
        if T < T_live or S < S_live or R < R_live + (1 if T > T_live else 0):
            raise StepError(f"a step of {T_live} tokens, {R_live} requests, {S_live} wanted rows does not fit the sizes {pad}")
        G = len(self.groups)
        P = table_stride or max(1, max(len(mgr.block_table(e.request_id, g)) for e in entries for g in range(G))) if G else 1
        total = 3 * T + (R + 1) + 2 * R + S + G * (T + R * P)
        pinned, ring_idx = self._ring.get(total)
        host = pinned.numpy()
        off = 0

        def take(n: int) -> tuple[np.ndarray, int]:
            nonlocal off
            view = host[off:off + n]
            begin = off
            off += n
            return view, begin

        tok, o_tok = take(T)
        pos, o_pos = take(T)
        treq, o_treq = take(T)
        qsl, o_qsl = take(R + 1)
        sl, o_sl = take(R)
        slots, o_slots = take(R)
        want, o_want = take(S)
        qsl[0] = 0
        t0 = 0
        w0 = 0
        if pad is not None:                      # the padding: no token ids but 0, one request for the spare tokens
            tok[T_live:] = 0
            pos[T_live:] = np.arange(T - T_live, dtype=np.int32)
            treq[T_live:] = R_live if R > R_live else 0
            qsl[R_live + 1:] = T
            sl[R_live:] = 0
            if R > R_live:
                sl[R_live] = T - T_live
            slots[R_live:] = -1
            want[S_live:] = 0
        for r, e in enumerate(entries):
            n = lens[r]
            tok[t0:t0 + n] = np.asarray(e.tokens, dtype=np.int32)
            pos[t0:t0 + n] = np.arange(starts[r], starts[r] + n, dtype=np.int32)
            treq[t0:t0 + n] = r
            qsl[r + 1] = t0 + n
            sl[r] = starts[r] + n
            slots[r] = mgr.slot(e.request_id)
            for w in e.want:
                want[w0] = t0 + w
                w0 += 1
            t0 += n
        group_offsets = []
        for g in range(G):
            sm, o_sm = take(T)
            bt, o_bt = take(R * P)
            bt[:] = -1
            sm[T_live:] = -1
            t0 = 0
            for r, e in enumerate(entries):
                table = mgr.block_table(e.request_id, g)
                if len(table) > P:
                    raise StepError(f"request {e.request_id!r} holds {len(table)} pages, more than the table stride {P}")
                row = np.asarray(table, dtype=np.int32)
                bt[r * P:r * P + len(table)] = row
                p = np.arange(starts[r], starts[r] + lens[r], dtype=np.int32)
                pages = row[p // self.page_size]
                if (pages < 0).any():
                    raise StepError(f"request {e.request_id!r}: a new token has no page in group {g}")
                sm[t0:t0 + lens[r]] = pages * self.page_size + p % self.page_size
                t0 += lens[r]
            group_offsets.append((o_sm, o_bt))

        if arena is not None:
            if arena.numel() < total:
                raise StepError(f"the step needs {total} words of metadata, its captured arena holds {arena.numel()}")
            dev = arena[:total]
        else:
            if self._arena is None or self._arena.numel() < total:
                self._arena = torch.empty(max(4096, 1 << (total - 1).bit_length()), dtype=torch.int32, device=self.device)
            dev = self._arena[:total]
        self.mark_device_begin()
        dev.copy_(pinned[:total], non_blocking=True)
        self._ring.mark(ring_idx)

        groups = {}
        for g, (o_sm, o_bt) in enumerate(group_offsets):
            groups[g] = GroupView(self.page_size, dev[o_bt:o_bt + R * P].view(R, P), dev[o_sm:o_sm + T])
        ctx = StepContext(
            num_tokens=T, num_requests=R,
            token_ids=dev[o_tok:o_tok + T], positions=dev[o_pos:o_pos + T], token_request=dev[o_treq:o_treq + T],
            query_start_loc=dev[o_qsl:o_qsl + R + 1], seq_lens=dev[o_sl:o_sl + R], state_slots=dev[o_slots:o_slots + R],
            query_start_loc_host=[int(v) for v in qsl], seq_lens_host=[int(v) for v in sl],
            state_slots_host=[int(v) for v in slots],
            max_query_len=max(max(lens), T - T_live), max_seq_len=max(int(v) for v in sl), groups=groups,
            decode_only=pad is None and all(n == 1 for n in lens),
        )
        for run, (src, writes) in self._run_cache.items():
            ctx.kv[run] = PagedKV(self.storage.run_cache[src], groups[self.storage.run_group[src]], writes)
        ctx.state = self.storage.state
        return ctx, dev[o_want:o_want + S]

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the batch and return float32 logits ``[sum(len(e.want)), vocab]`` in entry order (device tensor)."""
        self._validate(entries)
        self.storage.zero_slots(self.manager.take_newly_admitted())
        graph = self._step_graph(entries)
        if graph is not None:
            logits = graph.run(entries)
        else:
            ctx, want = self.build_context(entries)
            stream = self.model.forward(ctx)
            if want.numel():
                logits = self.model.logits(stream, want)
            else:
                logits = torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        for e in entries:
            self.manager.commit(e.request_id, len(e.tokens))
        self.steps_run += 1
        self.tokens_run += sum(len(e.tokens) for e in entries)
        return logits

    # ---- steps that are not all single tokens, as CUDA graphs ----------------------------------------------------
    # Launching the ~9 kernels of a layer one by one costs the host about as long as they run (each launch is a few
    # microseconds of Python, a kernel of a 2048-token portion 5-50 us; a step of 31 decoded tokens beside 48 prompt
    # tokens took 6.9 ms launch by launch).  Such a step is therefore padded to a bucket of (tokens, requests, wanted
    # rows) and run as a graph captured for the bucket: the first time a bucket comes it runs launch by launch, the
    # second time it is captured, from then on replayed.  The spare tokens belong to a request without pages (see
    # ``build_context``); nothing of them reaches the caller.
    # Above STEP_GRAPH_MAX_TOKENS a step's kernels run longer than the host needs to launch them, and a graph of that
    # size takes tens of milliseconds to capture and hundreds of megabytes to keep: those steps stay eager.
    STEP_GRAPH_MIN_TOKENS = 32
    STEP_GRAPH_MAX_TOKENS = 4096
    STEP_GRAPH_MAX_ENTRIES = 255
    STEP_GRAPH_LIMIT = 32

    @staticmethod
    def step_bucket(lens: Sequence[int], wants: Sequence[int]) -> Tuple[int, int, int]:
        """(tokens, requests, wanted rows) of the captured step that a batch of these query lengths and numbers of
        wanted rows runs in: tokens rounded up in steps of an eighth of their size (at least 16), requests to a power
        of two with room for the request that takes the spare tokens, wanted rows to as many as there are requests
        (a row each is the usual case, and the output head's time hardly depends on them) or the next power of two."""
        T, R, S = sum(lens), len(lens), sum(wants)
        step = max(16, 1 << max(0, (T - 1).bit_length() - 4))        # 2048 -> 128, 2049 -> 256: at most an eighth spare
        Rb = 1 << R.bit_length()
        return -(-T // step) * step, Rb, (max(Rb, 1 << (S - 1).bit_length())) if S else 0

    def _step_graph(self, entries: Sequence[StepEntry]) -> Optional["StepGraph"]:
        if not self.config.enable_cuda_graph or len(entries) > self.STEP_GRAPH_MAX_ENTRIES or not self.model.capturable:
            return None
        lens = tuple(len(e.tokens) for e in entries)
        if sum(lens) < self.STEP_GRAPH_MIN_TOKENS:
            return None
        key = self.step_bucket(lens, [len(e.want) for e in entries])
        if key[0] > self.STEP_GRAPH_MAX_TOKENS:
            return None
        graph = self._step_graphs.get(key)
        if graph is not None:
            graph.uses += 1
            return graph
        if len(self._step_seen) > 4096:
            self._step_seen.clear()
        seen = self._step_seen.get(key, 0) + 1
        self._step_seen[key] = seen
        if seen < 2:
            return None
        if len(self._step_graphs) >= self.STEP_GRAPH_LIMIT:
            # A graph makes room only for a bucket that has come more often than the graph's own:
            # a workload that cycles through more buckets than are kept then runs the rarer ones launch by launch
            # instead of capturing anew every time (a capture costs as much as tens of steps).
            least = min(self._step_graphs, key=lambda k: self._step_graphs[k].uses)
            if self._step_graphs[least].uses >= seen:
                return None
            self._step_graphs.pop(least)                                  # its memory pool goes with it
        graph = StepGraph(self, key)
        graph.uses = seen                        # it starts level with how often its bucket has come
        self._step_graphs[key] = graph
        return graph

    def graph_pool(self):
        """The one memory pool that all graphs of this runner record into.  They never run at the same time, so the
        intermediates of one may lie where another's do, and the pool grows to the largest graph instead of the sum of
        all; a graph's result (its logits) stays allocated and is never an intermediate of another.  A result is
        overwritten by whichever graph runs next, so it is consumed — sampled from, on the same stream — before the
        next step is launched."""
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        return self._graph_pool

    def warm_up(self, rows: Sequence[int] = (1, 2, 4, 8), longest: int = 2048) -> int:
        """Record the decode graphs for these numbers of requests and every class of context length up to ``longest``
        tokens ahead of the first request, instead of when each is first needed (a recording takes 10 to 20 ms, the
        first one of a process more).  The reference records all its buckets when it starts
        (csrc/executor/model_runner.cpp:40-52).  Returns how many graphs were recorded."""
        if not (self.config.enable_cuda_graph and self.model.capturable):
            return 0
        before = len(self._graphs)
        longest = min(longest, self.max_model_len)
        classes = [c for c in self.GRAPH_CONTEXTS if c < longest] + [longest]
        for n in rows:
            if 1 <= n <= min(self.config.max_num_seqs, self.GRAPH_BUCKETS[-1]):
                for c in classes:
                    self.decode_graph(n, c)
        return len(self._graphs) - before

    def capture_stream(self) -> torch.cuda.Stream:
        """The side stream graphs are recorded on (a recording may not run on the default stream)."""
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(self.device)
        return self._capture_stream

    def mark_device_begin(self) -> None:
        if self.timing is not None:
            self._timing_start = torch.cuda.Event(enable_timing=True)
            self._timing_start.record()

    def mark_device_end(self) -> None:
        if self.timing is not None and self._timing_start is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self.timing.append((self._timing_start, end))
            self._timing_start = None

    # ---- decode steps as CUDA graphs ---------------------------------------------------------------------
    # Row counts a graph is captured for.  Between powers of two there is a step in between: the launch shapes of a
    # graph (above all how the attention kernel splits the keys) are chosen for the bucket's rows, and 17 requests in a
    # graph made for 32 ran their attention at two thirds of the bandwidth of 16 in a graph made for 16.
    GRAPH_BUCKETS = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256)
    # A graph is also captured per class of context length: how the decode attention kernel splits the keys over
    # CTAs is fixed at capture, and a split chosen for the model's longest context is a poor one for short ones.
    GRAPH_CONTEXTS = (512, 2048, 8192, 32768, 131072)

    def can_use_graph(self, entries: Sequence[StepEntry]) -> bool:
        return (self.config.enable_cuda_graph and self.model.capturable and len(entries) <= self.GRAPH_BUCKETS[-1]
                and all(len(e.tokens) == 1 for e in entries))

    def decode_graph(self, rows: int, longest: Optional[int] = None) -> "DecodeGraph":
        """The graph for ``rows`` requests whose longest context (this step's token included) is ``longest``."""
        bucket = next(b for b in self.GRAPH_BUCKETS if b >= rows)
        longest = self.max_model_len if longest is None else longest
        context = min(self.max_model_len, next((c for c in self.GRAPH_CONTEXTS if c >= longest), self.max_model_len))
        graph = self._graphs.get((bucket, context))
        if graph is None:
            stride = (self.max_model_len + self.page_size - 1) // self.page_size
            graph = DecodeGraph(self, bucket, stride, context)
            graph.capture()
            self._graphs[(bucket, context)] = graph
        return graph

    def decode_step(self, entries: Sequence[StepEntry], trusted: bool = False,
                    token_ids_device: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One decode step (every entry brings one token and wants its logits) by graph replay.
        Returns float32 logits ``[len(entries), vocab]``; the tensor is overwritten by the next decode step.
        ``trusted``: the entries come from this package's scheduler, which has reserved their pages and sampled their
        tokens itself; the per-entry checks are skipped.  ``token_ids_device``: the step's input ids, one per entry, as
        an int32 tensor on the device (the sampler's output of the step before); the entries' own ids are then ignored."""
        if not trusted:
            self._validate_decode(entries)
        self.storage.zero_slots(self.manager.take_newly_admitted())
        mgr = self.manager
        starts = [mgr.num_tokens(e.request_id) for e in entries]
        graph = self.decode_graph(len(entries), max(starts) + 1)
        graph.upload(entries, starts, token_ids_device)
        logits = graph.replay()
        for e in entries:
            self.manager.commit(e.request_id, 1)
        self.steps_run += 1
        self.graph_steps += 1
        self.tokens_run += len(entries)
        return logits[:len(entries)]


def record_graph(device: torch.device, forward, stream: torch.cuda.Stream, pool=None):
    """Record ``forward()`` into a CUDA graph on ``stream`` and return ``(graph, what forward returned)``.

    Done by hand rather than under ``torch.cuda.graph``: that synchronises, collects garbage and empties the allocator's
    cache on the way in, which made a recording cost as much as twenty steps (0.2 s for a decode graph) and the steps
    after it pay for fresh device memory.  The cyclic collector is off meanwhile instead: collecting inside a recording
    could destroy another engine's graph, which is an error there; relaxed mode lets other threads use the allocator.
    ``pool``: a memory pool shared with graphs that never run at the same time as this one."""
    graph = torch.cuda.CUDAGraph()
    stream.wait_stream(torch.cuda.current_stream(device))
    collecting = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.stream(stream):
            if pool is not None:
                graph.capture_begin(pool=pool, capture_error_mode="relaxed")
            else:
                graph.capture_begin(capture_error_mode="relaxed")
            try:
                result = forward()
            finally:
                graph.capture_end()
    finally:
        if collecting:
            gc.enable()
    torch.cuda.current_stream(device).wait_stream(stream)
    return graph, result


class DecodeGraph:
    """A CUDA graph of one decode step for a fixed number of request rows (a bucket).

    The reference captures its forward pass per token-count bucket (powers of two) and launches attention
    between graph segments (csrc/executor/cuda_graph_runner.cpp:11-22, :51-115).  Here a bucket's whole
    step — embedding, every layer with its attention, final norm and output head — is one graph: the
    attention kernels read lengths and block tables from device memory, so their launch shape does not
    depend on the batch.  Rows beyond the live requests are padding: token 0, position 0, no cache write
    (slot -1), an empty block table; their logits are never read.

    All per-step inputs live in one device arena that is refreshed by a single copy from pinned memory.
    """

    def __init__(self, runner: "ModelRunner", rows: int, table_stride: int, context: Optional[int] = None) -> None:
        self._runner = weakref.ref(runner)       # no cycle: a dropped engine frees its graphs at once
        self.rows = rows
        self.stride = table_stride
        self.context = context or runner.max_model_len      # the context length the kernels' launch shapes are chosen for
        G = len(runner.groups)
        B, P = rows, table_stride
        self.layout = {}
        off = 0
        for name, n in [("tok", B), ("pos", B), ("treq", B), ("qsl", B + 1), ("sl", B), ("slots", B), ("want", B)]:
            self.layout[name] = (off, n)
            off += n
        for g in range(G):
            self.layout[f"sm{g}"] = (off, B)
            off += B
            self.layout[f"bt{g}"] = (off, B * P)
            off += B * P
        self.total = off
        self.pinned = [torch.empty(off, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.events: List[Optional[torch.cuda.Event]] = [None, None]
        self.row_state = [[[None] * rows for _ in range(G)] for _ in range(2)]   # per staging buffer, group, row
        self.turn = 0
        self.arena = torch.zeros(off, dtype=torch.int32, device=runner.device)
        for buf in self.pinned:
            host = buf.numpy()
            host[:] = 0
            self._fill_constants(host)
        self.ctx = self._context()
        self.logits: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.kernels_per_replay = 0

    @property
    def runner(self) -> "ModelRunner":
        runner = self._runner()
        if runner is None:
            raise RuntimeError("the engine of this decode graph is gone")
        return runner

    def _view(self, host: np.ndarray, name: str) -> np.ndarray:
        off, n = self.layout[name]
        return host[off:off + n]

    def _dev(self, name: str) -> torch.Tensor:
        off, n = self.layout[name]
        return self.arena[off:off + n]

    def _fill_constants(self, host: np.ndarray) -> None:
        B = self.rows
        self._view(host, "treq")[:] = np.arange(B, dtype=np.int32)
        self._view(host, "qsl")[:] = np.arange(B + 1, dtype=np.int32)
        self._view(host, "want")[:] = np.arange(B, dtype=np.int32)
        self._view(host, "sl")[:] = 1
        self._view(host, "slots")[:] = -1
        for g in range(len(self.runner.groups)):       # padding rows never write to the cache
            self._view(host, f"sm{g}")[:] = -1
            self._view(host, f"bt{g}")[:] = -1

    def _context(self) -> StepContext:
        r = self.runner
        B, P = self.rows, self.stride
        groups = {g: GroupView(r.page_size, self._dev(f"bt{g}").view(B, P), self._dev(f"sm{g}"))
                  for g in range(len(r.groups))}
        ctx = StepContext(
            num_tokens=B, num_requests=B, token_ids=self._dev("tok"), positions=self._dev("pos"),
            token_request=self._dev("treq"), query_start_loc=self._dev("qsl"), seq_lens=self._dev("sl"),
            state_slots=self._dev("slots"), query_start_loc_host=list(range(B + 1)), seq_lens_host=None,
            state_slots_host=None, max_query_len=1, max_seq_len=self.context, groups=groups, decode_only=True)
        for run, (src, writes) in r._run_cache.items():
            ctx.kv[run] = PagedKV(r.storage.run_cache[src], groups[r.storage.run_group[src]], writes)
        ctx.state = r.storage.state
        return ctx

    def _forward(self) -> torch.Tensor:
        stream = self.runner.model.forward(self.ctx)
        return self.runner.model.logits(stream, self._dev("want"))

    def upload(self, entries: Sequence[StepEntry], starts: Optional[List[int]] = None,
               token_ids_device: Optional[torch.Tensor] = None) -> None:
        r = self.runner
        mgr = r.manager
        i = self.turn
        self.turn ^= 1
        if self.events[i] is not None:
            self.events[i].synchronize()
        host = self.pinned[i].numpy()
        B, P, ps = self.rows, self.stride, r.page_size
        n = len(entries)
        tok, pos, sl, slots = (self._view(host, k) for k in ("tok", "pos", "sl", "slots"))
        if starts is None:
            starts = [mgr.num_tokens(e.request_id) for e in entries]
        tok[:n] = [e.tokens[0] for e in entries]
        tok[n:] = 0
        pos[:n] = starts
        pos[n:] = 0
        sl[:n] = np.asarray(starts, dtype=np.int32) + 1
        sl[n:] = 1
        slots[:n] = [mgr.slot(e.request_id) for e in entries]
        slots[n:] = -1          # padding rows own no state
        # Block-table rows change rarely (a page every page_size steps): each staging buffer remembers which
        # admission (the manager's serial, not the caller's id: an id may come back with other pages) and how many
        # pages every row holds, and only new entries are written.
        state = self.row_state[i]
        for g in range(len(r.groups)):
            sm = self._view(host, f"sm{g}")
            bt = self._view(host, f"bt{g}").reshape(B, P)
            windowed = r.groups[g].window is not None
            for row in range(n, B):
                if state[g][row] is not None:
                    bt[row, :] = -1
                    state[g][row] = None
            sm[n:] = -1
            for row, (e, start) in enumerate(zip(entries, starts)):
                table = mgr.block_table(e.request_id, g)
                k = len(table)
                if k > P:
                    raise StepError(f"request {e.request_id!r} holds {k} pages, more than the graph's table stride {P}")
                known = state[g][row]
                serial = mgr.serial(e.request_id)
                if not windowed and known is not None and known[0] == serial and known[1] <= k:
                    if known[1] < k:
                        bt[row, known[1]:k] = table[known[1]:k]
                else:
                    bt[row, :k] = table
                    bt[row, k:] = -1
                state[g][row] = (serial, k)
                page = table[start // ps]
                if page < 0:
                    raise StepError(f"request {e.request_id!r}: its new token has no page in group {g}")
                sm[row] = page * ps + start % ps
        r.mark_device_begin()
        self.arena.copy_(self.pinned[i], non_blocking=True)
        if self.events[i] is None:
            self.events[i] = torch.cuda.Event()
        self.events[i].record()
        if token_ids_device is not None:
            self._dev("tok")[:n].copy_(token_ids_device[:n], non_blocking=True)

    def capture(self) -> None:
        from .. import kernels

        # one eager run first: library handles and workspaces are created outside the capture
        self.arena.copy_(self.pinned[0], non_blocking=True)
        before = kernels.launch_count
        self._forward()
        self.kernels_per_replay = kernels.launch_count - before
        torch.cuda.synchronize(self.runner.device)
        self.graph, self.logits = record_graph(self.runner.device, self._forward, self.runner.capture_stream(),
                                               pool=self.runner.graph_pool())
        torch.cuda.synchronize(self.runner.device)

    def replay(self) -> torch.Tensor:
        from .. import kernels
        self.graph.replay()
        kernels.note_flagged_launch(replayed=True)      # the captured kernels have bounded waits that raise a flag
        return self.logits


class StepGraph:
    """A CUDA graph of one step of fixed sizes: so many tokens, requests and wanted rows (``ModelRunner.step_bucket``).

    Positions, cache slots, block tables, token ids, the requests' boundaries and the indices of the wanted rows are
    data in the graph's own device arena (packed by ``ModelRunner.build_context`` as for an eager step, padded to the
    graph's sizes, and refreshed by one copy), so any batch that fits the sizes replays it.  What shapes a launch — the
    attention kernels' tile counts — is sized for the worst split of the tokens over the requests
    (``StepContext.launch_query_lens``); CTAs beyond the batch's own tiles find no request and leave.  The first use
    runs the step eagerly (that is its result) and then records it; later uses replay.  The logits tensor is
    overwritten by the next replay of this or any other step graph of the runner (they share one memory pool); the
    engine samples from it, on the same stream, before it launches another step.
    """

    def __init__(self, runner: "ModelRunner", key: Tuple[int, int, int]) -> None:
        self._runner = weakref.ref(runner)
        self.key = key
        T, R, S = key
        G = len(runner.groups)
        self.stride = (runner.max_model_len + runner.page_size - 1) // runner.page_size
        total = 3 * T + (R + 1) + 2 * R + S + G * (T + R * self.stride)
        self.arena = torch.empty(total, dtype=torch.int32, device=runner.device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.uses = 1                            # times the runner has picked this graph (it decides what to drop by it)

    def run(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        from .. import kernels

        runner = self._runner()
        if runner is None:
            raise RuntimeError("the engine of this step graph is gone")
        T, R, S = self.key
        wanted = sum(len(e.want) for e in entries)
        ctx, want = runner.build_context(entries, table_stride=self.stride, arena=self.arena, pad=self.key)
        # what a replay cannot know stays off the host side of the context: launches are sized for the worst split of
        # the graph's tokens over its requests (one more 128-row tile than the tokens fill, one tile per further request)
        ctx.query_start_loc_host = None
        ctx.seq_lens_host = None
        ctx.state_slots_host = None
        ctx.launch_query_lens = [T + 128] + [1] * (R - 1)
        ctx.max_query_len = T
        ctx.max_seq_len = runner.max_model_len
        if self.graph is not None:
            self.graph.replay()
            kernels.note_flagged_launch(replayed=True)
            runner.step_graph_replays += 1
            return self.logits[:wanted]

        def forward() -> torch.Tensor:
            stream = runner.model.forward(ctx)
            if want.numel():
                return runner.model.logits(stream, want)
            return torch.empty((0, runner.vocab_size), dtype=torch.float32, device=runner.device)

        logits = forward()                       # this step's result; also creates what must exist before a capture
        self.graph, self.logits = record_graph(runner.device, forward, runner.capture_stream(), pool=runner.graph_pool())
        runner.step_graph_captures += 1
        return logits[:wanted]
