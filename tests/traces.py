"""Builders of replay traces (the step lines ``bin/trace_run`` reads) and the comparison of what comes back
with the plain implementation.  A trace is a list of dicts ``{"step", "entries": [{"id", "tokens", "want"}], "end"}``.
"""
from __future__ import annotations

import io
import json
import os
from typing import Dict, List, Sequence

import numpy as np
import torch

import plain_qwen3


def whole(requests: Dict[str, Sequence[int]]) -> List[dict]:
    """Each request alone and whole: one step per request, logits wanted everywhere."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def tail_decode(requests: Dict[str, Sequence[int]], tail: int = 32) -> List[dict]:
    """Most of each request in one step, then its last ``tail`` tokens one by one."""
    steps = []
    s = 0
    for rid, toks in requests.items():
        toks = list(toks)
        head = max(1, len(toks) - tail)
        steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        s += 1
        for p in range(head, len(toks)):
            steps.append({"step": s, "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
            s += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests: Dict[str, Sequence[int]], sizes: Sequence[int] = (7, 2, 13, 3, 2, 21, 5, 2, 34, 16, 2, 17)) -> List[dict]:
    """Each request alone, cut into portions of changing size, down to two tokens."""
    steps = []
    s = 0
    k = 0
    for rid, toks in requests.items():
        toks = list(toks)
        p = 0
        while p < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - p)
            k += 1
            steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[p:p + n], "want": list(range(n))}],
                          "end": [rid] if p + n == len(toks) else []})
            p += n
            s += 1
    return steps


def mixed(requests: Dict[str, Sequence[int]], max_live: int = 4, prefill_until: Dict[str, int] | None = None,
          sizes: Sequence[int] = (5, 2, 11, 3, 24, 2, 7), skip_every: int = 5) -> List[dict]:
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of others in one step.

    A request is fed in portions up to ``prefill_until[rid]`` (default: two thirds of it) and token by token
    after that; every ``skip_every``-th turn a request sits a step out.  A finished request ends in that
    step, and the next waiting request starts in the following one, on the pages just given back.
    """
    order = list(requests)
    waiting = list(order)
    live: List[str] = []
    done_at: Dict[str, int] = {rid: 0 for rid in order}
    steps = []
    s = 0
    k = 0
    turn = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            live.append(waiting.pop(0))
        entries = []
        ended = []
        for rid in list(live):
            turn += 1
            toks = list(requests[rid])
            p = done_at[rid]
            if skip_every and turn % skip_every == 0 and len(live) > 1 and p > 0:
                continue
            limit = (prefill_until or {}).get(rid, max(1, 2 * len(toks) // 3))
            if p < limit:
                n = min(sizes[k % len(sizes)], limit - p)
                k += 1
            else:
                n = 1
            n = min(n, len(toks) - p)
            entries.append({"id": rid, "tokens": toks[p:p + n], "want": list(range(n))})
            done_at[rid] = p + n
            if p + n == len(toks):
                ended.append(rid)
                live.remove(rid)
        if entries:
            steps.append({"step": s, "entries": entries, "end": ended})
            s += 1
    return steps


def live_token_peak(steps: List[dict], rounding: int = 64) -> int:
    """The most tokens live requests hold at any time, each request's count rounded up to ``rounding``."""
    held: Dict[str, int] = {}
    peak = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum((n + rounding - 1) // rounding * rounding for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def to_lines(steps: List[dict]) -> str:
    return "".join(json.dumps(st) + "\n" for st in steps)


def collect(steps: List[dict], out_dir: str, vocab: int) -> Dict[str, Dict[int, np.ndarray]]:
    """{request: {position: logits row}} from the ``<step>.f32`` files of a replay."""
    got: Dict[str, Dict[int, np.ndarray]] = {}
    done: Dict[str, int] = {}
    for st in steps:
        wanted = sum(len(e["want"]) for e in st["entries"])
        rows = None
        if wanted:
            path = os.path.join(out_dir, f"{st['step']}.f32")
            rows = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
        r = 0
        for e in st["entries"]:
            base = done.get(e["id"], 0)
            for w in e["want"]:
                got.setdefault(e["id"], {})[base + w] = rows[r]
                r += 1
            done[e["id"]] = base + len(e["tokens"])
    return got


def replay_in_process(model_dir: str, dtype: str, steps: List[dict], out_dir: str, max_tokens: int, block_size: int,
                      cuda_graph: bool = False, passes: int = 1, max_live: int = 8):
    """Run a trace through ``cuinfer_b200.engine.replay`` in this process (same code as ``bin/trace_run``).
    ``passes``: run the whole trace this often through the same runner (a step shape is captured into a CUDA graph
    only when it comes back); the files of the last pass stay."""
    from cuinfer_b200.engine import replay

    runner = replay.make_runner(model_dir, dtype, max_tokens, block_size, max_live=max_live, cuda_graph=cuda_graph)
    for _ in range(passes):
        log = io.StringIO()
        replay.run_trace(runner, to_lines(steps).splitlines(), out_dir, log=log)
        assert log.getvalue().split() == [w for st in steps for w in ("done", str(st["step"]))]
    runner.manager.check()
    assert not runner.manager.live_requests(), "every request of the trace ended, so nothing may stay held"
    return runner


def compare_with_plain(model_dir: str, requests: Dict[str, Sequence[int]], got, tolerance: float, label: str = ""):
    """Every collected row against the plain implementation's logits of the whole sequence.
    Returns the largest error seen, as a fraction of the largest plain logit of its sequence."""
    cfg, weights = plain_qwen3.load_folder(model_dir)
    worst = 0.0
    for rid, toks in requests.items():
        ref = plain_qwen3.forward(cfg, weights, list(toks)).numpy()
        scale = float(np.abs(ref).max())
        rows = got.get(rid, {})
        assert rows, f"no logits came back for request {rid}"
        for pos, row in sorted(rows.items()):
            assert np.isfinite(row).all(), f"request {rid} position {pos}: logits are not finite"
            err = float(np.abs(row - ref[pos]).max()) / scale
            worst = max(worst, err)
            assert err <= tolerance, (
                f"request {rid}: first wrong position {pos} of {len(toks)} (error {err:.3e} of the largest logit, "
                f"allowed {tolerance:.1e})")
    if label:
        from conftest import note_error
        note_error("float32" if tolerance < 1e-3 else "bfloat16", label, worst)
    return worst
