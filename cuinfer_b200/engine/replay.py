"""Trace replay: feed given token ids through the model step by step and write the logits.

It samples nothing and schedules nothing.  It drives the same model, step function, cache manager and
kernels that generation uses (``ModelRunner.step``); the only thing of its own is the reading of the trace.
The reference has no such tool (its engine returns sampled ids only, csrc/executor/model_runner.cpp:94-107).

Input, one JSON object per line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step are one batch.  For a step in which logits are wanted, ``<out>/<step>.f32`` holds them
as little-endian float32 ``[wanted, vocab]`` in the order of the entries and of ``want``.  After each step
``done <step>`` is printed and flushed.  Requests named in ``end`` give back what they hold after the step.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional

from .. import kernels
from ..config import EngineConfig
from .runner import ModelRunner, StepEntry

TRACE_TOKEN_ROUNDING = 64


def make_runner(model_dir: str, dtype: str, max_tokens: int, block_size: int = 16, max_live: int = 8,
                cuda_graph: bool = False) -> ModelRunner:
    """A runner whose page pool holds exactly ``max_tokens`` tokens (rounded up to whole pages).
    ``cuda_graph``: steps go the way generation sends them — a step of single tokens that all want their logits
    through ``ModelRunner.decode_step`` (one CUDA graph per bucket of rows and class of context length), a
    step of other shape, padded to a bucket of sizes that has come before, through the graph captured for the
    bucket; default: every step eagerly."""
    if max_tokens <= 0:
        raise ValueError("--max-tokens must be positive")
    unit = max(TRACE_TOKEN_ROUNDING, block_size)
    rounded = (max_tokens + unit - 1) // unit * unit
    pages = (rounded + block_size - 1) // block_size
    config = EngineConfig(model_path=model_dir, block_size=block_size, dtype=dtype, num_blocks=pages,
                          max_num_seqs=max_live, max_num_scheduled_tokens=1 << 30, enable_cuda_graph=cuda_graph)
    return ModelRunner(model_dir, config)


def run_trace(runner: ModelRunner, lines, out_dir: str, log=sys.stdout) -> int:
    os.makedirs(out_dir, exist_ok=True)
    steps = 0
    for raw in lines:
        raw = raw.strip()
        if not raw:
            continue
        try:
            rec = json.loads(raw)
            step_id = rec["step"]
            entries = [StepEntry(e["id"], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])])
                       for e in rec.get("entries", [])]
            ended = list(rec.get("end", []))
        except (ValueError, KeyError, TypeError) as exc:
            raise SystemExit(f"trace_run: cannot read step line {raw[:120]!r}: {exc}")
        if entries:
            for e in entries:
                if not runner.reserve(e.request_id, len(e.tokens)):
                    raise SystemExit(
                        f"trace_run: step {step_id}: no room for {len(e.tokens)} more tokens of request {e.request_id!r} "
                        f"({runner.manager.num_free_pages()} pages of {runner.page_size} tokens free); --max-tokens is too small")
            if runner.can_use_graph(entries) and all(list(e.want) == [0] for e in entries):
                logits = runner.decode_step(entries)
            else:
                logits = runner.step(entries)
            if logits.shape[0]:
                host = logits.float().cpu().contiguous().numpy().astype("<f4", copy=False)
                kernels.check_error_flags()
                with open(os.path.join(out_dir, f"{step_id}.f32"), "wb") as fh:
                    fh.write(host.tobytes())
        for rid in ended:
            runner.release(rid)
        print(f"done {step_id}", file=log, flush=True)
        steps += 1
    return steps


def main(argv: Optional[List[str]] = None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    parser.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    parser.add_argument("--graphs", action="store_true",
                        help="run decode steps and steps whose bucket of sizes has come before from CUDA graphs, as generation does")
    args = parser.parse_args(argv)
    runner = make_runner(args.model, args.dtype, args.max_tokens, args.block_size, cuda_graph=args.graphs)
    run_trace(runner, sys.stdin, args.out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
