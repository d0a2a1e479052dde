"""The engine against the plain implementation, under every way of cutting the work, in 32-bit and bfloat16.

Each test replays token ids through ``cuinfer_b200.engine.replay`` (the code behind ``bin/trace_run``): the same
model, step function, cache manager and kernels that generation uses.
"""
from __future__ import annotations

import os
import subprocess
import sys

import numpy as np
import pytest

import traces
from conftest import ROOT, TOLERANCE, random_tokens

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B", "C", "D"]


def _requests(cfg, lengths, seed):
    return {f"r{i}": random_tokens(cfg["vocab_size"], n, seed * 100 + i) for i, n in enumerate(lengths)}


def _run(model_folders, name, dtype, steps, requests, tmp_path, max_tokens=None):
    folders, cfg, block = model_folders[name]
    folder = folders[dtype]
    out = str(tmp_path / f"out_{name}_{dtype}")
    peak = traces.live_token_peak(steps)
    runner = traces.replay_in_process(folder, dtype, steps, out, max_tokens or peak, block)
    got = traces.collect(steps, out, cfg["vocab_size"])
    worst = traces.compare_with_plain(folder, requests, got, TOLERANCE[dtype])
    return runner, worst


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(model_folders, name, dtype, tmp_path):
    cfg = model_folders[name][1]
    requests = _requests(cfg, [1, 5, 17, 33, 100, 161], seed=1)
    _run(model_folders, name, dtype, traces.whole(requests), requests, tmp_path)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_tokens_one_by_one(model_folders, name, dtype, tmp_path):
    cfg = model_folders[name][1]
    requests = _requests(cfg, [40, 97, 130], seed=2)
    _run(model_folders, name, dtype, traces.tail_decode(requests, 32), requests, tmp_path)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_changing_size(model_folders, name, dtype, tmp_path):
    cfg = model_folders[name][1]
    requests = _requests(cfg, [64, 131, 90], seed=3)
    _run(model_folders, name, dtype, traces.portions(requests), requests, tmp_path)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_batches_with_page_reuse(model_folders, name, dtype, tmp_path):
    cfg = model_folders[name][1]
    requests = _requests(cfg, [70, 33, 120, 58, 90, 45, 101], seed=4)
    steps = traces.mixed(requests, max_live=4)
    peak = traces.live_token_peak(steps)
    total = sum((len(t) + 63) // 64 * 64 for t in requests.values())
    assert peak < total, "the pool must be smaller than all requests together, so that pages are used again"
    assert any(len(st["entries"]) > 1 and {len(e["tokens"]) for e in st["entries"]} != {1} and
               any(len(e["tokens"]) == 1 for e in st["entries"]) for st in steps), "portions beside decoded tokens"
    runner, _ = _run(model_folders, name, dtype, steps, requests, tmp_path, max_tokens=peak)
    assert runner.num_pages * runner.page_size == peak


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(model_folders, dtype, tmp_path):
    """Hundreds of single-token steps after a short prompt, across many pages."""
    cfg = model_folders["C"][1]
    requests = _requests(cfg, [420], seed=5)
    _run(model_folders, "C", dtype, traces.tail_decode(requests, 400), requests, tmp_path)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence(model_folders, dtype, tmp_path):
    """Positions 0, 1, 2: one key, no history, page offset zero."""
    cfg = model_folders["B"][1]
    requests = _requests(cfg, [1, 2, 3], seed=6)
    _run(model_folders, "B", dtype, traces.tail_decode(requests, 3), requests, tmp_path)


def test_decode_through_tma_and_long_prompts(model_folders, tmp_path, monkeypatch):
    """The head-128 model in bfloat16 with the decode kernel forced onto its TMA path (the engine keeps short key
    streams on cp.async) and prompts of several row tiles: whole, then cut into portions beside decoded tokens."""
    from cuinfer_b200 import kernels
    monkeypatch.setattr(kernels, "DECODE_TMA_MIN_KEYS", 0)
    cfg = model_folders["D"][1]
    requests = _requests(cfg, [300, 170, 45, 260], seed=8)
    _run(model_folders, "D", "bfloat16", traces.tail_decode(requests, 40), requests, tmp_path)
    steps = traces.mixed(requests, max_live=3, sizes=(130, 2, 40, 3, 150, 7))
    _run(model_folders, "D", "bfloat16", steps, requests, tmp_path, max_tokens=traces.live_token_peak(steps))


def test_trace_run_program(model_folders, tmp_path):
    """``bin/trace_run`` as a user calls it: lines on stdin, ``done`` lines back, files in --out, exit 0."""
    folders, cfg, block = model_folders["A"]
    folder = folders["float32"]
    requests = _requests(cfg, [37, 20], seed=7)
    steps = traces.mixed(requests, max_live=2)
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
         "--out", str(out), "--max-tokens", str(traces.live_token_peak(steps))],
        input=traces.to_lines(steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {st['step']}" for st in steps]
    got = traces.collect(steps, str(out), cfg["vocab_size"])
    traces.compare_with_plain(folder, requests, got, TOLERANCE["float32"])
