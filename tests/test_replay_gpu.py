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
    worst = traces.compare_with_plain(folder, requests, got, TOLERANCE[dtype], label=f"replay of tiny {name}")
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


CUTS = {
    "whole": (lambda r: traces.whole(r), [1, 5, 17, 33, 100, 161]),
    "tail": (lambda r: traces.tail_decode(r, 32), [40, 97, 130]),
    "portions": (lambda r: traces.portions(r), [64, 131, 90]),
    "mixed": (lambda r: traces.mixed(r, max_live=4), [70, 33, 120, 58, 90, 45, 101]),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "D"])
@pytest.mark.parametrize("cut", sorted(CUTS))
def test_cuts_through_cuda_graphs(model_folders, name, dtype, cut, tmp_path, monkeypatch):
    """The four cuts again, through the paths generation really takes: every step of single tokens is a replayed
    decode graph (padding rows, incremental block-table upload), every other step is padded to a bucket of sizes and,
    once the bucket has come back, a replayed step graph (spare tokens in a request without pages, spare requests,
    spare wanted rows).  The trace runs three times through one runner and the logits of the last pass, all from
    replays, are compared at the same tolerance as eager steps."""
    from cuinfer_b200.engine.runner import ModelRunner
    monkeypatch.setattr(ModelRunner, "STEP_GRAPH_MIN_TOKENS", 2)
    monkeypatch.setattr(ModelRunner, "STEP_GRAPH_LIMIT", 64)
    folders, cfg, block = model_folders[name]
    folder = folders[dtype]
    build, lengths = CUTS[cut]
    requests = _requests(cfg, lengths, seed=11)
    steps = build(requests)
    out = str(tmp_path / "out")
    runner = traces.replay_in_process(folder, dtype, steps, out, traces.live_token_peak(steps), block,
                                      cuda_graph=True, passes=3)
    got = traces.collect(steps, out, cfg["vocab_size"])
    traces.compare_with_plain(folder, requests, got, TOLERANCE[dtype], label=f"graph replay {cut} of tiny {name}")
    decode_steps = sum(all(len(e["tokens"]) == 1 and e["want"] == [0] for e in st["entries"]) for st in steps)
    assert runner.graph_steps == 3 * decode_steps
    other = len(steps) - decode_steps
    shapes = {tuple((len(e["tokens"]), len(e["want"])) for e in st["entries"]) for st in steps
              if not all(len(e["tokens"]) == 1 and e["want"] == [0] for e in st["entries"])}
    buckets = {ModelRunner.step_bucket([n for n, _ in shape], [w for _, w in shape]) for shape in shapes}
    # a bucket of sizes runs launch by launch when it first comes, is captured when it comes back (in pass 2 at the
    # latest), and pass 3 replays everything
    assert runner.step_graph_replays >= other and len(runner._step_graphs) == len(buckets)


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_graph_buckets_and_padding_rows(model_folders, dtype, tmp_path):
    """Decode steps with 17, 9 and 3 live requests: graphs for 24, 12 and 4 rows with 7, 3 and 1 padding rows, the
    rows of requests that ended cleared for those that move up.  Logits of every step against the plain model."""
    folders, cfg, block = model_folders["B"]
    folder = folders[dtype]
    requests = _requests(cfg, [20 + 3 * i for i in range(17)], seed=12)
    ids = list(requests)
    steps, s, done = [], 0, {}
    for rid in ids:                                  # prompts, one request a step, all but the last 12 tokens
        head = len(requests[rid]) - 12
        steps.append({"step": s, "entries": [{"id": rid, "tokens": requests[rid][:head], "want": [head - 1]}], "end": []})
        done[rid] = head
        s += 1
    live = list(ids)
    for round_no in range(12):
        entries = [{"id": r, "tokens": [requests[r][done[r]]], "want": [0]} for r in live]
        for r in live:
            done[r] += 1
        leaving = []
        if round_no == 3:
            leaving = live[:8]                       # 9 stay and move up to rows 0..8
        elif round_no == 7:
            leaving = live[3:]                       # 3 stay
        elif round_no == 11:
            leaving = list(live)
        steps.append({"step": s, "entries": entries, "end": leaving})
        live = [r for r in live if r not in leaving]
        s += 1
    out = str(tmp_path / "out")
    runner = traces.replay_in_process(folder, dtype, steps, out, traces.live_token_peak(steps), block,
                                      cuda_graph=True, max_live=32)
    assert sorted(b for b, _c in runner._graphs) == [4, 12, 24]
    got = traces.collect(steps, out, cfg["vocab_size"])
    import plain_qwen3
    cfg_p, weights = plain_qwen3.load_folder(folder)
    for rid, rows in got.items():
        ref = plain_qwen3.forward(cfg_p, weights, list(requests[rid])).numpy()
        scale = float(np.abs(ref).max())
        for pos, row in rows.items():
            err = float(np.abs(row - ref[pos]).max()) / scale
            assert err <= TOLERANCE[dtype], (rid, pos, err)


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_graph_across_context_classes(model_folders, dtype, tmp_path):
    """A request that decodes from 500 to 530 tokens changes the class of context length its decode graph is
    captured for (512 -> 2048): another graph, another split of the keys, the same logits."""
    folders, cfg, block = model_folders["C"]
    requests = _requests(cfg, [530, 140], seed=13)
    steps = traces.tail_decode(requests, 30)
    out = str(tmp_path / "out")
    runner = traces.replay_in_process(folders[dtype], dtype, steps, out, traces.live_token_peak(steps), block,
                                      cuda_graph=True)
    assert sorted(c for _b, c in runner._graphs) == [512, min(2048, cfg["max_position_embeddings"])]
    got = traces.collect(steps, out, cfg["vocab_size"])
    traces.compare_with_plain(folders[dtype], requests, got, TOLERANCE[dtype])


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


def test_step_graphs_pad_to_their_bucket_and_do_not_thrash(model_folders, monkeypatch):
    """Steps of other shapes in one bucket replay one captured graph and give the logits of eager steps; with room
    for two graphs and three buckets in turn, the third keeps running launch by launch instead of pushing a graph out
    every time it comes (a capture costs as much as tens of steps)."""
    from cuinfer_b200.engine import replay
    from cuinfer_b200.engine.runner import ModelRunner, StepEntry

    monkeypatch.setattr(ModelRunner, "STEP_GRAPH_MIN_TOKENS", 2)
    monkeypatch.setattr(ModelRunner, "STEP_GRAPH_LIMIT", 2)
    folders, cfg, block = model_folders["D"]
    graphed = replay.make_runner(folders["bfloat16"], "bfloat16", 4096, block, cuda_graph=True)
    eager = replay.make_runner(folders["bfloat16"], "bfloat16", 4096, block, cuda_graph=False)
    shapes = {"a": [[33, 5, 1], [30, 1, 9], [36, 2, 1]],         # bucket (48, 4, 4): 9, 8 and 9 spare tokens
              "b": [[70], [66]],                                   # bucket (80, 2, 2)
              "c": [[100, 3], [97, 12]]}                           # bucket (112, 4, 4)
    serial = 0
    worst = 0.0
    for round_ in range(6):
        for name in "abc":
            lens = shapes[name][round_ % len(shapes[name])]
            ids = [f"{name}{round_}_{i}" for i in range(len(lens))]
            tokens = [random_tokens(cfg["vocab_size"], n, 900 + serial + i) for i, n in enumerate(lens)]
            serial += 7
            out = []
            for runner in (graphed, eager):
                entries = [StepEntry(i, t, [len(t) - 1]) for i, t in zip(ids, tokens)]
                for e in entries:
                    assert runner.reserve(e.request_id, len(e.tokens))
                out.append(runner.step(entries).float().cpu())
                for i in ids:
                    runner.release(i)
                runner.manager.check()
            scale = float(out[1].abs().max())
            worst = max(worst, float((out[0] - out[1]).abs().max()) / scale)
    assert worst <= 2e-2, worst          # same kernels on the same rows; only the row count of the products differs
    # "a" and "b" are captured when they come the second time; "c" finds both places taken by graphs that are used as
    # often as it comes, and never pushes one out
    assert len(graphed._step_graphs) == 2 and graphed.step_graph_captures == 2
    assert graphed.step_graph_replays == 2 * 4


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_context_of_eight_thousand_tokens(dtype, tmp_path):
    """A request of 8 230 tokens — past the third class of context lengths that decode graphs are recorded for, 515 pages
    in its block table, rotation angles at positions no other test reaches — beside a short one: the prompt in three
    portions (each starting thousands of keys into the cache), then thirty tokens one by one in a two-row decode graph
    whose rows hold 8 200 and 60 keys.  bfloat16 on head size 128 (tcgen05 attention with a long prefix, decode through
    TMA with many splits), 32-bit on the all-sizes kernels; against the plain implementation at the wanted places."""
    import plain_qwen3
    import torch
    from conftest import GAINS, TINY_A, TINY_D, note_error
    from cuinfer_b200.weights import write_random_model

    base = TINY_D if dtype == "bfloat16" else TINY_A
    cfg = dict(base, num_hidden_layers=1 if dtype == "bfloat16" else 2, max_position_embeddings=9216)
    folder = str(tmp_path / "long_model")
    write_random_model(folder, cfg, 21, std=0.05, gain_std=0.1, dtype=dtype, gains=GAINS[dtype])
    long_ids = random_tokens(cfg["vocab_size"], 8230, 77)
    short_ids = random_tokens(cfg["vocab_size"], 90, 78)
    steps, s = [], 0
    for lo, hi, want in [(0, 3000, [2999]), (3000, 6000, [0, 1500, 2999]), (6000, 8200, [0, 2199])]:
        steps.append({"step": s, "entries": [{"id": "long", "tokens": long_ids[lo:hi], "want": want}], "end": []})
        s += 1
    steps.append({"step": s, "entries": [{"id": "short", "tokens": short_ids[:60], "want": [59]}], "end": []})
    s += 1
    for i in range(30):
        steps.append({"step": s, "entries": [{"id": "long", "tokens": [long_ids[8200 + i]], "want": [0]},
                                               {"id": "short", "tokens": [short_ids[60 + i]], "want": [0]}],
                      "end": ["long", "short"] if i == 29 else []})
        s += 1
    out = str(tmp_path / "out")
    runner = traces.replay_in_process(folder, dtype, steps, out, traces.live_token_peak(steps), 16, cuda_graph=True)
    assert runner.graph_steps == 30
    got = traces.collect(steps, out, cfg["vocab_size"])
    pcfg, weights = plain_qwen3.load_folder(folder)
    worst = 0.0
    for rid, ids in (("long", long_ids), ("short", short_ids)):
        places = sorted(got[rid])
        ref = plain_qwen3.logits_at(pcfg, weights, ids, places).numpy()
        scale = float(np.abs(ref).max())
        for row, place in zip(ref, places):
            assert np.isfinite(got[rid][place]).all()
            err = float(np.abs(got[rid][place] - row).max()) / scale
            worst = max(worst, err)
            assert err <= TOLERANCE[dtype], f"request {rid}: position {place} is off by {err:.3e} of the largest logit"
    note_error(dtype, "a context of 8 230 tokens", worst)
