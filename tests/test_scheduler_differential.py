"""The scheduler and the cache manager against the reference's own, step by step, on the CPU.

When a checkout of the reference is at hand (``$CUINFER_REFERENCE_SOURCE``, default: a folder ``reference`` beside
this repository), its
``csrc/scheduler/scheduler.cpp`` and ``csrc/scheduler/kv_cache_manager.cpp`` are compiled unchanged, in a temporary
folder, with a small driver (``tests/differential/reference_scheduler_driver.cpp``), ``nlohmann/json.hpp`` from an
installed package and a two-macro stand-in for ``msgpack.hpp``; nothing is copied into this repository.  The same
scenario then runs through both schedulers, with the model replaced by "every sample is token 1", and every step's
decisions are compared: which requests run, from which position, how many tokens, whether the portion samples,
whether it counts as prefill, the block ids each request holds (both pools hand out and take back pages first in,
first out, so the ids agree too), and which requests finish with which reason.  Skipped where the reference or a
compiler is missing.  Prefix caching is off on the reference's side (it is not built here).
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

import pytest

from cuinfer_b200.cache import CacheGroupSpec, CacheManager
from cuinfer_b200.engine.scheduler import FinishReason, Scheduler
from cuinfer_b200.sampling import SamplingParams

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE = os.environ.get("CUINFER_REFERENCE_SOURCE",
                           os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))

MSGPACK_STUB = "#pragma once\n#define MSGPACK_DEFINE_MAP(...)\n#define MSGPACK_ADD_ENUM(...)\n"


def _json_header():
    for base in sys.path:
        if base and os.path.isdir(base):
            for pattern in ("include/nlohmann/json.hpp", "include/*/thirdparty/nlohmann/json.hpp", "nlohmann/json.hpp"):
                hits = glob.glob(os.path.join(base, pattern))
                if hits:
                    return hits[0]
    for path in ("/usr/include/nlohmann/json.hpp", "/usr/local/include/nlohmann/json.hpp"):
        if os.path.exists(path):
            return path
    return None


@pytest.fixture(scope="module")
def reference_driver(tmp_path_factory):
    csrc = os.path.join(REFERENCE, "csrc")
    if not os.path.exists(os.path.join(csrc, "scheduler", "scheduler.cpp")):
        pytest.skip("no checkout of the reference here")
    gxx = shutil.which("g++")
    header = _json_header()
    if gxx is None or header is None:
        pytest.skip("no g++ or no nlohmann/json.hpp here")
    work = tmp_path_factory.mktemp("reference_scheduler")
    os.makedirs(work / "stub" / "nlohmann")
    (work / "stub" / "msgpack.hpp").write_text(MSGPACK_STUB)
    shutil.copyfile(header, work / "stub" / "nlohmann" / "json.hpp")
    exe = str(work / "driver")
    cmd = [gxx, "-std=c++20", "-O1", f"-I{csrc}", f"-I{work / 'stub'}", "-o", exe,
           os.path.join(HERE, "differential", "reference_scheduler_driver.cpp"),
           os.path.join(csrc, "scheduler", "scheduler.cpp"), os.path.join(csrc, "scheduler", "kv_cache_manager.cpp")]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        pytest.skip(f"the reference's scheduler does not compile here: {proc.stderr[-300:]}")
    return exe


REASONS = {FinishReason.RUNNING: 0, FinishReason.STOP: 1, FinishReason.LENGTH: 2}


def _ours(config, script):
    max_seqs, budget, max_len, block, pages = config
    mgr = CacheManager([CacheGroupSpec((0,), 2, 16, None)], block, pages, max_seqs)
    sched = Scheduler(mgr, max_num_seqs=max_seqs, max_num_scheduled_tokens=budget, max_model_len=max_len)
    lines, step = [], 0
    for op in script:
        if op[0] == "add":
            _, rid, n, max_out = op
            sched.add_request(rid, [2] * n, SamplingParams(temperature=0.0, max_tokens=max_out, ignore_eos=True))
        elif op[0] == "abort":
            sched.abort_requests([op[1]])
        else:
            scheduled = sched.schedule()
            if not scheduled:
                lines.append(f"idle {step}")
            sampled = []
            for s in scheduled:
                rid = s.request.request_id
                blocks = " ".join(str(b) for b in mgr.block_table(rid, 0))
                lines.append(f"sched {step} {rid} {s.position_offset} {len(s.tokens)} {int(s.needs_sampling)} "
                             f"{int(s.is_prefill)} {blocks}".rstrip())
                mgr.commit(rid, len(s.tokens))
                if s.needs_sampling:
                    sampled.append((rid, 1))
            mgr.check()
            for o in sched.update(sampled):
                assert o.finish_reason in REASONS, f"our scheduler decided {o.finish_reason} where the reference has no such case"
                lines.append(f"out {step} {o.request_id} {REASONS[o.finish_reason]}")
            step += 1
    return lines


def _theirs(exe, config, script):
    text = "config " + " ".join(str(v) for v in config) + "\n"
    for op in script:
        text += " ".join(str(v) for v in op) + "\n"
    proc = subprocess.run([exe], input=text, capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0, proc.stderr[-500:]
    return proc.stdout.splitlines()


def _steps(n):
    return [("step",)] * n


SCENARIOS = {
    # three prompts under a budget of 24: the third is cut 2 + 22 + 9 beside the others' decoded tokens
    "portions_6_pages": ((8, 24, 256, 16, 6), [("add", "a", 5, 8), ("add", "b", 17, 8), ("add", "c", 33, 8)] + _steps(14)),
    # the same with 4 pages: the last running request is preempted, recomputed later on pages given back
    "preemption_4_pages": ((8, 24, 256, 16, 4), [("add", "a", 5, 8), ("add", "b", 17, 8), ("add", "c", 33, 8)] + _steps(40)),
    # tiny B's workload: prompts 1 / 31 / 64 / 100, 12 outputs, portions of 24, pages of 32 tokens
    "tiny_b": ((4, 24, 768, 32, 12), [("add", "r0", 1, 12), ("add", "r1", 31, 12), ("add", "r2", 64, 12),
                                      ("add", "r3", 100, 12)] + _steps(40)),
    # more requests than max_num_seqs, arrivals and an abort in between, tight pages, finish by max_model_len
    "arrivals_aborts_limits": ((3, 40, 64, 8, 14), [("add", "a", 30, 40), ("add", "b", 9, 5), ("step",), ("add", "c", 21, 9),
                                                     ("add", "d", 3, 30)] + _steps(5) + [("abort", "c"), ("add", "e", 50, 20)] +
                               _steps(12) + [("add", "f", 7, 3), ("abort", "nobody")] + _steps(60)),
    # one token of budget per step: everything crawls, order must still agree
    "budget_of_seven": ((8, 7, 128, 4, 40), [("add", "a", 19, 6), ("add", "b", 8, 6), ("add", "c", 30, 2)] + _steps(45)),
}


@pytest.mark.parametrize("name", sorted(SCENARIOS))
def test_scheduler_decides_as_the_reference_does(reference_driver, name):
    config, script = SCENARIOS[name]
    ours = _ours(config, script)
    theirs = _theirs(reference_driver, config, script)
    for i, (a, b) in enumerate(zip(ours, theirs)):
        assert a == b, f"{name}: first difference at line {i}: ours {a!r}, the reference {b!r}"
    assert len(ours) == len(theirs)
    assert any(line.startswith("out") and line.endswith(" 2") for line in ours)         # something did finish
    if name == "preemption_4_pages":
        # a request that ran before runs again from position 0 with more tokens than its prompt: it was preempted
        assert any(l.split()[2] == "c" and l.split()[3] == "0" and int(l.split()[4]) > 2 for l in ours if l.startswith("sched"))
