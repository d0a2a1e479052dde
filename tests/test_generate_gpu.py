"""Generation through the Python entry point and the command line, against the plain implementation."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen3
from conftest import ROOT, random_tokens

pytestmark = pytest.mark.gpu


def _near_best(cfg, weights, prompt, tokens, slack):
    """Every generated token is the plain argmax, or within ``slack`` of it (a near-tie that rounding may flip)."""
    ids = list(prompt)
    for t in tokens:
        row = plain_qwen3.forward(cfg, weights, ids)[-1]
        assert float(row.max() - row[t]) <= slack * float(row.abs().max()), (prompt, tokens, t)
        ids.append(t)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_float32_equals_plain(model_folders, name):
    from cuinfer_b200 import LLM, SamplingParams

    folders, cfg, block = model_folders[name]
    folder = folders["float32"]
    pcfg, weights = plain_qwen3.load_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, 50 + i) for i, n in enumerate([5, 17, 33, 1])]
    llm = LLM(folder, dtype="float32", block_size=block, num_blocks=64, max_num_seqs=4, max_num_scheduled_tokens=24)
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    for prompt, res in zip(prompts, out):
        assert res.finish_reason == "length" and len(res.token_ids) == 8
        assert res.token_ids == plain_qwen3.greedy_generate(pcfg, weights, prompt, 8)
    assert llm.engine.stats["prefill_tokens"] == sum(len(p) for p in prompts)
    llm.engine.runner.manager.check()
    assert not llm.engine.runner.manager.live_requests()


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_greedy_generation_bfloat16_is_near_best(model_folders, name):
    from cuinfer_b200 import LLM, SamplingParams

    folders, cfg, block = model_folders[name]
    folder = folders["bfloat16"]
    pcfg, weights = plain_qwen3.load_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, 60 + i) for i, n in enumerate([9, 30, 2])]
    llm = LLM(folder, dtype="bfloat16", block_size=block, num_blocks=64, max_num_seqs=4, max_num_scheduled_tokens=16)
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    for prompt, res in zip(prompts, out):
        _near_best(pcfg, weights, prompt, res.token_ids, 0.04)


def test_preemption_and_recompute_give_the_same_tokens(model_folders):
    """With so few pages that requests are preempted and recomputed, greedy float32 output is unchanged."""
    from cuinfer_b200 import LLM, SamplingParams

    folders, cfg, block = model_folders["A"]
    folder = folders["float32"]
    prompts = [random_tokens(cfg["vocab_size"], n, 70 + i) for i, n in enumerate([30, 31, 20, 14])]
    params = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    roomy = LLM(folder, dtype="float32", block_size=16, num_blocks=64, max_num_seqs=4, max_num_scheduled_tokens=64)
    want = [r.token_ids for r in roomy.generate(prompts, params)]
    assert roomy.engine.scheduler.num_preemptions == 0
    tight = LLM(folder, dtype="float32", block_size=16, num_blocks=8, max_num_seqs=4, max_num_scheduled_tokens=64)
    got = [r.token_ids for r in tight.generate(prompts, params)]
    assert tight.engine.scheduler.num_preemptions > 0
    assert got == want
    tight.engine.runner.manager.check()


def test_eos_stops_and_is_returned(model_folders):
    from cuinfer_b200 import LLM, SamplingParams

    folders, cfg, block = model_folders["A"]
    folder = folders["float32"]
    pcfg, weights = plain_qwen3.load_folder(folder)
    prompt = random_tokens(cfg["vocab_size"], 12, 80)
    free_run = plain_qwen3.greedy_generate(pcfg, weights, prompt, 6)
    # make the third generated token the end-of-sequence id of a copy of the model
    import shutil, tempfile
    with tempfile.TemporaryDirectory() as tmp:
        shutil.copytree(folder, tmp, dirs_exist_ok=True)
        raw = json.load(open(os.path.join(tmp, "config.json")))
        raw["eos_token_id"] = free_run[2]
        json.dump(raw, open(os.path.join(tmp, "config.json"), "w"))
        llm = LLM(tmp, dtype="float32", num_blocks=16)
        stop = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=6))[0]
        first = free_run.index(free_run[2])
        assert stop.finish_reason == "stop" and stop.token_ids == free_run[:first + 1]
        go_on = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))[0]
        assert go_on.finish_reason == "length" and go_on.token_ids == free_run


def test_run_ahead_gives_the_same_outputs(model_folders):
    """Launching the next decode step before the ids of the one in flight have been read changes nothing: requests of
    different lengths and budgets (so that the run-ahead stops and starts), one that stops at an end-of-sequence token
    while its next step is already in flight, one that is aborted in flight, temperature sampling with a seed."""
    import shutil, tempfile
    from cuinfer_b200 import LLM, SamplingParams

    folders, cfg, block = model_folders["B"]
    folder = folders["float32"]
    pcfg, weights = plain_qwen3.load_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, 400 + i) for i, n in enumerate([9, 40, 3, 77, 21])]
    free = plain_qwen3.greedy_generate(pcfg, weights, prompts[1], 10)
    with tempfile.TemporaryDirectory() as tmp:
        shutil.copytree(folder, tmp, dirs_exist_ok=True)
        raw = json.load(open(os.path.join(tmp, "config.json")))
        raw["eos_token_id"] = free[4]                 # request 1 stops at its fifth token
        json.dump(raw, open(os.path.join(tmp, "config.json"), "w"))
        params = [SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True),
                  SamplingParams(temperature=0.0, max_tokens=10),
                  SamplingParams(temperature=0.8, top_k=40, top_p=0.95, max_tokens=7, ignore_eos=True, seed=5),
                  SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True),
                  SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)]
        results = {}
        for ahead in (False, True):
            llm = LLM(tmp, dtype="float32", block_size=block, num_blocks=40, max_num_seqs=8, decode_run_ahead=ahead)
            out = llm.generate(prompts, params)
            results[ahead] = [(r.token_ids, r.finish_reason) for r in out]
            engine = llm.engine
            assert (engine.stats["run_ahead_steps"] > 0) == ahead
            engine.runner.manager.check()
            assert not engine.runner.manager.live_requests()
            if ahead:
                # abort while a step is in flight: the aborted row is dropped, the other request is not disturbed
                engine.add_request("x", prompts[0], SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True))
                engine.add_request("y", prompts[4], SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True))
                got = {"x": [], "y": []}
                steps = 0
                while engine.has_requests():
                    for o in engine.step():
                        got[o.request_id].extend(o.new_token_ids)
                    steps += 1
                    if steps == 4:
                        engine.abort(["x"])
                assert got["y"] == results[True][4][0][:9] and len(got["x"]) < 9
                engine.runner.manager.check()
                assert not engine.runner.manager.live_requests()
        assert results[True] == results[False]
        assert results[True][1] == (free[:5], "stop")
        assert results[True][0][0] == plain_qwen3.greedy_generate(pcfg, weights, prompts[0], 12)


def test_decode_graphs_per_context_class(model_folders):
    """Decoding across a context-class boundary (512) switches to another captured graph; the tokens are those of
    the plain implementation, in 32-bit and (near-best) on the head-128 model in bfloat16."""
    from cuinfer_b200 import LLM, SamplingParams

    folders, cfg, block = model_folders["B"]
    pcfg, weights = plain_qwen3.load_folder(folders["float32"])
    prompts = [random_tokens(cfg["vocab_size"], n, 70 + i) for i, n in enumerate([505, 40])]
    llm = LLM(folders["float32"], dtype="float32", block_size=block, num_blocks=40, max_num_seqs=4)
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    for prompt, res in zip(prompts, out):
        assert res.token_ids == plain_qwen3.greedy_generate(pcfg, weights, prompt, 12)
    keys = sorted(llm.engine.runner._graphs)
    assert {k[1] for k in keys} == {512, cfg["max_position_embeddings"]}, keys       # 512, then 2048 capped by the model
    folders, cfg, block = model_folders["D"]
    pcfg, weights = plain_qwen3.load_folder(folders["bfloat16"])
    prompt = random_tokens(cfg["vocab_size"], 508, 77)
    llm = LLM(folders["bfloat16"], dtype="bfloat16", block_size=block, num_blocks=40, max_num_seqs=2)
    res = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))[0]
    _near_best(pcfg, weights, prompt, res.token_ids, 0.04)
    assert len(llm.engine.runner._graphs) == 2


def test_repeated_prompt_shapes_replay_a_graph(model_folders):
    """A prompt-sized step whose bucket of sizes has come before is captured and then replayed: four rounds of prompts of the
    same lengths but other tokens, on other pages of the pool (pages that were given back are taken last), give the
    plain implementation's tokens every time."""
    from cuinfer_b200 import LLM, SamplingParams

    folders, cfg, block = model_folders["B"]
    pcfg, weights = plain_qwen3.load_folder(folders["float32"])
    llm = LLM(folders["float32"], dtype="float32", block_size=block, num_blocks=48, max_num_seqs=4,
              max_num_scheduled_tokens=1024)
    for round_ in range(4):
        prompts = [random_tokens(cfg["vocab_size"], n, 300 + 10 * round_ + i) for i, n in enumerate([300, 270])]
        out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
        for prompt, res in zip(prompts, out):
            assert res.token_ids == plain_qwen3.greedy_generate(pcfg, weights, prompt, 5), round_
    runner = llm.engine.runner
    assert len(runner._step_graphs) == 1 and runner.step_graph_replays == 2
    runner.manager.check()
    # bfloat16 on the head-128 model: the tensor-core kernels inside the captured step
    folders, cfg, block = model_folders["D"]
    pcfg, weights = plain_qwen3.load_folder(folders["bfloat16"])
    llm = LLM(folders["bfloat16"], dtype="bfloat16", block_size=block, num_blocks=64, max_num_seqs=2, max_num_scheduled_tokens=1024)
    for round_ in range(3):
        prompt = random_tokens(cfg["vocab_size"], 400, 500 + round_)
        res = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))[0]
        _near_best(pcfg, weights, prompt, res.token_ids, 0.04)
    assert llm.engine.runner.step_graph_replays >= 1


def test_entry_point_refuses_bad_requests(model_folders):
    from cuinfer_b200 import LLM, SamplingParams

    folders, cfg, block = model_folders["A"]
    llm = LLM(folders["float32"], dtype="float32", num_blocks=16)
    limit = cfg["max_position_embeddings"]
    for prompt, params, word in [
        ([], SamplingParams(), "at least one"),
        ([1] * limit, SamplingParams(max_tokens=1), "shorter"),
        ([1] * 10, SamplingParams(max_tokens=limit), "exceeds"),
        ([1, cfg["vocab_size"]], SamplingParams(max_tokens=2), "vocabulary"),
        ([1, -1], SamplingParams(max_tokens=2), "vocabulary"),
    ]:
        with pytest.raises(ValueError, match=word):
            llm.generate([prompt], params)
    for bad in (dict(temperature=-1.0), dict(top_k=-1), dict(top_p=0.0), dict(top_p=1.5), dict(max_tokens=0)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
    assert not llm.engine.has_requests()


def test_sampling_is_reproducible_and_independent_of_the_batch(model_folders):
    from cuinfer_b200 import LLM, SamplingParams

    folders, cfg, block = model_folders["B"]
    folder = folders["float32"]
    prompts = [random_tokens(cfg["vocab_size"], n, 90 + i) for i, n in enumerate([7, 21, 40])]
    params = SamplingParams(temperature=0.9, top_k=50, top_p=0.9, max_tokens=10, ignore_eos=True, seed=1234)
    a = LLM(folder, dtype="float32", block_size=block, num_blocks=32, max_num_scheduled_tokens=16, seed=1)
    run1 = [r.token_ids for r in a.generate(prompts, params)]
    b = LLM(folder, dtype="float32", block_size=block, num_blocks=32, max_num_scheduled_tokens=512, seed=2)
    run2 = [r.token_ids for r in b.generate(prompts, params)]
    assert run1 == run2                       # same seed in the request: same tokens, however prompts were cut
    other = [r.token_ids for r in b.generate(prompts, SamplingParams(temperature=0.9, top_k=50, top_p=0.9,
                                                                       max_tokens=10, ignore_eos=True, seed=99))]
    assert other != run1


def test_command_line(model_folders, tmp_path):
    folders, cfg, block = model_folders["A"]
    folder = folders["float32"]
    pcfg, weights = plain_qwen3.load_folder(folder)
    prompt = random_tokens(cfg["vocab_size"], 9, 95)
    proc = subprocess.run(
        [sys.executable, "-m", "cuinfer_b200", "generate", "--model", folder, "--dtype", "float32",
         "--prompt-ids", ",".join(map(str, prompt)), "--prompt-ids", "4 5 6", "--max-tokens", "5", "--temperature", "0",
         "--ignore-eos", "--num-blocks", "16", "--max-num-seqs", "4"],
        capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 2 and lines[0]["prompt_token_ids"] == prompt
    assert lines[0]["token_ids"] == plain_qwen3.greedy_generate(pcfg, weights, prompt, 5)
    assert lines[1]["finish_reason"] == "length"
    bad = subprocess.run([sys.executable, "-m", "cuinfer_b200", "generate", "--model", folder, "--prompt-ids", "1",
                          "--block-size", "0"], capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert bad.returncode != 0 and "block_size" in bad.stderr


def test_random_workloads_do_not_depend_on_engine_settings(model_folders):
    """Requests that arrive over time with random lengths, budgets and sampling options (greedy and seeded), some
    aborted on the way: float32 outputs are the same with and without CUDA graphs and run-ahead, with pages so few that
    requests are preempted and recomputed, and with a small token budget and few sequences."""
    import random

    from cuinfer_b200 import SamplingParams
    from cuinfer_b200.config import EngineConfig
    from cuinfer_b200.engine.core import EngineCore

    folders, cfg, block = model_folders["B"]
    folder, vocab, longest = folders["float32"], cfg["vocab_size"], cfg["max_position_embeddings"]

    def workload(seed):
        rnd = random.Random(seed)
        requests = []
        for i in range(rnd.randint(12, 24)):
            budget = rnd.choice([1, 2, 3, 8, 20, 40])
            n = min(rnd.choice([1, 2, 5, 17, 33, 64, 100, 150]), longest - budget - 1)
            greedy = rnd.random() < 0.6
            params = SamplingParams(temperature=0.0 if greedy else rnd.choice([0.7, 1.0]), top_k=0 if greedy else rnd.choice([0, 20]),
                                    top_p=1.0 if greedy else rnd.choice([1.0, 0.9]), max_tokens=budget,
                                    ignore_eos=rnd.random() < 0.7, seed=None if greedy else rnd.randint(0, 99))
            requests.append(dict(id=f"r{i}", arrive=rnd.randint(0, 12), prompt=random_tokens(vocab, n, seed * 100 + i),
                                 params=params, abort_at=rnd.randint(3, 30) if rnd.random() < 0.15 else None))
        return requests

    def run(requests, **options):
        engine = EngineCore(EngineConfig(model_path=folder, dtype="float32", block_size=block, seed=1, **options))
        tokens, reasons = {r["id"]: [] for r in requests}, {}
        pending = sorted(requests, key=lambda r: r["arrive"])
        step = 0
        while pending or engine.has_requests():
            while pending and pending[0]["arrive"] <= step:
                r = pending.pop(0)
                engine.add_request(r["id"], r["prompt"], r["params"])
            engine.abort([r["id"] for r in requests if r["abort_at"] == step and r["id"] in engine.scheduler.requests])
            for out in engine.step():
                tokens[out.request_id].extend(out.new_token_ids)
                reasons[out.request_id] = out.finish_reason.value
            step += 1
            assert step < 3000, "no progress"
        engine.runner.manager.check()
        assert not engine.runner.manager.live_requests()
        return tokens, reasons, engine

    roomy = dict(num_blocks=400, max_num_seqs=16, max_num_scheduled_tokens=256)
    preempted = ahead = 0
    for seed in (10, 11, 12):
        requests = workload(seed)
        want, want_reasons, _ = run(requests, enable_cuda_graph=False, decode_run_ahead=False, **roomy)
        for options in (roomy, dict(roomy, decode_run_ahead=False),
                        dict(roomy, num_blocks=(190 + block - 1) // block + 3),
                        dict(roomy, max_num_seqs=4, max_num_scheduled_tokens=48)):
            got, reasons, engine = run(requests, **options)
            preempted += engine.scheduler.num_preemptions
            ahead += engine.stats["run_ahead_steps"]
            for r in requests:
                rid = r["id"]
                if r["abort_at"] is not None or "capacity" in (reasons.get(rid), want_reasons.get(rid)):
                    common = min(len(got[rid]), len(want[rid]))     # how far it got depends on the schedule
                    assert got[rid][:common] == want[rid][:common], (seed, options, rid)
                else:
                    assert got[rid] == want[rid] and reasons.get(rid) == want_reasons.get(rid), (seed, options, rid)
    assert preempted > 0 and ahead > 0


def _drive(engine, wanted_ids):
    """Step the engine until the requests ``wanted_ids`` are gone; returns their tokens."""
    out = {rid: [] for rid in wanted_ids}
    guard = 0
    while any(rid in engine.scheduler.requests for rid in wanted_ids):
        for o in engine.step():
            if o.request_id in out:
                out[o.request_id].extend(o.new_token_ids)
        guard += 1
        assert guard < 2000
    return out


@pytest.mark.parametrize("live", [1, 2])
def test_request_id_that_comes_back_gets_its_own_pages(model_folders, live):
    """A caller's request id may be used again after the request has ended (a conversation id).  The second
    request lands in the same row of the same decode graph with at least as many pages, from other places of the
    pool: the block-table rows that the graph keeps on the device must be written anew, or its attention reads the
    first request's pages.  Also after an abort.  Graphs on, float32, against the plain implementation."""
    from cuinfer_b200 import SamplingParams
    from cuinfer_b200.config import EngineConfig
    from cuinfer_b200.engine.core import EngineCore

    folders, cfg, block = model_folders["A"]
    folder = folders["float32"]
    pcfg, weights = plain_qwen3.load_folder(folder)
    engine = EngineCore(EngineConfig(model_path=folder, dtype="float32", block_size=block, num_blocks=40,
                                     max_num_seqs=4, max_num_scheduled_tokens=256, enable_cuda_graph=True))
    params = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    ids = ["x", "y"][:live]
    lengths = [[20, 37], [41, 40], [52, 49]]              # each round at least as many pages as the round before
    for round_no, lens in enumerate(lengths):
        prompts = {rid: random_tokens(cfg["vocab_size"], lens[i], 900 + 10 * round_no + i) for i, rid in enumerate(ids)}
        for rid in ids:
            engine.add_request(rid, prompts[rid], params)
        if round_no == 1:
            # abort in the middle of decoding, then the same ids once more with the same prompts
            for _ in range(8):
                engine.step()
            engine.abort(ids)
            while engine.has_requests():
                engine.step()
            for rid in ids:
                engine.add_request(rid, prompts[rid], params)
        got = _drive(engine, ids)
        for rid in ids:
            assert got[rid] == plain_qwen3.greedy_generate(pcfg, weights, prompts[rid], 24), (round_no, rid)
    assert engine.runner.graph_steps > 40
    engine.runner.manager.check()


@pytest.mark.parametrize("stored, engine", [("float32", "float32"), ("bfloat16", "bfloat16"), ("float32", "bfloat16")])
def test_weights_drawn_on_the_device_equal_the_host_generator(tmp_path, stored, engine):
    """A folder that names a recipe instead of holding tensors: the engine fills its weights on the device, bit for
    bit the values the host generator writes into a file (same seed, same names), under the same precision rule
    (a gain stored in 32 bits stays so on a bfloat16 engine); and generation from both folders gives the same tokens."""
    from conftest import TINY_B
    from cuinfer_b200 import LLM, SamplingParams
    from cuinfer_b200.weights import write_random_model

    kw = dict(std=0.05, gain_std=0.1, dtype=stored, gains={"q_norm": 2.0}, generator="counter")
    on_disk = write_random_model(str(tmp_path / "disk"), TINY_B, 9, **kw)
    recipe = write_random_model(str(tmp_path / "recipe"), TINY_B, 9, materialize=False, **kw)
    a = LLM(on_disk, dtype=engine, block_size=16, num_blocks=32, max_num_seqs=4)
    b = LLM(recipe, dtype=engine, block_size=16, num_blocks=32, max_num_seqs=4)
    ma, mb = a.engine.runner.model, b.engine.runner.model
    pairs = [(ma.embedding, mb.embedding), (ma.lm_head.weight, mb.lm_head.weight), (ma.final_norm.weight, mb.final_norm.weight)]
    for x, y in zip(ma.blocks, mb.blocks):
        pairs += [(x.mixer.qkv.weight, y.mixer.qkv.weight), (x.mixer.o.weight, y.mixer.o.weight),
                  (x.mixer.q_norm_weight, y.mixer.q_norm_weight), (x.mixer.k_norm_weight, y.mixer.k_norm_weight),
                  (x.feed_forward.gate_up.weight, y.feed_forward.gate_up.weight), (x.feed_forward.down.weight, y.feed_forward.down.weight),
                  (x.mixer_norm.weight, y.mixer_norm.weight), (x.feed_forward_norm.weight, y.feed_forward_norm.weight)]
    for x, y in pairs:
        assert x.dtype == y.dtype and x.shape == y.shape and torch.equal(x.cpu(), y.cpu())
    if stored == "float32" and engine == "bfloat16":
        assert ma.final_norm.weight.dtype == torch.float32 and ma.embedding.dtype == torch.bfloat16
    prompts = [random_tokens(TINY_B["vocab_size"], n, 950 + i) for i, n in enumerate([11, 40])]
    p = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    assert [r.token_ids for r in a.generate(prompts, p)] == [r.token_ids for r in b.generate(prompts, p)]


def test_warm_up_records_the_decode_graphs_ahead(model_folders):
    """After ``warm_up`` the first decode steps find their graphs recorded: generation adds none, and gives the plain
    implementation's tokens."""
    from cuinfer_b200 import LLM, SamplingParams

    folders, cfg, block = model_folders["B"]
    pcfg, weights = plain_qwen3.load_folder(folders["float32"])
    llm = LLM(folders["float32"], dtype="float32", block_size=block, num_blocks=64, max_num_seqs=4)
    recorded = llm.warm_up(batch_sizes=(1, 2, 3), longest=600)
    runner = llm.engine.runner
    assert recorded == len(runner._graphs) == 3 * 2        # rows 1, 2 and 4 (for 3), context classes 512 and 600
    assert llm.warm_up(batch_sizes=(1, 2, 3), longest=600) == 0
    prompts = [random_tokens(cfg["vocab_size"], n, 640 + i) for i, n in enumerate([40, 33, 21])]
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    for prompt, res in zip(prompts, out):
        assert res.token_ids == plain_qwen3.greedy_generate(pcfg, weights, prompt, 6)
    assert len(runner._graphs) == 6 and runner.graph_steps > 0
    runner.manager.check()
