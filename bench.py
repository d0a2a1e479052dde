"""Benchmark: decode tokens/s of the Qwen3-0.6B shape at batch 8 and context 4096 on one B200, bfloat16, random
weights; plus prefill of 2,048 tokens, decode at batch 1 and 64, and the decode step's share of the HBM roofline.

``python bench.py --gpus 1 --steps K --warmup W`` prints ONE JSON line.  A step is one decode step of the whole
batch.  ``value`` is decoded tokens per second counted on the device (CUDA events from the step's first copy to
its sampler kernel, summed over the K steps); ``e2e`` is the same through the engine's public step call with
host token ids in and out (each step's input copy from pinned memory and the read-back of the sampled ids are
inside the timed region).  Between timed steps nothing is flushed: a step reads over 1 GB of weights and cache,
far more than the 126 MB L2.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: the Qwen3-0.6B shape; benchmark context 4096, KV block size 16.
MODEL = dict(
    architectures=["Qwen3ForCausalLM"], num_hidden_layers=28, hidden_size=1024, num_attention_heads=16,
    num_key_value_heads=8, head_dim=128, intermediate_size=3072, vocab_size=151936, rope_theta=1000000.0,
    rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=4096, torch_dtype="bfloat16")
# The other shapes of BASELINE.json (configs[3], configs[4]); chosen with --shape, with --layers fewer layers.
SHAPES = {
    "0.6b": ("Qwen3-0.6B shape (BASELINE configs[2])", MODEL),
    "8b": ("Qwen3-8B shape (BASELINE configs[3])", dict(
        MODEL, num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
        intermediate_size=12288, tie_word_embeddings=False)),
    "32b": ("Qwen3-32B shape (BASELINE configs[4])", dict(
        MODEL, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8,
        intermediate_size=25600, tie_word_embeddings=False)),
}
MODEL_NAME = SHAPES["0.6b"][0]
CONTEXT = 4096
BLOCK_SIZE = 16
PREFILL_TOKENS = 2048


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            peaks = json.load(fh)
        peaks["source"] = "measured"
        return peaks
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the measurement runs.

    nvidia-smi needs a tenth of a second before its first sample and the timed steps of the small shape take less than
    that together, so the sampler starts before the requests are prefilled (the GPU is under this process's load from
    then on) and every sample carries its time: ``stop(window)`` reports the samples inside the timed window when
    there are at least three, else all samples from the prefill on, and says which."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.proc = None
        self.path = None

    def start(self) -> None:
        exe = shutil.which("nvidia-smi")
        if not exe:
            return
        fd, self.path = tempfile.mkstemp(prefix="clocks_", suffix=".csv")
        os.close(fd)
        self.proc = subprocess.Popen([exe, "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                      "-lms", "50"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)

    def stop(self, window=None) -> dict:
        """``window``: (start, end) of the timed steps as ``time.time()`` values."""
        import datetime

        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        samples, max_clock = [], None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as fh:
            for line in fh:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    when = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    clock = float(parts[1])
                    max_clock = float(parts[2])
                except ValueError:
                    continue
                samples.append((when, clock, {n for n, v in zip(names, parts[3:7]) if v.lower().startswith("active")}))
        os.remove(self.path)
        inside = [x for x in samples if window and window[0] <= x[0] <= window[1]]
        used, where = (inside, "timed steps") if len(inside) >= 3 else (samples, "prefill, warm-up and timed steps")
        reasons = set().union(*[x[2] for x in used]) if used else set()
        return {"sm_mhz": statistics.median(x[1] for x in used) if used else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(used), "window": where}


def weight_bytes(cfg: dict, layers: int) -> int:
    """Bytes of every weight a decode step reads once (bfloat16): the layers' matrices and norms, the final norm
    and the output head (the embedding table when tied; a decode step gathers only B rows of the input table)."""
    H, I, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    Q, KV = cfg["num_attention_heads"] * d, cfg["num_key_value_heads"] * d
    per_layer = H * (Q + 2 * KV) + Q * H + 3 * H * I + 2 * H + 2 * d
    return 2 * (layers * per_layer + H + cfg["vocab_size"] * H)


def kv_bytes_per_token(cfg: dict, layers: int) -> int:
    return 2 * layers * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg: dict, layers: int, T: int) -> float:
    H, I, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    Q, KV = cfg["num_attention_heads"] * d, cfg["num_key_value_heads"] * d
    linear = 2.0 * T * layers * (H * (Q + 2 * KV) + Q * H + 3 * H * I)
    attention = 2.0 * T * T * Q * layers          # QK^T and PV over the causal half
    return linear + attention + 2.0 * cfg["vocab_size"] * H


def make_engine(folder: str, batch: int, args):
    from cuinfer_b200.config import EngineConfig
    from cuinfer_b200.engine.core import EngineCore

    pages_per_request = (CONTEXT + BLOCK_SIZE - 1) // BLOCK_SIZE
    # --pool-from-memory: the cache pool is what 90 % of the device holds beside the weights, as in serving
    pages = None if args.pool_from_memory else batch * pages_per_request + 8
    config = EngineConfig(model_path=folder, block_size=BLOCK_SIZE, dtype="bfloat16", gpu_memory_utilization=0.9,
                          num_blocks=pages, max_num_seqs=max(batch, 8),
                          max_num_scheduled_tokens=8192, enable_cuda_graph=not args.disable_cuda_graph, seed=0)
    return EngineCore(config)


def measure_decode(folder: str, batch: int, steps: int, warmup: int, args, sample_clocks: bool = False,
                   context: int = 0) -> dict:
    """Prefill ``batch`` requests so that decoding ends at ``context`` tokens (default: CONTEXT), then time ``steps``
    decode steps."""
    import torch

    from cuinfer_b200 import SamplingParams, kernels

    context = context or CONTEXT
    engine = make_engine(folder, batch, args)
    total_steps = warmup + steps
    # prompts are admitted a few per step under the token budget, so early requests decode while later ones
    # are still being prefilled: leave room for those extra tokens below the context limit
    prefill_steps = (batch * context + 8191) // 8192 + 2
    prompt_len = context - total_steps - prefill_steps - 1
    gen = torch.Generator().manual_seed(1234 + batch)
    params = SamplingParams(temperature=0.0, max_tokens=context - prompt_len, ignore_eos=True)
    clocks = ClockSampler()
    if sample_clocks:
        clocks.start()
    for i in range(batch):
        prompt = torch.randint(0, MODEL["vocab_size"], (prompt_len,), generator=gen).tolist()
        engine.add_request(f"b{i}", prompt, params)
    # prefill (untimed): until every request has produced its first token
    while any(r.num_output_tokens == 0 for r in engine.scheduler.requests.values()):
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    ctx_start = statistics.mean(len(r.token_ids) for r in engine.scheduler.requests.values())
    engine.runner.timing = []
    launches_before = kernels.launch_count
    graph_before = engine.runner.graph_steps
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_push(f"timed_decode_b{batch}")      # lets a profiler pick the timed launches (--nvtx-include)
    window_start = time.time()
    t0 = time.perf_counter()
    tokens = 0
    for _ in range(steps):
        tokens += sum(len(o.new_token_ids) for o in engine.step())
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    torch.cuda.nvtx.range_pop()
    clock_info = clocks.stop((window_start, time.time())) if sample_clocks else None
    device_ms = sum(a.elapsed_time(b) for a, b in engine.runner.timing)
    pairs = len(engine.runner.timing)
    engine.runner.timing = None
    assert tokens == batch * steps and pairs == steps, (tokens, pairs)
    graph_steps = engine.runner.graph_steps - graph_before
    per_replay = max((g.kernels_per_replay for g in engine.runner._graphs.values()), default=0)
    launches = (kernels.launch_count - launches_before) + graph_steps * per_replay
    ctx_mid = ctx_start + steps / 2.0        # mean tokens a request holds during the timed steps
    out = {
        "tokens_per_s": tokens / (device_ms / 1e3), "ms_per_step": device_ms / steps,
        "e2e_tokens_per_s": tokens / wall, "e2e_ms_per_step": wall * 1e3 / steps, "launches": launches,
        "graph_steps": graph_steps, "context_mid": ctx_mid, "prompt_len": prompt_len, "clocks": clock_info,
        # the step's arena (token ids, positions, slot mapping, lengths, block-table rows) from pinned memory;
        # greedy sampling options stay on the device from step to step
        "h2d_bytes": (engine.runner._graphs[next(iter(engine.runner._graphs))].total * 4 if engine.runner._graphs else 0),
        "d2h_bytes": batch * 4,
    }
    while engine.has_requests():
        engine.abort(list(engine.scheduler.requests))
    del engine
    torch.cuda.empty_cache()
    return out


def measure_generate(folder: str, in_flight: int, args, prompt_len: int = 1024, outputs: int = 128) -> dict:
    """The reference's own workload (benchmark.sh:67-97: random prompts of 1 024 tokens, 128 outputs, a fixed number of
    requests in flight) through ``LLM.generate``-style continuous batching: ``3 * in_flight`` requests are fed so that
    ``in_flight`` are live at any time (a new one is added when one ends), host token ids in and out.  Every step is
    a new mix of prompt portions and decoded tokens, so this is where the host's share of a step shows."""
    import torch

    from cuinfer_b200 import SamplingParams
    from cuinfer_b200.config import EngineConfig
    from cuinfer_b200.engine.core import EngineCore

    pages = in_flight * ((prompt_len + outputs + BLOCK_SIZE) // BLOCK_SIZE + 1) + 8
    engine = EngineCore(EngineConfig(model_path=folder, block_size=BLOCK_SIZE, dtype="bfloat16", num_blocks=pages,
                                     max_num_seqs=max(in_flight, 8), max_num_scheduled_tokens=8192,
                                     enable_cuda_graph=not args.disable_cuda_graph, seed=0))
    gen = torch.Generator().manual_seed(4321 + in_flight)
    total = 3 * in_flight
    prompts = [torch.randint(0, MODEL["vocab_size"], (prompt_len,), generator=gen).tolist() for _ in range(total)]
    params = SamplingParams(temperature=0.0, max_tokens=outputs, ignore_eos=True)

    def run(first: int, count: int) -> tuple[int, float]:
        nxt, done, tokens = first, 0, 0
        for _ in range(min(in_flight, count)):
            engine.add_request(f"g{nxt}", prompts[nxt % total], params)
            nxt += 1
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        while engine.has_requests():
            for o in engine.step():
                tokens += len(o.new_token_ids)
                if o.finish_reason.value != "running":
                    done += 1
                    if nxt < first + count:
                        engine.add_request(f"g{nxt}", prompts[nxt % total], params)
                        nxt += 1
        torch.cuda.synchronize()
        return tokens, time.perf_counter() - t0

    run(0, in_flight)                                   # warm-up, twice: kernels loaded, then the step shapes that come
    run(0, in_flight)                                   # back are captured as graphs (a server does this once)
    steps0, graph0, replay0 = engine.runner.steps_run, engine.runner.graph_steps, engine.runner.step_graph_replays
    tokens, wall = run(in_flight, total)
    steps = engine.runner.steps_run - steps0
    graphs = (engine.runner.graph_steps - graph0) + (engine.runner.step_graph_replays - replay0)
    out = {"output_tokens_per_s": round(tokens / wall, 1), "total_tokens_per_s": round((tokens + total * prompt_len) / wall, 1),
           "requests": total, "steps": steps, "steps_from_graphs": graphs, "wall_s": round(wall, 3)}
    del engine
    torch.cuda.empty_cache()
    return out


def measure_prefill(folder: str, args) -> dict:
    import torch

    from cuinfer_b200.engine.runner import StepEntry

    engine = make_engine(folder, 1, args)
    runner = engine.runner
    gen = torch.Generator().manual_seed(99)
    tokens = torch.randint(0, MODEL["vocab_size"], (PREFILL_TOKENS,), generator=gen).tolist()
    times = []
    for it in range(3 + 5):
        assert runner.reserve("p", PREFILL_TOKENS)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        if it >= 3:
            torch.cuda.nvtx.range_push("timed_prefill")
        logits = runner.step([StepEntry("p", tokens, [PREFILL_TOKENS - 1])])
        if it >= 3:
            torch.cuda.nvtx.range_pop()
        b.record()
        torch.cuda.synchronize()
        runner.release("p")
        if it >= 3:
            times.append(a.elapsed_time(b))
        assert logits.shape == (1, MODEL["vocab_size"])
    del engine
    torch.cuda.empty_cache()
    return {"ms": statistics.median(times)}


def write_reference_model(folder: str, cfg: dict, seed: int) -> None:
    """A model folder for the reference arm, written without any of this repository's code: the tensor names and
    shapes the reference looks up (csrc/model/causal_lm.cpp:35-53, csrc/model/layers/attention.cpp:22-40,
    csrc/model/layers/mlp.cpp:12-17) as bfloat16 N(0, 0.02), gains 1, in one safetensors file."""
    import struct

    import torch

    H, I, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    Q, KV = cfg["num_attention_heads"] * d, cfg["num_key_value_heads"] * d
    shapes = {"model.embed_tokens.weight": (cfg["vocab_size"], H), "model.norm.weight": (H,)}
    if not cfg["tie_word_embeddings"]:
        shapes["lm_head.weight"] = (cfg["vocab_size"], H)
    for i in range(cfg["num_hidden_layers"]):
        pre = f"model.layers.{i}."
        shapes.update({
            pre + "input_layernorm.weight": (H,), pre + "post_attention_layernorm.weight": (H,),
            pre + "self_attn.q_proj.weight": (Q, H), pre + "self_attn.k_proj.weight": (KV, H),
            pre + "self_attn.v_proj.weight": (KV, H), pre + "self_attn.o_proj.weight": (H, Q),
            pre + "self_attn.q_norm.weight": (d,), pre + "self_attn.k_norm.weight": (d,),
            pre + "mlp.gate_proj.weight": (I, H), pre + "mlp.up_proj.weight": (I, H), pre + "mlp.down_proj.weight": (H, I)})
    header, offset = {}, 0
    for name, shape in shapes.items():
        size = 2
        for n in shape:
            size *= n
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [offset, offset + size]}
        offset += size
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    gen = torch.Generator().manual_seed(seed)
    with open(os.path.join(folder, "model.safetensors"), "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name, shape in shapes.items():
            if name.endswith("norm.weight"):
                t = torch.ones(shape, dtype=torch.bfloat16)
            else:
                t = (torch.randn(shape, generator=gen, dtype=torch.float32) * 0.02).to(torch.bfloat16)
            fh.write(t.view(torch.int16).numpy().tobytes())
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(dict(cfg, eos_token_id=cfg["vocab_size"] - 1), fh)


def reference_arm(args) -> int:
    """The same metric on the same configuration through the UNMODIFIED reference engine: its scheduler and model
    runner (stock kernels, cuBLAS, CUDA graphs, sampler) driven by ``baseline/reference_bench.cpp``, which runs the
    loop of csrc/engine/engine_core.cpp:93-105 without the socket.  Nothing of cuinfer_b200 is imported."""
    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": " ".join(why.split())[:600]}))
        return 0

    if args.shape != "0.6b" or args.layers not in (0, MODEL["num_hidden_layers"]):
        return unavailable("the reference's kernels take hidden size 1024 or 2048 only (csrc/ops/rms_norm.cu:115-130); "
                           "the arm runs the 0.6B shape at full depth")
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import build_reference
        binary = build_reference.build()
    except Exception as exc:      # noqa: BLE001 - any build problem makes the arm unavailable, with its message
        return unavailable(f"the reference engine could not be built here: {exc}")
    if shutil.which("nvidia-smi") is None:
        return unavailable("no GPU on this machine")
    args.warmup = max(args.warmup, 3)
    cfg = dict(MODEL, max_position_embeddings=CONTEXT)
    tmp = tempfile.mkdtemp(prefix="cuinfer_reference_bench_")

    def run(batch: int, steps: int, prefill_tokens: int, mode: str = "bench") -> dict:
        cmd = [binary, "--mode", mode, "--prompt-len", "1024", "--max-tokens", "128", "--model", tmp, "--batch", str(batch), "--context", str(CONTEXT),
               "--steps", str(steps), "--warmup", str(args.warmup), "--prefill-tokens", str(prefill_tokens),
               "--block-size", str(BLOCK_SIZE), "--max-num-scheduled-tokens", "8192", "--max-num-seqs", "256",
               "--gpu-memory-utilization", "0.9", "--seed", "1234"]
        if args.disable_cuda_graph:
            cmd.append("--disable-cuda-graph")
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
        if proc.returncode != 0:
            raise RuntimeError(f"reference_bench exited with {proc.returncode}: {proc.stderr[-400:]}")
        return json.loads(proc.stdout.strip().splitlines()[-1])

    try:
        write_reference_model(tmp, cfg, seed=0)
        clocks = ClockSampler()
        clocks.start()
        main_run = run(args.batch, args.steps, PREFILL_TOKENS if not args.skip_points else 0)
        clock_info = clocks.stop()
        points = {}
        if not args.skip_points:
            for b in (1, 64):
                r = run(b, min(args.steps, 128), 0)
                points[f"decode_b{b}"] = round(b * 1e3 / r["device_ms_per_step"], 1)
        mixed = {f"in_flight_{c}": run(c, 1, 0, mode="serve") for c in (8, 32)} if args.mixed else None
    except Exception as exc:      # noqa: BLE001
        return unavailable(f"the reference engine did not run: {exc}")
    finally:
        shutil.rmtree(tmp, ignore_errors=True)

    peaks = load_peaks()
    line = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2048 tokens; % of roofline",
        "value": round(args.batch * 1e3 / main_run["device_ms_per_step"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(main_run["device_ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02) seed 0, uniform-random token ids", "impl": "reference",
        "config": {
            "model": MODEL_NAME, "layers": MODEL["num_hidden_layers"], "layers_full": MODEL["num_hidden_layers"],
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "tied_embeddings": True, "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": main_run["prompt_len"],
            "kv_block_size": BLOCK_SIZE, "parallelism": "single GPU", "cuda_graph": not args.disable_cuda_graph,
            "l2": "no flush: each step reads >1 GB, far more than the 126 MB L2", "peaks": peaks["source"],
        },
        "e2e": {"value": round(args.batch * 1e3 / main_run["ms_per_step"], 1), "unit": "tokens/s",
                "ms_per_step": round(main_run["ms_per_step"], 4),
                "h2d_bytes_per_step": main_run["h2d_bytes_per_step"], "d2h_bytes_per_step": main_run["d2h_bytes_per_step"]},
        "gpu_launches": None,
        "clocks": clock_info,
    }
    if main_run.get("prefill_ms"):
        line["prefill"] = {"value": round(PREFILL_TOKENS * 1e3 / main_run["prefill_ms"], 1), "tokens": PREFILL_TOKENS,
                           "ms": round(main_run["prefill_ms"], 3),
                           "frac": round(prefill_flops(cfg, cfg["num_hidden_layers"], PREFILL_TOKENS)
                                         / (main_run["prefill_ms"] / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}
    if points:
        line["points"] = points
    if mixed:
        line["mixed"] = mixed
    print(json.dumps(line))
    return 0


def main() -> int:
    global MODEL, MODEL_NAME, CONTEXT
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--shape", default="0.6b", choices=sorted(SHAPES), help="layer sizes (default: the 0.6B shape)")
    parser.add_argument("--layers", type=int, default=0,
                        help="fewer layers than the configuration's, if memory or time needs it (reported)")
    parser.add_argument("--context", type=int, default=CONTEXT,
                        help="tokens a request holds when decoding ends (default: the baseline's context length)")
    parser.add_argument("--disable-cuda-graph", action="store_true")
    parser.add_argument("--skip-points", action="store_true", help="skip batch 1 / 64 and the prefill measurement")
    parser.add_argument("--pool-from-memory", action="store_true",
                        help="size the cache pool from the device's free memory (90 %%) instead of what the batch needs")
    parser.add_argument("--mixed", action="store_true",
                        help="also run the reference's serving workload (1 024-token prompts, 128 outputs, 8 and 32 requests "
                             "in flight) through the engine's continuous batching")
    args = parser.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    MODEL_NAME, MODEL = SHAPES[args.shape]
    if args.context != CONTEXT:
        CONTEXT = args.context
        MODEL = dict(MODEL, max_position_embeddings=max(CONTEXT, MODEL["max_position_embeddings"]))
    if args.layers <= 0:
        args.layers = MODEL["num_hidden_layers"]
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.steps + args.warmup + 40 >= CONTEXT:
        parser.error("steps + warmup must stay below the context length")

    import torch

    from cuinfer_b200.weights import write_random_model

    peaks = load_peaks()
    cfg = dict(MODEL, num_hidden_layers=args.layers)
    tmp = tempfile.mkdtemp(prefix="cuinfer_b200_bench_")
    try:
        # a recipe, not tensors: the engine draws the weights on the device while it loads (seed 0, N(0, 0.02), gains 1)
        write_random_model(tmp, cfg, seed=0, std=0.02, dtype="bfloat16", generator="counter", materialize=False)
        main_run = measure_decode(tmp, args.batch, args.steps, args.warmup, args, sample_clocks=True)
        points, prefill, mixed = {}, None, None
        if not args.skip_points:
            for b in (1, 64):
                r = measure_decode(tmp, b, min(args.steps, 128), args.warmup, args)
                points[f"decode_b{b}"] = round(r["tokens_per_s"], 1)
            for ctx in (2048, 3072):
                if ctx < CONTEXT:
                    r = measure_decode(tmp, args.batch, min(args.steps, 128), args.warmup, args, context=ctx)
                    points[f"decode_b{args.batch}_ctx{ctx}"] = round(r["tokens_per_s"], 1)
            if args.mixed:
                mixed = {f"in_flight_{c}": measure_generate(tmp, c, args) for c in (8, 32)}
            p = measure_prefill(tmp, args)
            flops = prefill_flops(cfg, args.layers, PREFILL_TOKENS)
            prefill = {"value": round(PREFILL_TOKENS / (p["ms"] / 1e3), 1), "tokens": PREFILL_TOKENS,
                       "ms": round(p["ms"], 3), "frac": round(flops / (p["ms"] / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}
    finally:
        shutil.rmtree(tmp, ignore_errors=True)

    step_bytes = weight_bytes(cfg, args.layers) + args.batch * main_run["context_mid"] * kv_bytes_per_token(cfg, args.layers)
    achieved = step_bytes / (main_run["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2048 tokens; % of roofline",
        "value": round(main_run["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02) seed 0, uniform-random token ids", "impl": "ours",
        "config": {
            "model": MODEL_NAME, "layers": args.layers,
            "layers_full": MODEL["num_hidden_layers"], "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "tied_embeddings": bool(cfg["tie_word_embeddings"]), "global_batch": args.batch, "seq_len": CONTEXT,
            "prompt_len": main_run["prompt_len"], "kv_block_size": BLOCK_SIZE, "parallelism": "single GPU",
            "cuda_graph": not args.disable_cuda_graph, "l2": "no flush: each step reads >1 GB, far more than the 126 MB L2",
            "peaks": peaks["source"],
        },
        "e2e": {"value": round(main_run["e2e_tokens_per_s"], 1), "unit": "tokens/s",
                "ms_per_step": round(main_run["e2e_ms_per_step"], 4),
                "h2d_bytes_per_step": main_run["h2d_bytes"], "d2h_bytes_per_step": main_run["d2h_bytes"]},
        "gpu_launches": main_run["launches"],
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
    }
    if prefill is not None:
        line["prefill"] = prefill
    if points:
        line["points"] = points
    if mixed:
        line["mixed"] = mixed
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
