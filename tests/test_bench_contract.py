"""What bench.py promises without a GPU: more than one GPU is refused with one line and exit code 2, the reference
arm prints its one JSON line and exits 0, and the byte and flop counts behind the roofline figures are what the
layer sizes say."""
from __future__ import annotations

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_more_than_one_gpu_is_refused_with_one_line():
    p = _run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert p.returncode == 2
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_prints_its_line():
    p = _run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert p.returncode == 0
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_bytes_and_flops_of_the_default_shape():
    import bench

    cfg, L = bench.MODEL, bench.MODEL["num_hidden_layers"]
    H, I, V, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["head_dim"]
    Q, KV = cfg["num_attention_heads"] * d, cfg["num_key_value_heads"] * d
    per_layer = H * (Q + 2 * KV) + Q * H + 3 * H * I + 2 * H + 2 * d
    assert bench.weight_bytes(cfg, L) == 2 * (L * per_layer + H + V * H)         # tied head: the table is read once
    assert bench.kv_bytes_per_token(cfg, L) == L * 2 * KV * 2                     # keys and values, bfloat16
    T = bench.PREFILL_TOKENS
    assert bench.prefill_flops(cfg, L, T) == 2.0 * T * L * (H * (Q + 2 * KV) + Q * H + 3 * H * I) + 2.0 * T * T * Q * L + 2.0 * V * H
    # the shapes the benchmark can be asked for are the baseline's, and the default is the 0.6B one
    assert bench.MODEL_NAME.startswith("Qwen3-0.6B") and set(bench.SHAPES) == {"0.6b", "8b", "32b"}
    assert (H, Q, KV, I, V, L) == (1024, 2048, 1024, 3072, 151936, 28) and bench.CONTEXT == 4096 and bench.BLOCK_SIZE == 16
