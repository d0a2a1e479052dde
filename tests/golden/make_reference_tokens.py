"""Makes tests/golden/reference_tokens.json: greedy tokens of the UNMODIFIED reference engine (typr7/cuInfer) on a small
random model, as an anchor for the plain implementation that does not rest on this repository's reading of the formulas.

The reference's model code exists only as CUDA kernels with fixed sizes (hidden 1024/2048, head size 128), so it cannot
be compared on the CPU or on the tiny configurations; it can be compiled offline and run on a GPU
(``baseline/build_reference.py``, ``baseline/reference_bench.cpp --mode generate``).  This script, run once on a B200,

    python tests/golden/make_reference_tokens.py

writes a three-layer model with the layer widths of the Qwen3-0.6B shape and a vocabulary of 2 048 (weights from the
counter-based generator, which gives the same bits on every machine), lets the reference generate 24 greedy tokens for
six prompts, and stores prompts and tokens.  ``tests/test_plain.py`` rebuilds the same weights on the CPU and checks that
every stored token is the plain implementation's best token, or within bfloat16 rounding of it.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline"))

CONFIG = dict(architectures=["Qwen3ForCausalLM"], torch_dtype="bfloat16", hidden_act="silu", num_hidden_layers=3,
              hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072,
              vocab_size=2048, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
              max_position_embeddings=512, eos_token_id=1)
WEIGHTS = dict(seed=77, std=0.05, gain_std=0.1, dtype="bfloat16", gains={"q_norm": 2.0}, generator="counter")
PROMPT_LENGTHS = [1, 7, 16, 33, 90, 200]
NEW_TOKENS = 24


def prompts():
    import torch
    g = torch.Generator().manual_seed(4242)
    return [torch.randint(0, CONFIG["vocab_size"], (n,), generator=g).tolist() for n in PROMPT_LENGTHS]


def main() -> int:
    import build_reference
    from cuinfer_b200.weights import write_random_model

    binary = build_reference.build()
    with tempfile.TemporaryDirectory() as tmp:
        folder = write_random_model(os.path.join(tmp, "model"), CONFIG, **WEIGHTS)
        prompt_file = os.path.join(tmp, "prompts.txt")
        with open(prompt_file, "w") as fh:
            for p in prompts():
                fh.write(" ".join(str(t) for t in p) + "\n")
        proc = subprocess.run([binary, "--mode", "generate", "--model", folder, "--prompts", prompt_file,
                               "--max-tokens", str(NEW_TOKENS), "--gpu-memory-utilization", "0.3"],
                              capture_output=True, text=True, timeout=1200)
        if proc.returncode != 0:
            print(proc.stderr[-2000:], file=sys.stderr)
            return 1
        tokens = [[int(t) for t in line.split()] for line in proc.stdout.strip().splitlines() if line and line[0].isdigit()]
    assert len(tokens) == len(PROMPT_LENGTHS) and all(len(t) == NEW_TOKENS for t in tokens), tokens
    out = dict(made_by="tests/golden/make_reference_tokens.py", engine="typr7/cuInfer, csrc unmodified, bfloat16, greedy",
               config=CONFIG, weights=WEIGHTS, prompts=prompts(), tokens=tokens)
    with open(os.path.join(HERE, "reference_tokens.json"), "w") as fh:
        json.dump(out, fh)
    print(f"wrote {len(tokens)} x {NEW_TOKENS} tokens")
    return 0


if __name__ == "__main__":
    sys.exit(main())
