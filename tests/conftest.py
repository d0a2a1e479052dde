"""Shared test set-up: the ``gpu`` marker, the tiny configurations, model folders made in temporary
directories, and helpers that replay traces through the engine and compare with the plain implementation."""
from __future__ import annotations

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def _cfg(**kw):
    base = dict(architectures=["Qwen3ForCausalLM"], torch_dtype="float32", hidden_act="silu")
    base.update(kw)
    return base


# Three tiny configurations that differ in every size and option the architecture has.
TINY_A = _cfg(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=True, max_position_embeddings=512, eos_token_id=3)
TINY_B = _cfg(num_hidden_layers=3, hidden_size=96, num_attention_heads=8, num_key_value_heads=2, head_dim=32,
              intermediate_size=320, vocab_size=1000, rope_theta=1000000.0, rms_norm_eps=1e-5,
              tie_word_embeddings=False, max_position_embeddings=768, eos_token_id=[7, 9])
TINY_C = _cfg(num_hidden_layers=1, hidden_size=80, num_attention_heads=6, num_key_value_heads=3, head_dim=48,
              intermediate_size=176, vocab_size=517, rope_theta=500000.0, rms_norm_eps=3e-6,
              tie_word_embeddings=False, max_position_embeddings=1536)
# head size 128 with two query heads per kv head: the shape that the tensor-core attention kernels and, from 128 rows
# on, the tcgen05 projections take in bfloat16 (A, B and C run on the all-sizes kernels); the feed-forward is wider
# than 4096, so that its down projection takes the weight-streaming kernel in decode steps
TINY_D = _cfg(num_hidden_layers=2, hidden_size=192, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
              intermediate_size=4224, vocab_size=777, rope_theta=1000000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=True, max_position_embeddings=1024, eos_token_id=5)

TINY = {"A": (TINY_A, dict(seed=0, std=0.05, gain_std=0.0, block_size=16)),
        "B": (TINY_B, dict(seed=1, std=0.04, gain_std=0.1, block_size=32)),
        "C": (TINY_C, dict(seed=2, std=0.06, gain_std=0.2, block_size=16)),
        "D": (TINY_D, dict(seed=3, std=0.05, gain_std=0.1, block_size=16))}

# Largest |engine - plain| allowed, as a fraction of the largest |plain logit| of the sequence.
# float32: both sides compute in 32 bits; only the order of sums differs.
# bfloat16: engine and plain read the same bfloat16 weights; the engine rounds activations to bfloat16 where
# it stores them (normed rows, qkv, rotated q/k, attention output, projections, gate/up, their product).  A CPU
# emulation that rounds at exactly those places is off by up to 2.0e-2 on these models.
# Both bounds are 1.5 times the largest error that a full run of the gpu tests reports at its end (8.8e-6 and
# 2.1e-2); a run that comes near them is worth a look even when it passes.
TOLERANCE = {"float32": 1.4e-5, "bfloat16": 3.2e-2}

# Gains on the q/k norm weights spread the attention scores out, so that a wrong, missing or stale key changes
# the logits.  The 32-bit models are sharp (score spread ~4.5); the bfloat16 ones milder (spread ~2), because
# the rounding error of a score grows with its size.
GAINS = {"float32": {"q_norm": 3.0, "k_norm": 1.5}, "bfloat16": {"q_norm": 2.0, "k_norm": 1.0}}


# The largest error every comparison with the plain implementation saw, per dtype; printed at the end of a run, so
# that the bound can be kept close to what is measured.
WORST_ERRORS = {}


def note_error(dtype: str, where: str, err: float) -> None:
    if err > WORST_ERRORS.get(dtype, ("", -1.0))[1]:
        WORST_ERRORS[dtype] = (where, err)


def pytest_terminal_summary(terminalreporter):
    for dtype, (where, err) in sorted(WORST_ERRORS.items()):
        terminalreporter.write_line(f"largest {dtype} error against the plain implementation: {err:.3e} of the largest "
                                    f"logit ({where}); allowed {TOLERANCE[dtype]:.1e}")


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """{name: ({dtype: folder}, config dict, block_size)}.  The float32 folder stores float32 weights, the
    bfloat16 folder bfloat16 weights; the plain implementation reads the same folder as the engine."""
    from cuinfer_b200.weights import write_random_model

    out = {}
    for name, (cfg, opt) in TINY.items():
        folders = {}
        for dtype in ("float32", "bfloat16"):
            folder = str(tmp_path_factory.mktemp(f"tiny_{name}_{dtype}"))
            write_random_model(folder, cfg, opt["seed"], std=opt["std"], gain_std=opt["gain_std"], dtype=dtype,
                               gains=GAINS[dtype])
            folders[dtype] = folder
        out[name] = (folders, cfg, opt["block_size"])
    return out


def random_tokens(vocab: int, n: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
