"""bfloat16 logits at the layer sizes the benchmark runs, as a composition: two-layer models with the widths of
the Qwen3-0.6B, 8B and 32B shapes (hidden 1024 / 4096 / 5120, 16-8 / 32-8 / 64-8 heads of 128, feed-forward 3072 /
12288 / 25600, vocabulary 151 936, tied / untied) through the replay path, against the plain implementation on the
CPU.  Fewer layers than the shapes have (2 of 28 / 36 / 64), not smaller layers: every projection, the attention
and the output head take the kernels that the dispatch rules choose at these sizes — the norm folded into the
few-rows projection up to K = 2048, the plain few-rows kernel at 4096, the weight-streaming kernel above, CTA-pair
tiles and the library product for prompt-sized steps, the 151 936-wide head — in the order a benchmark step runs them.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_qwen3
import traces
from conftest import GAINS, TOLERANCE, note_error, random_tokens

pytestmark = pytest.mark.gpu

VOCAB = 151936
SHAPES = {
    "0.6b": dict(hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, intermediate_size=3072,
                 tie_word_embeddings=True),
    "8b": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, intermediate_size=12288,
               tie_word_embeddings=False),
    "32b": dict(hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, intermediate_size=25600,
                tie_word_embeddings=False),
}


def _config(shape):
    return dict(architectures=["Qwen3ForCausalLM"], torch_dtype="bfloat16", hidden_act="silu", num_hidden_layers=2,
                head_dim=128, vocab_size=VOCAB, rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=1024,
                eos_token_id=1, **SHAPES[shape])


@pytest.mark.parametrize("shape", sorted(SHAPES))
def test_bfloat16_logits_at_real_layer_sizes(shape, tmp_path):
    from cuinfer_b200.weights import write_random_model

    cfg = _config(shape)
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=21, std=0.02, gain_std=0.1, dtype="bfloat16",
                                gains=GAINS["bfloat16"])
    pcfg, weights = plain_qwen3.load_folder(folder)
    lengths = [300, 150, 64, 200]
    requests = {f"r{i}": random_tokens(VOCAB, n, 2100 + i) for i, n in enumerate(lengths)}
    want_positions = {rid: sorted({0, 1, len(t) // 2 - 1, len(t) // 2, len(t) - 2, len(t) - 1}) for rid, t in requests.items()}
    steps = []
    # 1. the first request whole, logits wanted at a handful of places; then its last 16 tokens again one by one
    #    (as another request, so that the decode steps read pages written by a prompt-sized step)
    a = requests["r0"]
    steps.append({"step": 0, "entries": [{"id": "whole", "tokens": a, "want": want_positions["r0"]}], "end": ["whole"]})
    steps.append({"step": 1, "entries": [{"id": "tail", "tokens": a[:-16], "want": [len(a) - 17]}], "end": []})
    for j in range(16):
        steps.append({"step": 2 + j, "entries": [{"id": "tail", "tokens": [a[len(a) - 16 + j]], "want": [0]}],
                      "end": ["tail"] if j == 15 else []})
    # 2. one mixed step of four requests: a whole prompt, a portion that ends a prompt, two single decoded tokens
    s = len(steps)
    b, c, d = requests["r1"], requests["r2"], requests["r3"]
    steps.append({"step": s, "entries": [{"id": "b", "tokens": b[:100], "want": []}, {"id": "c", "tokens": c[:-1], "want": []},
                                         {"id": "d", "tokens": d[:-1], "want": []}], "end": []})
    steps.append({"step": s + 1, "entries": [{"id": "a2", "tokens": a[:120], "want": [0, 119]},
                                             {"id": "b", "tokens": b[100:], "want": [0, len(b) - 101]},
                                             {"id": "c", "tokens": c[-1:], "want": [0]},
                                             {"id": "d", "tokens": d[-1:], "want": [0]}], "end": ["a2", "b", "c", "d"]})
    out = str(tmp_path / "out")
    traces.replay_in_process(folder, "bfloat16", steps, out, traces.live_token_peak(steps), 16, cuda_graph=True)
    # collect by hand: request names differ from the token lists they replay
    source = {"whole": "r0", "tail": "r0", "a2": "r0", "b": "r1", "c": "r2", "d": "r3"}
    got = traces.collect(steps, out, VOCAB)
    worst = 0.0
    for name, rows in got.items():
        toks = requests[source[name]]
        places = sorted(rows)
        ref = plain_qwen3.logits_at(pcfg, weights, toks[:max(places) + 1], places).numpy()
        for place, want in zip(places, ref):
            assert np.isfinite(rows[place]).all()
            err = float(np.abs(rows[place] - want).max()) / float(np.abs(want).max())
            worst = max(worst, err)
            assert err <= TOLERANCE["bfloat16"], f"{shape}: request {name} position {place}: error {err:.3e}"
    note_error("bfloat16", f"real sizes {shape}", worst)
    print(f"\n[{shape}] largest bfloat16 error: {worst:.3e} of the largest logit")
