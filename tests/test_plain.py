"""Spot checks of the plain implementation itself (CPU): each part against a case whose answer is known."""
from __future__ import annotations

import math

import torch

import plain_qwen3 as P
from conftest import TINY_A, TINY_B, random_tokens
from cuinfer_b200.weights import write_random_model


def test_rms_norm_of_a_constant_vector():
    x = torch.full((3, 8), 2.0)
    w = torch.arange(8, dtype=torch.float32)
    out = P.rms_norm(x, w, 1e-6)
    assert torch.allclose(out, w.expand(3, 8) * (2.0 / math.sqrt(4.0 + 1e-6)), atol=1e-6)


def test_rope_is_identity_at_position_zero_and_a_rotation_elsewhere():
    u = torch.randn(4, 2, 16)
    cos, sin = P.rope_cos_sin(10000.0, 16, torch.arange(4))
    out = P.apply_rope(u, cos, sin)
    assert torch.equal(out[0], u[0])
    assert torch.allclose(out.norm(dim=-1), u.norm(dim=-1), atol=1e-5)        # pairs are rotated, lengths kept
    # first pair (i = 0, f = 1): angle = position
    p = 3
    a, b = u[p, 0, 0], u[p, 0, 8]
    assert torch.allclose(out[p, 0, 0], a * math.cos(p) - b * math.sin(p), atol=1e-5)
    assert torch.allclose(out[p, 0, 8], b * math.cos(p) + a * math.sin(p), atol=1e-5)
    # relative property: <rope(q, m), rope(k, n)> depends on m - n only
    q, k = torch.randn(1, 1, 16), torch.randn(1, 1, 16)
    def dot(m, n):
        cm, sm = P.rope_cos_sin(10000.0, 16, torch.tensor([m]))
        cn, sn = P.rope_cos_sin(10000.0, 16, torch.tensor([n]))
        return (P.apply_rope(q, cm, sm) * P.apply_rope(k, cn, sn)).sum()
    assert torch.allclose(dot(5, 2), dot(9, 6), atol=1e-4)


def test_attention_first_token_returns_its_value_and_heads_share_kv():
    q, k, v = torch.randn(5, 4, 8), torch.randn(5, 2, 8), torch.randn(5, 2, 8)
    out = P.causal_attention(q, k, v, 8 ** -0.5)
    assert torch.allclose(out[0, 0], v[0, 0], atol=1e-6) and torch.allclose(out[0, 3], v[0, 1], atol=1e-6)
    # a key that dominates the scores pulls the output to its value
    k2 = k.clone()
    k2[2, 0] = q[4, 1] * 50
    out2 = P.causal_attention(q, k2, v, 8 ** -0.5)
    assert torch.allclose(out2[4, 1], v[2, 0], atol=1e-3)
    # window 2: position 4 sees keys 3 and 4 only
    out3 = P.causal_attention(q, k2, v, 8 ** -0.5, window=2)
    ref = torch.softmax((q[4, 1] @ k2[3:5, 0].T) * 8 ** -0.5, -1) @ v[3:5, 0]
    assert torch.allclose(out3[4, 1], ref, atol=1e-6)


def test_logits_at_a_position_do_not_depend_on_later_tokens(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_B, 3, std=0.05)
    cfg, w = P.load_folder(folder)
    ids = random_tokens(cfg["vocab_size"], 20, 1)
    full = P.forward(cfg, w, ids)
    assert torch.allclose(P.forward(cfg, w, ids[:11]), full[:11], atol=1e-5)
    assert full.shape == (20, 1000)


def test_tied_head_uses_the_embedding(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_A, 0)
    cfg, w = P.load_folder(folder)
    assert "lm_head.weight" not in w
    logits = P.forward(cfg, w, [1, 2, 3])
    w2 = dict(w)
    w2["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    assert torch.equal(P.forward(dict(cfg, tie_word_embeddings=False), w2, [1, 2, 3]), logits)


def test_plain_sampler():
    logits = torch.tensor([0.0, 3.0, 3.0, 1.0, -2.0])
    assert P.sample_plain(logits, 0.0, 0, 1.0, 0.7) == 1                  # greedy, lowest id on a tie
    assert P.sample_plain(logits, 1.0, 1, 1.0, 0.7) == 1
    draws = {P.sample_plain(logits, 1.0, 2, 1.0, u / 20) for u in range(20)}
    assert draws == {1, 2}                                                 # top-2 with a tie keeps both
    draws = {P.sample_plain(logits, 1.0, 0, 0.5, u / 20) for u in range(20)}
    assert draws == {1, 2}                                                 # the two ties are needed to reach 0.5
    draws = [P.sample_plain(logits, 1.0, 0, 1.0, u / 1000) for u in range(1000)]
    p = torch.softmax(logits, 0)
    for i in range(5):
        assert abs(draws.count(i) / 1000 - float(p[i])) < 0.01


def test_plain_agrees_with_the_reference_engine_golden_tokens(tmp_path):
    """tests/golden/reference_tokens.json holds greedy tokens that the UNMODIFIED reference engine generated on a
    B200 for a small random model (three layers of the Qwen3-0.6B widths, vocabulary 2 048; the script beside the file
    made it).  The same weights are rebuilt here (counter-based generator: the same bits on every machine) and the plain
    implementation is run over prompt + tokens: every token of the reference must be the plain implementation's best
    token at its place, or, where bfloat16 rounding can turn a near-tie, within a small margin of the best."""
    import json
    import os

    from cuinfer_b200.weights import write_random_model

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_tokens.json")
    golden = json.load(open(path))
    folder = write_random_model(str(tmp_path / "m"), golden["config"], **golden["weights"])
    cfg, weights = P.load_folder(folder)
    exact = total = 0
    for prompt, tokens in zip(golden["prompts"], golden["tokens"]):
        ids = list(prompt) + list(tokens)
        logits = P.forward(cfg, weights, ids[:-1])
        for j, tok in enumerate(tokens):
            row = logits[len(prompt) - 1 + j]
            total += 1
            exact += int(torch.argmax(row)) == tok
            assert float(row.max() - row[tok]) <= 0.03 * float(row.abs().max()), (len(prompt), j, tok, int(torch.argmax(row)))
    assert exact >= 0.9 * total, f"only {exact} of {total} tokens are the plain implementation's best"
