"""Host-side choices that need no GPU: how the decode attention's keys are split over CTAs, the uniform numbers of
sampling, the size limit of the L2 hints."""
from __future__ import annotations

import random

import torch

from cuinfer_b200 import kernels
from cuinfer_b200.sampling.sampler import uniform


def test_decode_splits_is_sane_for_every_shape():
    rnd = random.Random(0)
    for _ in range(400):
        requests = rnd.choice([1, 2, 3, 5, 8, 12, 17, 32, 64, 200])
        kv_heads = rnd.choice([1, 2, 4, 8, 16])
        keys = rnd.choice([1, 15, 64, 65, 500, 1024, 4096, 5000, 32768, 131072])
        for tma in (False, True):                               # the cache layout allows the TMA path or not
            s = kernels.decode_splits(requests, kv_heads, keys, tma=tma)
            assert 1 <= s <= 64
            if s > 1:
                share = -(-(-(-keys // s)) // 64) * 64        # keys per CTA, in steps of 64
                assert (s - 1) * share < keys                   # the last CTA still has keys to read
    # few (request, kv head) pairs and many keys: split; the GPU already full of pairs: do not
    assert kernels.decode_splits(1, 8, 4096) > 8 and kernels.decode_splits(8, 8, 4096) >= 2
    assert kernels.decode_splits(64, 8, 4096) == 1 and kernels.decode_splits(256, 8, 512) == 1
    assert kernels.decode_splits(1, 8, 16) == 1                 # one block of keys cannot be shared
    # 24 requests x 8 heads leave a third of the GPU free, but a second round of CTAs would cost more than it brings
    assert kernels.decode_splits(24, 8, 2048, tma=True) == 1 and kernels.decode_uses_tma(2048, 1)
    assert not kernels.decode_uses_tma(4096, 32)                # short streams per CTA stay on cp.async
    # more keys never mean fewer CTAs for the same batch
    for requests in (1, 2, 8):
        counts = [kernels.decode_splits(requests, 8, n) for n in (256, 1024, 4096, 16384)]
        assert counts == sorted(counts)


def test_uniform_numbers_depend_on_seed_request_and_index_only():
    seen = set()
    for seed in (0, 1, 12345):
        for key in (0, 7, 2 ** 40 + 3):
            for index in range(50):
                u = uniform(seed, key, index)
                assert 0.0 <= u < 1.0 and u == uniform(seed, key, index)
                assert u * (1 << 24) == int(u * (1 << 24))      # 24 random bits: exact in float32
                seen.add(u)
    assert len(seen) > 440                                      # 450 draws, (almost) all different
    draws = [uniform(3, 9, i) for i in range(4000)]
    assert 0.47 < sum(draws) / len(draws) < 0.53
    assert 0.22 < sum(d < 0.25 for d in draws) / len(draws) < 0.28


def test_l2_hints_are_given_for_small_weights_only():
    small = torch.empty(1024, 1024, dtype=torch.bfloat16)
    large = torch.empty(kernels.L2_HINT_MAX_BYTES // 2 + 8, dtype=torch.bfloat16)
    assert kernels._l2_hint(small) is small and kernels._l2_hint(large) is None and kernels._l2_hint(None) is None


def test_step_buckets_hold_their_batches_with_little_to_spare():
    """The sizes a step is padded to before it runs as a captured graph: never smaller than the batch, one request to
    spare for the spare tokens, at most an eighth (or 15) more tokens, and few distinct buckets."""
    from cuinfer_b200.engine.runner import ModelRunner

    rnd = random.Random(1)
    seen = set()
    for _ in range(3000):
        R = rnd.choice([1, 1, 2, 3, 8, 17, 33, 100, 255])
        lens = [rnd.choice([1, 1, 1, 2, 7, 60, 500, 2000]) for _ in range(R)]
        wants = [rnd.choice([0, 1, 1, 2]) for _ in range(R)]
        T, S = sum(lens), sum(wants)
        Tb, Rb, Sb = ModelRunner.step_bucket(lens, wants)
        assert T <= Tb <= max(T + 15, T + T // 8 + 1) and Tb % 16 == 0
        assert R < Rb <= 2 * R and Rb & (Rb - 1) == 0
        assert S <= Sb <= max(2 * S - 1, Rb if S else 0) and Sb & (Sb - 1) == 0
        seen.add(Tb)
    assert len(seen) < 120
    assert ModelRunner.step_bucket([2048], [1]) == (2048, 2, 2) and ModelRunner.step_bucket([8192], [1])[0] == 8192
