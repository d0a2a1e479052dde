"""The entry point that allocates nothing: ``cib_paged_attention_decode_static``.

Some users of the kernel library cannot allocate device memory when they call it: a host program that has already
given all free device memory to the cache pool, or a C serving loop that must keep cudaMalloc/cudaFree (which
synchronise the whole device) out of its steps.  For them the split-key decode attention has a variant whose
scratch lives in a fixed ``__device__`` array inside the library.  This test calls that variant through its
exported C symbol, twice in a row with different inputs, and checks each result against the ordinary entry point
(``cib_paged_attention_decode`` with a torch-allocated scratch) within the tolerance of the kernel tests, one of
them also against a plain 32-bit attention on the CPU.  It checks what the entry point is for — the device's
free memory and torch's own allocation count are the same before and after a call — and that a call too large for
the built-in array is refused.  The file sorts last so that a run that stops at
the first failure has already run every other test.
"""
from __future__ import annotations

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
STATIC_SCRATCH_FLOATS = 2 * 1024 * 1024        # kStaticScratchFloats in attention_decode_static.h


def _entry(lib):
    fn = lib.cib_paged_attention_decode_static
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P, I, P, I, P, I, I, P, I, P, I, I, I, I, F, I, I, P]
    fn.restype = I
    return fn


def _call(fn, q, out, cache, bt, sl, nq, nkv, d, scale, window, splits):
    return fn(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), cache.data_ptr(), cache.shape[0], cache.shape[3],
              bt.data_ptr(), bt.stride(0), sl.data_ptr(), q.shape[0], nq, nkv, d, float(scale), int(window), int(splits),
              torch.cuda.current_stream().cuda_stream)


def test_static_scratch_entry_point_matches_the_allocating_one():
    from cuinfer_b200 import kernels
    from test_kernels_gpu import attention_case, attention_reference, close

    lib = kernels.library()
    fn = _entry(lib)
    # two calls in a row, different shapes: the second sees whatever the first left in the shared array
    for seed, (nq, nkv, d, ps, splits, lens) in enumerate([
        (16, 8, 128, 16, 5, [1, 17, 64, 333, 1000, 2, 129, 640]),
        (8, 2, 64, 32, 3, [700, 3, 96]),
        (4, 2, 256, 16, 1, [50, 301]),                 # one split: no partial results, head size 256
        (6, 3, 256, 16, 4, [1, 200, 77]),
    ]):
        case = attention_case(torch.bfloat16, nq, nkv, d, lens, [1] * len(lens), ps, seed=50 + seed, sharp=True)
        q, cache, bt = case["wide"].to(DEV), case["cache"].to(DEV), case["bt"].to(DEV)
        sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
        scale = 1.0 / math.sqrt(d)
        want = torch.empty(len(lens), nq * d, dtype=torch.bfloat16, device=DEV)
        kernels.paged_attention_decode(q, want, cache, bt, sl, nq, nkv, d, scale, 0, splits)
        got = torch.full_like(want, 3.0)
        # the first launch of a kernel may load its code onto the device; after it a call allocates nothing
        rc = _call(fn, q, got, cache, bt, sl, nq, nkv, d, scale, 0, splits)
        assert rc == 0, lib.cib_last_error().decode()
        got.fill_(3.0)
        torch.cuda.synchronize()
        free_before, allocated_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        rc = _call(fn, q, got, cache, bt, sl, nq, nkv, d, scale, 0, splits)
        assert rc == 0, lib.cib_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_allocated() == allocated_before
        close(got, want, 1.5e-2)
        assert torch.equal(got.cpu(), want.cpu())          # same kernel, same inputs: the very same bits
        if seed in (1, 2):  # and not only against itself: a plain 32-bit attention over the same cache
            close(got, attention_reference(case, lens, [1] * len(lens), scale), 1.5e-2)
    # a call beyond the built-in array is refused with a message, and nothing is written
    R, nq, nkv, d, splits = 64, 16, 8, 128, 17
    assert R * nq * splits * (d + 2) > STATIC_SCRATCH_FLOATS
    q = torch.zeros(R, (nq + 2 * nkv) * d, dtype=torch.bfloat16, device=DEV)
    out = torch.full((R, nq * d), 3.0, dtype=torch.bfloat16, device=DEV)
    cache = torch.zeros(4, 2, nkv, 16, d, dtype=torch.bfloat16, device=DEV)
    bt = torch.zeros(R, 2, dtype=torch.int32, device=DEV)
    sl = torch.ones(R, dtype=torch.int32, device=DEV)
    rc = _call(fn, q, out, cache, bt, sl, nq, nkv, d, 1.0, 0, splits)
    assert rc != 0
    msg = lib.cib_last_error().decode()
    assert "built-in array holds" in msg and "floats of scratch" in msg
    torch.cuda.synchronize()
    assert float(out.float().min()) == 3.0
