"""Each CUDA kernel alone against a plain 32-bit reference of the same op, at sizes other than the engine's."""
from __future__ import annotations

import math
import random

import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _k():
    from cuinfer_b200 import kernels
    return kernels


def rand(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def close(got, want, tol):
    got, want = got.float().cpu(), want.float().cpu()
    err = float((got - want).abs().max()) / max(1e-12, float(want.abs().max()))
    assert err <= tol, f"error {err:.3e} of the largest value, allowed {tol:.1e}"


TOL = {torch.float32: 2e-6, torch.bfloat16: 1.2e-2}


# ---- embedding, norm, gather, silu ------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V, H", [(517, 80), (1000, 1027), (64, 4096)])
def test_embedding_gather(dtype, V, H):
    k = _k()
    table = rand(V, H, seed=1, dtype=dtype).to(DEV)
    ids = torch.tensor([0, V - 1, 3, 3, V // 2], dtype=torch.int32, device=DEV)
    out = torch.empty(5, H, dtype=torch.float32, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    k.embedding_gather(ids, table, out, flag)
    assert torch.equal(out.cpu(), table.float().cpu()[ids.cpu().long()]) and int(flag.item()) == 0
    bad = torch.tensor([1, V], dtype=torch.int32, device=DEV)
    out2 = torch.ones(2, H, dtype=torch.float32, device=DEV)
    k.embedding_gather(bad, table, out2, flag)
    assert int(flag.item()) == 1 and float(out2[1].abs().max()) == 0.0        # out of range: zeros and a flag, no fault


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [80, 1027, 5120])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(dtype, H, wdtype):
    k = _k()
    if dtype == torch.float32 and wdtype == torch.bfloat16:
        pytest.skip("a 32-bit engine holds 32-bit gains")
    rows = 7
    res = rand(rows, H, seed=2, scale=3.0)
    delta = rand(rows, H, seed=3, dtype=dtype)
    w = (1 + rand(H, seed=4, scale=0.2)).to(wdtype)
    eps = 3e-5
    r_dev = res.clone().to(DEV)
    out = torch.empty(rows, H, dtype=dtype, device=DEV)
    k.add_rmsnorm(r_dev, delta.to(DEV), w.to(DEV), eps, out)
    x = res + delta.float()
    close(r_dev, x, 1e-7)
    close(out, P.rms_norm(x, w.float(), eps), TOL[dtype])
    # without a delta the residual is untouched
    r2 = res.clone().to(DEV)
    k.add_rmsnorm(r2, None, w.to(DEV), eps, out)
    assert torch.equal(r2.cpu(), res)
    close(out, P.rms_norm(res, w.float(), eps), TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,H", [(256, 72), (301, 1000), (259, 1024), (257, 2048), (300, 2052)])
def test_add_rmsnorm_many_rows(dtype, rows, H):
    """From 256 rows on a warp takes a whole row (up to 2048 values; wider rows stay with the block kernel): widths
    that do not fill the lanes, a last block with idle warps, and the add-only and norm-only forms."""
    k = _k()
    res = rand(rows, H, seed=12, scale=3.0)
    delta = rand(rows, H, seed=13, dtype=dtype)
    w = (1 + rand(H, seed=14, scale=0.2)).to(dtype)
    r_dev = res.clone().to(DEV)
    out = torch.full((rows, H), float("nan"), dtype=dtype, device=DEV)
    k.add_rmsnorm(r_dev, delta.to(DEV), w.to(DEV), 2e-6, out)
    x = res + delta.float()
    close(r_dev, x, 1e-7)
    close(out, P.rms_norm(x, w.float(), 2e-6), TOL[dtype])
    r2 = res.clone().to(DEV)
    k.add_rmsnorm(r2, None, w.to(DEV), 2e-6, out)                  # norm only
    assert torch.equal(r2.cpu(), res)
    close(out, P.rms_norm(res, w.float(), 2e-6), TOL[dtype])
    k.add_rmsnorm(r2, delta.to(DEV), None, 2e-6, None)              # add only
    close(r2, x, 1e-7)


def test_gather_rows():
    k = _k()
    res, delta = rand(9, 83, seed=5), rand(9, 83, seed=6, dtype=torch.bfloat16)
    idx = torch.tensor([8, 0, 4, 4], dtype=torch.int32)
    out = torch.empty(4, 83, dtype=torch.float32, device=DEV)
    k.gather_rows(res.to(DEV), delta.to(DEV), idx.to(DEV), out)
    close(out, (res + delta.float())[idx.long()], 1e-7)
    k.gather_rows(res.to(DEV), None, idx.to(DEV), out)
    assert torch.equal(out.cpu(), res[idx.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("I", [176, 333, 3072])
def test_silu_mul(dtype, I):
    k = _k()
    gu = rand(5, 2 * I, seed=7, scale=3.0, dtype=dtype)
    out = torch.empty(5, I, dtype=dtype, device=DEV)
    k.silu_mul(gu.to(DEV), out)
    g, u = gu.float()[:, :I], gu.float()[:, I:]
    close(out, g / (1 + torch.exp(-g)) * u, TOL[dtype])


# ---- matrix product ---------------------------------------------------------------------------------------

@pytest.mark.parametrize("M, N, K", [(1, 1000, 96), (7, 517, 80), (65, 130, 33), (200, 64, 1027)])
@pytest.mark.parametrize("dtypes", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                    (torch.bfloat16, torch.float32)])
def test_gemm_generic(M, N, K, dtypes):
    k = _k()
    din, dout = dtypes
    a, w = rand(M, K, seed=8, dtype=din), rand(N, K, seed=9, dtype=din)
    out = torch.empty(M, N, dtype=dout, device=DEV)
    k.gemm_generic(a.to(DEV), w.to(DEV), out)
    want = a.double() @ w.double().T
    close(out, want, 1e-5 if dout == torch.float32 else 6e-3)
    # a row's result does not depend on the rows beside it
    one = torch.empty(1, N, dtype=dout, device=DEV)
    k.gemm_generic(a[M // 2:M // 2 + 1].to(DEV), w.to(DEV), one)
    assert torch.equal(one[0].cpu(), out[M // 2].cpu())


@pytest.mark.parametrize("M, N, K", [(128, 128, 64), (128, 256, 128), (17, 1000, 96), (300, 517 + 3, 72),
                                     (2048, 4096, 1024), (640, 1024, 3072), (129, 6144, 1024), (200, 136, 2048)])
@pytest.mark.parametrize("f32_out", [False, True])
def test_gemm_tcgen05(M, N, K, f32_out):
    k = _k()
    assert k.gemm_tcgen05_supports(M, N, K)
    a, w = rand(M, K, seed=21, dtype=torch.bfloat16), rand(N, K, seed=22, scale=0.05, dtype=torch.bfloat16)
    out = torch.full((M, N), 7.0, dtype=torch.float32 if f32_out else torch.bfloat16, device=DEV)
    k.gemm_tcgen05(a.to(DEV), w.to(DEV), out)
    k.check_error_flags()
    want = a.to(DEV).double() @ w.to(DEV).double().T
    close(out, want, 2e-5 if f32_out else 6e-3)
    # rows strided inside a wider buffer (a packed row), and a second call on the same stream
    wide = torch.zeros(M, K + 64, dtype=torch.bfloat16, device=DEV)
    wide[:, :K] = a.to(DEV)
    out2 = torch.empty_like(out)
    k.gemm_tcgen05(wide[:, :K], w.to(DEV), out2)
    k.check_error_flags()
    assert torch.equal(out2.cpu(), out.cpu())


@pytest.mark.parametrize("M, I, K", [(128, 128, 64), (300, 3072, 1024), (2048, 200, 136), (129, 1000, 72), (513, 64, 2048)])
def test_gemm_tcgen05_gated(M, I, K):
    """Gate rows and up rows in one tile, silu(gate) * up from the 32-bit accumulators: widths that end inside a
    tile, and rows that end inside one."""
    k = _k()
    a = rand(M, K, seed=23, dtype=torch.bfloat16)
    w = rand(2 * I, K, seed=24, scale=0.08, dtype=torch.bfloat16)
    out = torch.full((M, I), 7.0, dtype=torch.bfloat16, device=DEV)
    k.gemm_tcgen05(a.to(DEV), w.to(DEV), out, silu_pair=True)
    k.check_error_flags()
    y = a.double() @ w.double().T
    want = torch.nn.functional.silu(y[:, :I]) * y[:, I:]
    close(out, want, 6e-3)
    # as part of a wider buffer, the columns beside it stay as they were
    wide = torch.full((M, I + 24), 7.0, dtype=torch.bfloat16, device=DEV)
    k.gemm_tcgen05(a.to(DEV), w.to(DEV), wide[:, :I], silu_pair=True)
    k.check_error_flags()
    assert torch.equal(wide[:, :I].cpu(), out.cpu()) and bool((wide[:, I:] == 7.0).all())


@pytest.mark.parametrize("M", [1, 8, 16, 17, 40, 64, 100, 128])
@pytest.mark.parametrize("N, K", [(1024, 1024), (136, 72), (4096, 4096), (1000, 2048), (256, 12288)])
@pytest.mark.parametrize("f32_out", [False, True])
def test_gemm_wstream(M, N, K, f32_out):
    """Weights as the streamed tensor-core operand: every row-count class, feature counts that end inside a tile,
    K that ends inside a step, and shapes whose K is split over a cluster (few tiles, long K)."""
    k = _k()
    assert k.gemm_wstream_supports(M, N, K)
    a, w = rand(M, K, seed=25, dtype=torch.bfloat16), rand(N, K, seed=26, scale=0.05, dtype=torch.bfloat16)
    out = torch.full((M, N), 7.0, dtype=torch.float32 if f32_out else torch.bfloat16, device=DEV)
    for _ in range(2):
        k.gemm_wstream(a.to(DEV), w.to(DEV), out)
        k.check_error_flags()
    want = a.double() @ w.double().T
    close(out, want, 2e-5 if f32_out else 6e-3)
    assert not k.gemm_wstream_supports(129, N, K) and not k.gemm_wstream_supports(M, N, 20)


@pytest.mark.parametrize("M", [3, 16, 33, 128])
@pytest.mark.parametrize("I, K", [(3072, 1024), (200, 136), (64, 4096), (1000, 72)])
def test_gemm_wstream_gated(M, I, K):
    k = _k()
    a = rand(M, K, seed=27, dtype=torch.bfloat16)
    w = rand(2 * I, K, seed=28, scale=0.08, dtype=torch.bfloat16)
    wide = torch.full((M, I + 8), 7.0, dtype=torch.bfloat16, device=DEV)
    k.gemm_wstream(a.to(DEV), w.to(DEV), wide[:, :I], silu_pair=True)
    k.check_error_flags()
    y = a.double() @ w.double().T
    close(wide[:, :I], torch.nn.functional.silu(y[:, :I]) * y[:, I:], 6e-3)
    assert bool((wide[:, I:] == 7.0).all())


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N, K", [(1024, 1024), (48, 96), (1000, 2048), (3000, 72), (151936, 1024)])
def test_gemm_skinny(M, N, K):
    k = _k()
    assert k.gemm_skinny_supports(M, N, K)
    a, w = rand(M, K, seed=13, dtype=torch.bfloat16), rand(N, K, seed=14, scale=0.05, dtype=torch.bfloat16)
    want = a.double() @ w.double().T
    wd, ad = w.to(DEV), a.to(DEV)
    for dtype, tol in ((torch.bfloat16, 6e-3), (torch.float32, 2e-5)):
        out = torch.full((M, N), 7.0, dtype=dtype, device=DEV)
        k.gemm_skinny(wd, out, act=ad)
        close(out, want, tol)
    # a row's result does not depend on how many rows are beside it
    one = torch.empty(1, N, dtype=torch.float32, device=DEV)
    k.gemm_skinny(wd, one, act=ad[M - 1:M])
    full = torch.empty(M, N, dtype=torch.float32, device=DEV)
    k.gemm_skinny(wd, full, act=ad)
    assert torch.equal(one[0].cpu(), full[M - 1].cpu())


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("H, I", [(1024, 3072), (96, 320), (80, 176)])
@pytest.mark.parametrize("pending_dtype", [None, torch.bfloat16, torch.float32])
def test_gemm_skinny_with_norm_and_gated_epilogue(M, H, I, pending_dtype):
    k = _k()
    if not k.gemm_skinny_supports(M, 2 * I, H, True):
        pytest.skip("shape not taken")
    res = rand(M, H, seed=15, scale=2.0)
    pend = None if pending_dtype is None else rand(M, H, seed=16, dtype=pending_dtype)
    gain = (1 + rand(H, seed=17, scale=0.2)).to(torch.bfloat16)
    w = rand(2 * I, H, seed=18, scale=0.05, dtype=torch.bfloat16)
    eps = 1e-5
    x = res + (pend.float() if pend is not None else 0)
    normed = P.rms_norm(x, gain.float(), eps).to(torch.bfloat16).float()
    gu = normed.double() @ w.double().T
    # norm prologue, plain store
    res_out = torch.zeros(M, H, dtype=torch.float32, device=DEV)
    out = torch.empty(M, 2 * I, dtype=torch.bfloat16, device=DEV)
    k.gemm_skinny(w.to(DEV), out, residual=res.to(DEV), pending=pend.to(DEV) if pend is not None else None,
                  norm_weight=gain.to(DEV), eps=eps, residual_out=res_out)
    close(out, gu, 8e-3)
    close(res_out, x, 1e-7)
    # norm prologue and gated epilogue together
    act = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    k.gemm_skinny(w.to(DEV), act, residual=res.to(DEV), pending=pend.to(DEV) if pend is not None else None,
                  norm_weight=gain.to(DEV), eps=eps, residual_out=res_out, silu_pair=True)
    g, u = gu[:, :I], gu[:, I:]
    close(act, g / (1 + torch.exp(-g)) * u, 1e-2)
    # gated epilogue on plain activations
    act2 = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    k.gemm_skinny(w.to(DEV), act2, act=normed.to(torch.bfloat16).to(DEV), silu_pair=True)
    close(act2, g / (1 + torch.exp(-g)) * u, 1e-2)


def test_gemm_skinny_refuses_other_shapes():
    k = _k()
    assert not k.gemm_skinny_supports(17, 64, 64) and not k.gemm_skinny_supports(4, 64, 60)
    assert not k.gemm_skinny_supports(16, 64, 16384) and not k.gemm_skinny_supports(16, 64, 4096, True)
    with pytest.raises(k.KernelError, match="not taken"):
        k.gemm_skinny(torch.zeros(64, 60, dtype=torch.bfloat16, device=DEV), torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV),
                      act=torch.zeros(4, 60, dtype=torch.bfloat16, device=DEV))


# ---- q/k norm + rotary + cache write ------------------------------------------------------------------------

def paged_cache(k_dense, v_dense, page_size, num_pages, seed, dtype, poison=False):
    """Scatter per-request dense [n, nkv, d] keys/values into shuffled pages.
    Returns (cache [pages, 2, nkv, ps, d], tables list, slot list per request)."""
    g = torch.Generator().manual_seed(seed)
    nkv, d = k_dense[0].shape[1:]
    cache = (torch.randn(num_pages, 2, nkv, page_size, d, generator=g) * 50).to(dtype)   # stale garbage everywhere
    if poison:
        cache.fill_(float("nan"))         # slots that hold no token of a request must never reach a result
    order = torch.randperm(num_pages, generator=g).tolist()
    tables = []
    for kd, vd in zip(k_dense, v_dense):
        n = kd.shape[0]
        pages = [order.pop() for _ in range((n + page_size - 1) // page_size)]
        tables.append(pages)
        for j in range(n):
            cache[pages[j // page_size], 0, :, j % page_size] = kd[j].to(dtype)
            cache[pages[j // page_size], 1, :, j % page_size] = vd[j].to(dtype)
    return cache, tables


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq, nkv, d, rot", [(6, 3, 48, 48), (4, 1, 80, 32), (16, 8, 128, 128), (2, 2, 16, 0)])
def test_qk_norm_rope_kv_write(dtype, nq, nkv, d, rot):
    k = _k()
    T, ps, pages = 11, 4, 9
    width = (nq + 2 * nkv) * d
    qkv = rand(T, width, seed=10, dtype=dtype)
    positions = torch.tensor([0, 1, 2, 3, 4, 5, 17, 18, 40, 41, 42], dtype=torch.int32)
    slots = torch.tensor([4, 5, 6, 7, 8, 9, 30, 31, 0, 1, -1], dtype=torch.int32)     # the last token is padding
    qw, kw = 1 + rand(d, seed=11, scale=0.3), 1 + rand(d, seed=12, scale=0.3)
    eps, theta = 2e-5, 12345.0
    table = None
    if rot:
        half = rot // 2
        inv = 1.0 / torch.pow(torch.tensor(theta), torch.arange(half, dtype=torch.float32) * 2.0 / rot)
        ang = torch.arange(64, dtype=torch.float32)[:, None] * inv[None, :]
        table = torch.stack((torch.cos(ang), torch.sin(ang)), -1).contiguous().to(DEV)
    cache = torch.full((pages, 2, nkv, ps, d), 7.0, dtype=dtype, device=DEV)
    dev = qkv.clone().to(DEV)
    k.qk_norm_rope_kv_write(dev, positions.to(DEV), slots.to(DEV), qw.to(DEV), kw.to(DEV), eps, table, rot, cache,
                            nq, nkv, d)
    x = qkv.float()
    q = P.rms_norm(x[:, :nq * d].view(T, nq, d), qw, eps)
    kk = P.rms_norm(x[:, nq * d:(nq + nkv) * d].view(T, nkv, d), kw, eps)
    v = x[:, (nq + nkv) * d:].view(T, nkv, d)
    if rot:
        cos, sin = P.rope_cos_sin(theta, rot, positions)
        q, kk = P.apply_rope(q, cos, sin), P.apply_rope(kk, cos, sin)
    close(dev[:, :nq * d], q.reshape(T, -1), TOL[dtype])
    assert torch.equal(dev[:, nq * d:].cpu(), qkv[:, nq * d:])                       # k and v columns are left alone
    got = cache.float().cpu()
    touched = torch.zeros(pages, ps, dtype=torch.bool)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        touched[s // ps, s % ps] = True
        close(got[s // ps, 0, :, s % ps], kk[t], TOL[dtype])
        close(got[s // ps, 1, :, s % ps], v[t], TOL[dtype] if dtype == torch.bfloat16 else 0.0)
    mask = touched[:, None, None, :, None].expand_as(got)
    assert bool((got[~mask] == 7.0).all())                                           # nothing else was written
    # without norm weights and without a cache: queries are only rotated
    dev2 = qkv.clone().to(DEV)
    k.qk_norm_rope_kv_write(dev2, positions.to(DEV), None, None, None, eps, table, rot, None, nq, nkv, d)
    q2 = x[:, :nq * d].view(T, nq, d)
    if rot:
        q2 = P.apply_rope(q2, cos, sin)
    close(dev2[:, :nq * d], q2.reshape(T, -1), TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq, nkv, d, rot", [(16, 8, 128, 128), (5, 1, 64, 64), (3, 3, 256, 0), (6, 2, 96, 96), (7, 7, 256, 256)])
def test_qk_norm_rope_kv_write_many_tokens(dtype, nq, nkv, d, rot):
    """From a few hundred tokens on another kernel takes several heads per warp (for head sizes 64, 128, 256): it must
    give what the same call gives when it is cut into small pieces, which the test above checks against the plain
    formulas (the sums of squares are added in another order, so the last bit may differ)."""
    k = _k()
    T, ps = 700, 16
    pages = (T + ps - 1) // ps + 2
    qkv = rand(T, (nq + 2 * nkv) * d, seed=14, dtype=dtype).to(DEV)
    g = torch.Generator().manual_seed(15)
    positions = torch.randint(0, 900, (T,), generator=g, dtype=torch.int32).to(DEV)
    slots = torch.randperm(pages * ps, generator=g)[:T].to(torch.int32)
    slots[::37] = -1
    slots = slots.to(DEV)
    qw, kw = (1 + rand(d, seed=16, scale=0.3)).to(DEV), (1 + rand(d, seed=17, scale=0.3)).to(DEV)
    table = None
    if rot:
        inv = 1.0 / torch.pow(torch.tensor(10000.0), torch.arange(rot // 2, dtype=torch.float32) * 2.0 / rot)
        ang = torch.arange(900, dtype=torch.float32)[:, None] * inv[None, :]
        table = torch.stack((torch.cos(ang), torch.sin(ang)), -1).contiguous().to(DEV)
    whole, cache_w = qkv.clone(), torch.full((pages, 2, nkv, ps, d), 7.0, dtype=dtype, device=DEV)
    k.qk_norm_rope_kv_write(whole, positions, slots, qw, kw, 1e-6, table, rot, cache_w, nq, nkv, d)
    pieces, cache_p = qkv.clone(), torch.full((pages, 2, nkv, ps, d), 7.0, dtype=dtype, device=DEV)
    for a in range(0, T, 100):
        k.qk_norm_rope_kv_write(pieces[a:a + 100], positions[a:a + 100], slots[a:a + 100], qw, kw, 1e-6, table, rot,
                                cache_p, nq, nkv, d)
    close(whole, pieces.float().cpu(), TOL[dtype])
    close(cache_w, cache_p.float().cpu(), TOL[dtype])
    assert torch.equal(whole[:, nq * d:].cpu(), qkv[:, nq * d:].cpu())               # k and v columns are left alone
    assert not torch.equal(whole.cpu(), qkv.cpu())


# ---- attention --------------------------------------------------------------------------------------------------

def attention_case(dtype, nq, nkv, d, lens, new, page_size, seed, sharp=False, poison=False):
    """Requests with ``lens`` tokens in the cache, the last ``new`` of them being this step's queries."""
    g = torch.Generator().manual_seed(seed)
    ks, vs, qs = [], [], []
    for n, m in zip(lens, new):
        kd = torch.randn(n, nkv, d, generator=g)
        vd = torch.randn(n, nkv, d, generator=g)
        qd = torch.randn(m, nq, d, generator=g)
        if sharp and n > 3:
            # one far key per query head dominates: its value must come through almost alone
            far = 1 if n < 40 else n // 7
            for a in range(nq):
                kd[far, a // (nq // nkv)] = qd[-1, a] / qd[-1, a].norm() * 6.0 * math.sqrt(d) / (nq // nkv + 1) * (a % (nq // nkv) + 1)
        ks.append(kd.to(dtype).float()); vs.append(vd.to(dtype).float()); qs.append(qd.to(dtype).float())
    pages = sum((n + page_size - 1) // page_size for n in lens) + 3
    cache, tables = paged_cache(ks, vs, page_size, pages, seed + 1, dtype, poison)
    stride = max(len(t) for t in tables) + 2
    bt = torch.full((len(lens), stride), -1, dtype=torch.int32)
    for r, t in enumerate(tables):
        bt[r, :len(t)] = torch.tensor(t, dtype=torch.int32)
    q_rows = torch.cat([q.reshape(q.shape[0], -1) for q in qs], 0)
    # queries sit in the first nq*d columns of a wider row, as in a packed qkv row
    wide = torch.cat([q_rows, torch.full((q_rows.shape[0], 2 * nkv * d), 99.0)], 1).to(dtype)
    qsl = [0]
    for m in new:
        qsl.append(qsl[-1] + m)
    treq = [r for r, m in enumerate(new) for _ in range(m)]
    return dict(ks=ks, vs=vs, qs=qs, cache=cache, bt=bt, wide=wide, qsl=qsl, treq=treq)


def attention_reference(case, lens, new, scale, window=None):
    outs = []
    for kd, vd, qd, n, m in zip(case["ks"], case["vs"], case["qs"], lens, new):
        full_q = torch.zeros(n, qd.shape[1], qd.shape[2])
        full_q[n - m:] = qd
        outs.append(P.causal_attention(full_q, kd, vd, scale, window)[n - m:].reshape(m, -1))
    return torch.cat(outs, 0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq, nkv, d, ps", [(6, 3, 48, 16), (4, 1, 80, 5), (8, 2, 128, 32), (3, 3, 16, 1)])
@pytest.mark.parametrize("window", [None, 9])
def test_paged_attention_generic(dtype, nq, nkv, d, ps, window):
    k = _k()
    lens, new = [1, 37, 64, 130, 5], [1, 37, 1, 17, 2]
    case = attention_case(dtype, nq, nkv, d, lens, new, ps, seed=20, sharp=True)
    scale = 0.7 / math.sqrt(d)
    T = sum(new)
    out = torch.empty(T, nq * d, dtype=dtype, device=DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    k.paged_attention_generic(case["wide"].to(DEV), out, case["cache"].to(DEV), case["bt"].to(DEV), i32(case["qsl"]),
                              i32(lens), i32(case["treq"]), nq, nkv, d, scale, window or 0)
    close(out, attention_reference(case, lens, new, scale, window), 2e-5 if dtype == torch.float32 else 1.5e-2)


@pytest.mark.parametrize("nq, nkv, d, ps", [(16, 8, 128, 16), (8, 1, 64, 32), (12, 3, 128, 5), (32, 2, 256, 16),
                                            (4, 4, 64, 16)])
@pytest.mark.parametrize("splits", [1, 3, 8])
@pytest.mark.parametrize("window", [None, 50])
def test_paged_attention_decode(nq, nkv, d, ps, splits, window):
    k = _k()
    assert k.paged_attention_decode_supports(d, nq, nkv)
    lens = [1, 2, 15, 16, 17, 64, 333, 1000]
    new = [1] * len(lens)
    # slots that hold no token are NaN: pages that come whole (the TMA path, pages of 16, 32, ... slots without a
    # window) must not let them through
    case = attention_case(torch.bfloat16, nq, nkv, d, lens, new, ps, seed=30, sharp=True, poison=True)
    scale = 1.0 / math.sqrt(d)
    out = torch.full((len(lens), nq * d), 5.0, dtype=torch.bfloat16, device=DEV)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    cache, bt, wide = case["cache"].to(DEV), case["bt"].to(DEV), case["wide"].to(DEV)
    want = attention_reference(case, lens, new, scale, window)
    for tma in (None, False, None):        # both ways of fetching the cache; again: the split counters must be left at zero
        out.fill_(5.0)
        k.paged_attention_decode(wide, out, cache, bt, sl, nq, nkv, d, scale, window or 0, splits, tma=tma)
        k.check_error_flags()
        close(out, want, 1.5e-2)
    # the all-sizes kernel agrees on the same inputs
    gen = torch.empty_like(out)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    k.paged_attention_generic(wide, gen, cache, bt, i32(case["qsl"]), sl, i32(case["treq"]), nq, nkv, d, scale, window or 0)
    close(out, gen, 1.5e-2)


@pytest.mark.parametrize("nq, nkv, d, ps", [(16, 8, 128, 16), (8, 1, 64, 32), (12, 4, 128, 5), (6, 6, 64, 16)])
@pytest.mark.parametrize("window", [None, 40])
def test_paged_attention_prefill(nq, nkv, d, ps, window):
    """Portions of every length beside decoded tokens: tiles that end inside a request, cross the diagonal,
    start at a late position, and a far key that dominates."""
    k = _k()
    assert k.paged_attention_prefill_supports(d, nq, nkv)
    lens = [1, 37, 64, 130, 5, 300, 257, 1000]
    new = [1, 37, 1, 17, 2, 300, 129, 1]
    case = attention_case(torch.bfloat16, nq, nkv, d, lens, new, ps, seed=60, sharp=True)
    scale = 1.0 / math.sqrt(d)
    T = sum(new)
    out = torch.full((T, nq * d), 5.0, dtype=torch.bfloat16, device=DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    k.paged_attention_prefill(case["wide"].to(DEV), out, case["cache"].to(DEV), case["bt"].to(DEV), i32(case["qsl"]),
                              i32(lens), new, nq, nkv, d, scale, window or 0)
    close(out, attention_reference(case, lens, new, scale, window), 1.5e-2)


@pytest.mark.parametrize("nq, nkv, ps", [(16, 8, 16), (8, 1, 32), (4, 4, 8), (32, 2, 128), (2, 1, 256)])
@pytest.mark.parametrize("window", [None, 200])
def test_attention_tcgen05(nq, nkv, ps, window):
    """The tensor-memory attention kernel on portions of every length beside decoded tokens; cache slots that hold no
    token are NaN."""
    k = _k()
    d = 128
    assert k.attention_tcgen05_supports(d, nq, nkv, ps)
    lens = [1, 37, 64, 130, 5, 300, 257, 1000, 128, 640]
    new = [1, 37, 1, 17, 2, 300, 129, 1, 128, 513]
    case = attention_case(torch.bfloat16, nq, nkv, d, lens, new, ps, seed=80, sharp=True, poison=True)
    scale = 1.0 / math.sqrt(d)
    T = sum(new)
    out = torch.full((T, nq * d), 5.0, dtype=torch.bfloat16, device=DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    for _ in range(2):
        k.attention_tcgen05(case["wide"].to(DEV), out, case["cache"].to(DEV), case["bt"].to(DEV), i32(case["qsl"]),
                            i32(lens), new, nq, nkv, d, scale, window or 0)
        k.check_error_flags()
    close(out, attention_reference(case, lens, new, scale, window), 1.5e-2)
    assert not k.attention_tcgen05_supports(64, 8, 8, 16) and not k.attention_tcgen05_supports(128, 12, 4, 16)
    assert not k.attention_tcgen05_supports(128, 8, 8, 5) and not k.attention_tcgen05_supports(128, 8, 8, 4)


@pytest.mark.parametrize("seed", [1, 2])
def test_attention_tcgen05_random_batches(seed):
    """Drawn batches: 1 to 70 requests (more than the 32 that one pass of the request search takes), portions of 1 to
    513 tokens after 0 to 1 100 cached ones, every page size and ratio of heads the kernel takes, with and without a
    window, the same launch three times over."""
    k = _k()
    d = 128
    rnd = random.Random(seed)
    for it in range(8):
        nq, nkv = rnd.choice([(16, 8), (32, 8), (8, 8), (16, 2), (32, 2), (4, 1), (64, 8)])
        ps = rnd.choice([8, 16, 32, 64, 128, 256])
        requests = rnd.choice([1, 2, 3, 5, 9, 33, 40, 70])
        new = [rnd.choice([1, 1, 2, 3, 17, 63, 64, 65, 127, 128, 129, 200, 300, 513]) for _ in range(requests)]
        if requests > 20:
            new = [min(n, 70) for n in new]
        lens = [n + rnd.choice([0, 0, 1, 15, 16, 100, 127, 128, 500, 1100]) for n in new]
        window = rnd.choice([None, None, None, 1, 5, 64, 128, 300])
        assert k.attention_tcgen05_supports(d, nq, nkv, ps)
        case = attention_case(torch.bfloat16, nq, nkv, d, lens, new, ps, seed=1000 * seed + it, sharp=rnd.random() < 0.5, poison=True)
        scale = 1.0 / math.sqrt(d)
        out = torch.full((sum(new), nq * d), 5.0, dtype=torch.bfloat16, device=DEV)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        wide, cache, bt = case["wide"].to(DEV), case["cache"].to(DEV), case["bt"].to(DEV)
        for _ in range(3):
            k.attention_tcgen05(wide, out, cache, bt, i32(case["qsl"]), i32(lens), new, nq, nkv, d, scale, window or 0)
        k.check_error_flags()
        close(out, attention_reference(case, lens, new, scale, window), 1.5e-2)


@pytest.mark.parametrize("requests", [3, 45])
@pytest.mark.parametrize("splits", [2, 4])
def test_paged_attention_decode_cluster_and_memory_combine(requests, splits):
    """Two to four splits on the TMA path meet in a cluster's shared memory while all clusters of the launch run at
    once (3 requests x 8 heads), and through the scratch buffer when they would not (45 x 8 clusters): both against the
    plain attention, and the copy paths against each other."""
    k = _k()
    nq, nkv, d, ps = 16, 8, 128, 16
    rnd = random.Random(requests * 10 + splits)
    lens = [rnd.choice([1, 30, 64, 65, 200, 500, 1100]) for _ in range(requests)]
    new = [1] * requests
    case = attention_case(torch.bfloat16, nq, nkv, d, lens, new, ps, seed=90 + splits, sharp=True, poison=True)
    scale = 1.0 / math.sqrt(d)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    cache, bt, wide = case["cache"].to(DEV), case["bt"].to(DEV), case["wide"].to(DEV)
    want = attention_reference(case, lens, new, scale)
    outs = []
    for tma in (True, False, True):
        out = torch.full((requests, nq * d), 5.0, dtype=torch.bfloat16, device=DEV)
        k.paged_attention_decode(wide, out, cache, bt, sl, nq, nkv, d, scale, 0, splits, tma=tma)
        k.check_error_flags()
        close(out, want, 1.5e-2)
        outs.append(out)
    close(outs[0], outs[1], 1e-2)
    assert torch.equal(outs[0], outs[2])


def test_paged_attention_decode_refuses_other_sizes():
    k = _k()
    assert not k.paged_attention_decode_supports(48, 6, 3)
    assert not k.paged_attention_decode_supports(128, 34, 2)
    q = torch.zeros(1, 6 * 48 * 2, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(k.KernelError, match="not taken"):
        k.paged_attention_decode(q, torch.zeros(1, 6 * 48, dtype=torch.bfloat16, device=DEV),
                                 torch.zeros(2, 2, 3, 16, 48, dtype=torch.bfloat16, device=DEV),
                                 torch.zeros(1, 2, dtype=torch.int32, device=DEV),
                                 torch.ones(1, dtype=torch.int32, device=DEV), 6, 3, 48, 1.0, 0, 1)


# ---- sampling ----------------------------------------------------------------------------------------------------

def _sample(k, logits, rows):
    import struct
    raw = b"".join(struct.pack("<fiff", *r) for r in rows)
    params = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(DEV)
    out = torch.empty(len(rows), dtype=torch.int32, device=DEV)
    k.sample(logits.to(DEV), params, out)
    return out.cpu().tolist()


@pytest.mark.parametrize("V", [517, 1000, 151936])
def test_sampler_against_plain(V):
    k = _k()
    g = torch.Generator().manual_seed(40)
    logits = torch.randn(6, V, generator=g) * 3
    logits[1, 7] = logits[1, 400] = logits[1].max() + 1          # a tie for the maximum: the lowest id wins
    rows = [(0.0, 0, 1.0, 0.5), (0.0, 0, 1.0, 0.9), (1.0, 1, 1.0, 0.3), (0.7, 40, 1.0, 0.77), (1.3, 0, 0.8, 0.41),
            (0.9, 50, 0.9, 0.05)]
    got = _sample(k, logits, rows)
    want = [P.sample_plain(logits[i], *rows[i]) for i in range(6)]
    assert got == want and got[1] == 7
    # many draws of one row: same answers as the plain sampler for the same uniforms
    row = logits[4:5].repeat(64, 1)
    us = [(i + 0.5) / 64 for i in range(64)]
    got = _sample(k, row, [(1.1, 30, 0.85, u) for u in us])
    want = [P.sample_plain(logits[4], 1.1, 30, 0.85, u) for u in us]
    assert sum(a != b for a, b in zip(got, want)) == 0
    kth = torch.sort(logits[4], descending=True).values[29]
    assert all(logits[4, t] >= kth for t in got)


@pytest.mark.parametrize("V, ld", [(517, 517), (1000, 1003), (151936, 151936), (5, 8), (64, 64)])
def test_argmax_rows(V, ld):
    """Greedy sampling of every row by clusters of eight CTAs: the largest value, ties to the lowest id, the same
    answers as the general sampling kernel; rows that are not 16-byte aligned, vocabularies smaller than the threads."""
    k = _k()
    g = torch.Generator().manual_seed(41)
    rows = 9
    wide = torch.randn(rows, ld, generator=g) * 3
    logits = wide[:, :V]
    top = float(logits.max()) + 1
    logits[1, V - 1] = logits[1, V // 2] = top                 # a tie across the CTAs' shares: the lower id wins
    logits[2, 0] = top
    logits[3, V - 1] = top
    logits[4] = -float("inf")                                  # nothing to choose: id 0
    logits[5, : max(1, V // 3)] = float("nan")                 # values that are not numbers never win
    dev = wide.to(DEV)[:, :V]
    out = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
    k.argmax_rows(dev, out)
    got = out.cpu().tolist()
    want = [P.sample_plain(torch.nan_to_num(logits[i], nan=-float("inf")), 0.0, 0, 1.0, 0.5) for i in range(rows)]
    assert got == want and got[1] == V // 2 and got[2] == 0 and got[3] == V - 1 and got[4] == 0
    assert got == _sample(k, logits.contiguous(), [(0.0, 0, 1.0, 0.5)] * rows)


# ---- the failure path of the bounded waits --------------------------------------------------------------

def test_bounded_wait_that_runs_out_raises_the_error_word():
    """Every TMA / tcgen05 kernel waits on its mbarriers with a limit and raises the device's error word when the
    limit is reached; ``check_error_flags`` turns the word into an exception.  No healthy run takes that path, so a
    self-test kernel takes it harmlessly: it waits, with the kernels' own loop and a short limit, on a barrier that
    nothing arrives on, then gives up and returns.  The exception must come after a plain launch, and after a replay
    of a CUDA graph that holds the launch (the engine reads the word only now and then for replayed steps)."""
    k = _k()
    k.check_error_flags(force=True)                       # start clean
    gave_up = torch.zeros(1, dtype=torch.int32, device=DEV)
    k.selftest_bounded_wait(1_000_000, DEV, gave_up)
    with pytest.raises(k.KernelError, match="gave up waiting on a barrier \\(code 91\\)"):
        k.check_error_flags()
    assert int(gave_up.item()) == 1
    k.check_error_flags(force=True)                       # the word was cleared: nothing is raised twice
    # the same inside a captured graph; the word is read when a check is forced
    gave_up.zero_()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        k.selftest_bounded_wait(500_000, DEV, gave_up)
    k.check_error_flags(force=True)                       # capturing ran nothing
    assert int(gave_up.item()) == 0
    graph.replay()
    k.note_flagged_launch(replayed=True)
    k.check_error_flags()                                 # one replayed step: not looked at yet
    with pytest.raises(k.KernelError, match="code 91"):
        k.check_error_flags(force=True)
    assert int(gave_up.item()) == 1
    # a limit beyond what the self-test allows is refused on the host, nothing is launched
    with pytest.raises(k.KernelError, match="the limit must be between"):
        k.selftest_bounded_wait(10**12, DEV)
    k.check_error_flags(force=True)


def test_gated_epilogues_agree_on_large_gates():
    """silu(g) * u with gates far out (|g| up to ~200, where exp(-g) overflows 32 bits): the prompt-sized tcgen05
    kernel, the weight-streaming kernel and the few-rows kernel give the exact formula's value, none a NaN."""
    k = _k()
    K, I = 64, 128
    x = torch.zeros(128, K, dtype=torch.bfloat16)
    x[:, 0] = 1.0
    w = torch.zeros(2 * I, K, dtype=torch.bfloat16)
    gates = torch.linspace(-200.0, 200.0, I)
    w[:I, 0] = gates.to(torch.bfloat16)
    w[I:, 0] = 1.5
    g = w[:I, 0].float()
    want = (g / (1 + torch.exp(-g)) * 1.5).expand(128, I)
    for M, fn in [(128, k.gemm_tcgen05), (128, k.gemm_wstream), (8, None)]:
        out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
        if fn is None:
            k.gemm_skinny(w.to(DEV), out, act=x[:M].to(DEV), silu_pair=True)
        else:
            fn(x[:M].to(DEV), w.to(DEV), out, silu_pair=True)
        assert bool(torch.isfinite(out.float()).all())
        close(out, want[:M], 4e-3)
