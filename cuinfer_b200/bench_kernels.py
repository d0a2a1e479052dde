"""Micro-benchmarks of single kernels at model sizes: ``python -m cuinfer_b200.bench_kernels <kernel> [options]``.

Each run builds inputs larger than the L2 cache (or rotates over several copies so that every launch reads cold
data), times the kernel with CUDA events after warm-up and prints one JSON line with the achieved GB/s or
TFLOP/s.  The same command under ``ncu`` gives the counters kept in ``profiles/``.
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch

from . import kernels


def _time(fn, iters: int, warmup: int = 3) -> float:
    """Milliseconds per call.  The calls are captured into one CUDA graph and the graph is replayed, so that
    the figure is the device's time and not the time Python needs to issue a launch."""
    for _ in range(warmup):
        fn(0)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(iters):
            fn(i)
    graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters


def attention_decode(args) -> dict:
    R, ctx, nq, nkv, d, ps = args.batch, args.context, args.q_heads, args.kv_heads, args.head_dim, args.page_size
    pages_per = (ctx + ps - 1) // ps
    copies = max(1, args.copies)
    num_pages = R * pages_per * copies
    dev = "cuda:0"
    cache = torch.randn(num_pages, 2, nkv, ps, d, device=dev, dtype=torch.bfloat16)
    perm = torch.randperm(num_pages, device=dev).to(torch.int32).view(copies, R, pages_per)
    q = torch.randn(R, (nq + 2 * nkv) * d, device=dev, dtype=torch.bfloat16)
    out = torch.empty(R, nq * d, device=dev, dtype=torch.bfloat16)
    sl = torch.full((R,), ctx, dtype=torch.int32, device=dev)
    splits = args.splits or kernels.decode_splits(R, nkv, ctx, tma=kernels.decode_tma_takes(ps, d, 0))
    scale = 1.0 / math.sqrt(d)

    def run(i):
        kernels.paged_attention_decode(q, out, cache, perm[i % copies], sl, nq, nkv, d, scale, 0, splits)

    ms = _time(run, args.iters)
    bytes_read = R * ctx * nkv * d * 2 * 2
    return {"kernel": "paged_attention_decode", "batch": R, "context": ctx, "splits": splits, "ms": round(ms, 4),
            "GBps": round(bytes_read / ms / 1e6, 1), "bytes": bytes_read}


def attention_prefill(args) -> dict:
    """``--requests`` requests of ``--tokens`` new tokens each after ``--prefix`` cached ones, in one launch."""
    n, prefix, nq, nkv, d, ps = args.tokens, args.prefix, args.q_heads, args.kv_heads, args.head_dim, args.page_size
    R = max(1, args.requests)
    total = n + prefix
    pages = (total + ps - 1) // ps
    dev = "cuda:0"
    cache = torch.randn(R * pages, 2, nkv, ps, d, device=dev, dtype=torch.bfloat16)
    table = torch.randperm(R * pages, device=dev).to(torch.int32).view(R, pages)
    q = torch.randn(R * n, (nq + 2 * nkv) * d, device=dev, dtype=torch.bfloat16)
    out = torch.empty(R * n, nq * d, device=dev, dtype=torch.bfloat16)
    qsl = torch.arange(R + 1, dtype=torch.int32, device=dev) * n
    sl = torch.full((R,), total, dtype=torch.int32, device=dev)
    scale = 1.0 / math.sqrt(d)

    def run(i):
        if args.impl == "tcgen05":
            kernels.attention_tcgen05(q, out, cache, table, qsl, sl, [n] * R, nq, nkv, d, scale, 0)
        else:
            kernels.paged_attention_prefill(q, out, cache, table, qsl, sl, [n] * R, nq, nkv, d, scale, 0)

    ms = _time(run, args.iters)
    if args.impl == "tcgen05":
        kernels.check_error_flags()
    flops = R * 4.0 * nq * d * (n * prefix + n * (n + 1) / 2.0)
    return {"kernel": f"attention_prefill[{args.impl}]", "requests": R, "tokens": n, "prefix": prefix, "ms": round(ms, 4),
            "TFLOPs": round(flops / ms / 1e9, 1)}


def norm(args) -> dict:
    """Residual add + RMSNorm of ``--tokens`` rows of ``--hidden`` values (float32 residual, bfloat16 delta and output)."""
    n, H = args.tokens, args.hidden
    dev = "cuda:0"
    copies = max(1, args.copies)
    res = torch.randn(copies, n, H, device=dev)
    delta = torch.randn(copies, n, H, device=dev, dtype=torch.bfloat16)
    out = torch.empty(copies, n, H, device=dev, dtype=torch.bfloat16)
    w = torch.ones(H, device=dev, dtype=torch.bfloat16)

    def run(i):
        c = i % copies
        kernels.add_rmsnorm(res[c], delta[c], w, 1e-6, out[c])

    ms = _time(run, args.iters)
    moved = n * H * (4 + 2 + 4 + 2)
    return {"kernel": "add_rmsnorm", "tokens": n, "hidden": H, "ms": round(ms, 4), "GBps": round(moved / ms / 1e6, 1)}


def gemm(args) -> dict:
    from .parts.linear import matmul_nt

    M, N, K = args.m, args.n, args.k
    dev = "cuda:0"
    copies = max(1, args.copies)
    w = torch.randn(copies, N, K, device=dev, dtype=torch.bfloat16) * 0.02
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    out_dtype = torch.float32 if args.f32_out else torch.bfloat16
    kernels.use_pdl = bool(args.pdl)

    out = torch.empty(M, N, device=dev, dtype=out_dtype)

    def run(i):
        if args.impl == "tcgen05":
            kernels.gemm_tcgen05(x, w[i % copies], out)
        elif args.impl == "wstream":
            kernels.gemm_wstream(x, w[i % copies], out)
        elif args.impl == "skinny":
            kernels.gemm_skinny(w[i % copies], out, act=x)
        elif args.impl == "cublas":
            torch.mm(x, w[i % copies].t(), out=out)
        else:
            matmul_nt(x, w[i % copies], out_dtype)

    ms = _time(run, args.iters)
    if args.impl in ("tcgen05", "wstream"):
        kernels.check_error_flags()
    return {"kernel": f"matmul_nt[{args.impl}]", "M": M, "N": N, "K": K, "ms": round(ms, 4),
            "GBps": round((N * K + M * K + M * N) * 2 / ms / 1e6, 1), "TFLOPs": round(2.0 * M * N * K / ms / 1e9, 2)}


def rope(args) -> dict:
    """Per-head norm, rotary encoding and cache write of ``--tokens`` packed qkv rows."""
    T, nq, nkv, d, ps = args.tokens, args.q_heads, args.kv_heads, args.head_dim, args.page_size
    dev = "cuda:0"
    copies = max(1, args.copies)
    pages = (T + ps - 1) // ps
    qkv = torch.randn(copies, T, (nq + 2 * nkv) * d, device=dev, dtype=torch.bfloat16)
    cache = torch.zeros(copies * pages, 2, nkv, ps, d, device=dev, dtype=torch.bfloat16)
    positions = torch.arange(T, device=dev, dtype=torch.int32)
    slots = torch.randperm(pages, device=dev).repeat_interleave(ps)[:T].to(torch.int32) * ps + positions % ps
    qw = torch.ones(d, device=dev, dtype=torch.bfloat16)
    inv = 1.0 / torch.pow(torch.tensor(1e6), torch.arange(d // 2, dtype=torch.float32) * 2.0 / d)
    ang = torch.arange(T, dtype=torch.float32)[:, None] * inv[None, :]
    table = torch.stack((torch.cos(ang), torch.sin(ang)), -1).contiguous().to(dev)

    def run(i):
        c = i % copies
        kernels.qk_norm_rope_kv_write(qkv[c], positions, slots + c * pages * ps, qw, qw, 1e-6, table, d, cache, nq, nkv, d)

    ms = _time(run, args.iters)
    moved = T * (nq + 2 * nkv) * d * 2 * 2
    return {"kernel": "qk_norm_rope_kv_write", "tokens": T, "ms": round(ms, 4), "GBps": round(moved / ms / 1e6, 1)}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m cuinfer_b200.bench_kernels")
    sub = p.add_subparsers(dest="kernel", required=True)
    a = sub.add_parser("attention_decode")
    a.add_argument("--batch", type=int, default=8)
    a.add_argument("--context", type=int, default=4096)
    a.add_argument("--q-heads", type=int, default=16)
    a.add_argument("--kv-heads", type=int, default=8)
    a.add_argument("--head-dim", type=int, default=128)
    a.add_argument("--page-size", type=int, default=16)
    a.add_argument("--splits", type=int, default=0)
    a.add_argument("--copies", type=int, default=4, help="rotate over this many caches so that launches read cold data")
    a.add_argument("--iters", type=int, default=20)
    f = sub.add_parser("attention_prefill")
    f.add_argument("--tokens", type=int, default=2048)
    f.add_argument("--prefix", type=int, default=0)
    f.add_argument("--requests", type=int, default=1)
    f.add_argument("--q-heads", type=int, default=16)
    f.add_argument("--kv-heads", type=int, default=8)
    f.add_argument("--head-dim", type=int, default=128)
    f.add_argument("--page-size", type=int, default=16)
    f.add_argument("--impl", default="mma", choices=["mma", "tcgen05"])
    f.add_argument("--iters", type=int, default=10)
    ro = sub.add_parser("rope", help=rope.__doc__)
    ro.add_argument("--tokens", type=int, default=2048)
    ro.add_argument("--q-heads", type=int, default=16)
    ro.add_argument("--kv-heads", type=int, default=8)
    ro.add_argument("--head-dim", type=int, default=128)
    ro.add_argument("--page-size", type=int, default=16)
    ro.add_argument("--copies", type=int, default=8)
    ro.add_argument("--iters", type=int, default=16)
    no = sub.add_parser("norm", help=norm.__doc__)
    no.add_argument("--tokens", type=int, default=2048)
    no.add_argument("--hidden", type=int, default=1024)
    no.add_argument("--copies", type=int, default=8, help="buffers rotated through, so that the L2 does not keep them")
    no.add_argument("--iters", type=int, default=50)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8)
    g.add_argument("--n", type=int, default=4096)
    g.add_argument("--k", type=int, default=1024)
    g.add_argument("--f32-out", action="store_true")
    g.add_argument("--impl", default="auto", choices=["auto", "tcgen05", "wstream", "skinny", "cublas"])
    g.add_argument("--pdl", action="store_true", help="launch with programmatic dependent launch")
    g.add_argument("--copies", type=int, default=8)
    g.add_argument("--iters", type=int, default=20)
    args = p.parse_args(argv)
    result = {"attention_decode": attention_decode, "attention_prefill": attention_prefill, "gemm": gemm, "rope": rope, "norm": norm}[args.kernel](args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
