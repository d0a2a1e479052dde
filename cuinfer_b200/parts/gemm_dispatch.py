"""Choice of the bfloat16 matrix-product kernel for a given shape.

* up to 16 rows (decode steps), weights under 24 MB (every matrix of the Qwen3-0.6B layer sizes): the few-rows kernel
  (``gemm_skinny``), weights streamed once through registers, with the norm in its prologue and the SiLU gate in its
  epilogue; larger weights (the 8B and 32B layer sizes) go to the library, which measured faster on all of them —
  6144 x 4096: 11.5 us against 19.5 (few-rows) and 21.6 (weight-streaming); 24576 x 4096: 34.3 against 43.5 and 46.0;
  10240 x 5120: 22.3 against 39.6 and 33.8; 5120 x 25600: 44 against 69 (weight-streaming); 151936 x 4096: 198 against
  216 and 204 — except long K with few output features (4096 x 12288: weight-streaming tcgen05 kernel 22.4 us, library
  32.2), which stay on ``gemm_wstream``;
* 128 rows and more (prompt portions): the tcgen05 / TMA / TMEM kernel (``gemm_tcgen05``), with the SiLU gate in its
  epilogue for the gate/up projection — where the product has at least ``TCGEN05_MIN_TILES`` output tiles of
  128 x 128.  With fewer, every CTA walks the whole of K alone and the library, which splits K over more CTAs, measured
  1.3 to 2.7 times faster (2048 x 1024 x 2048: 8.8 us against 14.9), so those go to cuBLAS;
* in between, and for K that is not a multiple of 8: the library product (cuBLAS via ``torch.mm``; the reference
  calls cuBLAS for every projection, csrc/ops/projection.cu:32-44), or the FMA kernel for shapes cuBLAS's
  tensor-core paths do not take.

``CUINFER_B200_GEMM=cublas`` sends every prompt-sized product to the library, ``CUINFER_B200_GEMM=tcgen05`` every one
that the kernel takes to the kernel, ``CUINFER_B200_GEMM=own`` keeps the decode steps' large products on this package's
kernels as well (for comparisons).
"""
from __future__ import annotations

import torch

import os

from .. import kernels

TCGEN05_MIN_ROWS = 128
TCGEN05_MIN_TILES = 296          # output tiles of 128 x 128 from which the tcgen05 kernel is chosen over the library
FEW_ROWS = 16
FUSED_NORM_MAX_K = 2048          # the norm prologue keeps 32-bit rows of all of K in shared memory: beyond this one CTA per SM
FEW_ROWS_LONG_K = 4096           # above it the few-rows kernel is down to one CTA per SM (measured: 1.9 TB/s at K = 12288)
FEW_ROWS_LIBRARY_BYTES = 24 << 20   # weights from this size on: the library product, unless K is long and N small
WSTREAM_MIN_K, WSTREAM_MAX_N = 12288, 4096
_FORCE_CUBLAS = os.environ.get("CUINFER_B200_GEMM", "") == "cublas"
_FORCE_TCGEN05 = os.environ.get("CUINFER_B200_GEMM", "") == "tcgen05"
_FORCE_OWN = os.environ.get("CUINFER_B200_GEMM", "") in ("own", "tcgen05")       # decode steps too stay on this package's kernels


def few_rows_kernel(M: int, N: int, K: int) -> str:
    """Which kernel multiplies ``M <= 16`` rows with an [N, K] weight: "skinny", "wstream" or "library"."""
    if N * K * 2 >= FEW_ROWS_LIBRARY_BYTES and not _FORCE_OWN:
        if K >= WSTREAM_MIN_K and N <= WSTREAM_MAX_N and kernels.gemm_wstream_supports(M, N, K):
            return "wstream"
        return "library"
    if K > FEW_ROWS_LONG_K and kernels.gemm_wstream_supports(M, N, K):
        return "wstream"
    return "skinny"


def takes_tcgen05(x: torch.Tensor, weight: torch.Tensor, fused: bool = False) -> bool:
    """``fused``: the product carries an epilogue (the SiLU gate) that the library call would need another kernel for;
    it stays on the tcgen05 kernel whatever its size."""
    M, K = x.shape
    N = weight.shape[0]
    if not (M >= TCGEN05_MIN_ROWS and not _FORCE_CUBLAS and x.stride(1) == 1 and weight.stride(1) == 1
            and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and kernels.gemm_tcgen05_supports(M, N, K)):
        return False
    if fused or _FORCE_TCGEN05 or K % 8 or N % 8:
        return True
    return -(-M // 128) * -(-N // 128) >= TCGEN05_MIN_TILES


def bf16_gated_matmul_nt(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor | None:
    """silu(x gate^T) * (x up^T) for a weight of gate rows then up rows, in one tcgen05 kernel, when the shape is one
    it takes (prompt-sized, half of N a multiple of 8); None otherwise."""
    N = weight.shape[0]
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or N % 16 or not takes_tcgen05(x, weight, fused=True):
        return None
    out = torch.empty((x.shape[0], N // 2), dtype=torch.bfloat16, device=x.device)
    kernels.gemm_tcgen05(x, weight, out, silu_pair=True)
    return out


def bf16_matmul_nt(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = x[M, K] @ weight[N, K]^T; x and weight bfloat16, out bfloat16 or float32."""
    M, K = x.shape
    N = weight.shape[0]
    if M <= FEW_ROWS and weight.stride(1) == 1 and x.stride(1) == 1:
        choice = few_rows_kernel(M, N, K)
        if choice == "wstream" and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0:
            kernels.gemm_wstream(x, weight, out)
            return
        if choice == "skinny" and weight.is_contiguous() and kernels.gemm_skinny_supports(M, N, K):
            kernels.gemm_skinny(weight, out, act=x)
            return
    library_ok = K % 8 == 0 and N % 8 == 0 and x.is_contiguous() and weight.is_contiguous()
    if takes_tcgen05(x, weight, fused=not library_ok):       # a product the library call cannot take stays on the kernel
        kernels.gemm_tcgen05(x, weight, out)
        return
    if library_ok:
        if out.dtype == torch.bfloat16:
            torch.mm(x, weight.t(), out=out)
            return
        if out.dtype == torch.float32:
            tmp = torch.mm(x, weight.t(), out_dtype=torch.float32)
            out.copy_(tmp)
            return
    kernels.gemm_generic(x, weight, out)
