"""Choice of the bfloat16 matrix-product kernel for a given shape.

Order of preference: this package's tensor-core kernels, then the library product (cuBLAS via
``torch.mm``; the reference calls cuBLAS for every projection, csrc/ops/projection.cu:32-44), then
the FMA kernel for shapes cuBLAS's tensor-core paths do not take.  A shape no kernel takes raises.
"""
from __future__ import annotations

import torch

from .. import kernels


def bf16_matmul_nt(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = x[M, K] @ weight[N, K]^T; x and weight bfloat16, out bfloat16 or float32."""
    M, K = x.shape
    N = weight.shape[0]
    if M <= 16 and weight.is_contiguous() and kernels.gemm_skinny_supports(M, N, K):
        kernels.gemm_skinny(weight, out, act=x)
        return
    if K % 8 == 0 and N % 8 == 0 and x.is_contiguous() and weight.is_contiguous():
        if out.dtype == torch.bfloat16:
            torch.mm(x, weight.t(), out=out)
            return
        if out.dtype == torch.float32:
            tmp = torch.mm(x, weight.t(), out_dtype=torch.float32)
            out.copy_(tmp)
            return
    kernels.gemm_generic(x, weight, out)
