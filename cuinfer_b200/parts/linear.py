"""A projection ``y = x · Wᵀ`` over one weight matrix ``[out, in]``, possibly several checkpoint matrices
stacked along ``out`` (the reference's ``Linear``, csrc/model/layers/linear.cpp:35-95, stacks q/k/v and
gate/up the same way and has no bias).

Which kernel multiplies is decided here, per call, from the engine dtype and the shape:

* float32: the FMA kernel (``gemm_generic``), true 32-bit, any shape;
* bfloat16: the tensor-core kernels of this package where they take the shape; otherwise the library
  product (cuBLAS through ``torch.mm``), which is what the reference uses for every projection
  (csrc/ops/projection.cu:32-44); shapes that are not a multiple of 8 go to ``gemm_generic``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import kernels
from .base import LazyNorm
from .spec import TensorSpec


def matmul_nt(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x[M, K] @ weight[N, K]^T`` → ``[M, N]`` in ``out_dtype`` (default: x's dtype)."""
    M, K = x.shape
    N = weight.shape[0]
    out_dtype = out_dtype or x.dtype
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    if M == 0:
        return out
    if x.dtype == torch.float32:
        kernels.gemm_generic(x, weight, out)
        return out
    from . import gemm_dispatch
    gemm_dispatch.bf16_matmul_nt(x, weight, out)
    return out


class Linear:
    def __init__(self, names: Sequence[str], out_features: Sequence[int], in_features: int, dtype: torch.dtype) -> None:
        if len(names) != len(out_features):
            raise ValueError("one out_features per name")
        self.names = list(names)
        self.out_features = list(out_features)
        self.in_features = in_features
        self.dtype = dtype
        self.weight: Optional[torch.Tensor] = None
        self.warm_next: Optional[torch.Tensor] = None     # what the step reads right after this projection (a hint for the L2)

    def tensors(self) -> List[TensorSpec]:
        return [TensorSpec(n, (o, self.in_features)) for n, o in zip(self.names, self.out_features)]

    def load(self, store) -> None:
        specs = self.tensors()
        self.weight = store.get(specs[0]) if len(specs) == 1 else store.get_stacked(specs)
        if self.weight.dtype != self.dtype:
            self.weight = self.weight.to(self.dtype)

    def workspace_bytes(self, tokens: int, silu_pair: bool = False) -> int:
        """Bytes of the projection's output for ``tokens`` rows (with ``silu_pair`` the stacked product may exist
        beside the gated one)."""
        width = 2 if self.dtype == torch.bfloat16 else 4
        n = sum(self.out_features)
        return tokens * (n + n // 2 if silu_pair else n) * width

    def tie(self, weight: torch.Tensor) -> None:
        """Use another tensor's storage as this projection's weight (a tied output head)."""
        if tuple(weight.shape) != (sum(self.out_features), self.in_features):
            raise ValueError(f"tied weight has shape {list(weight.shape)}")
        self.weight = weight

    def forward(self, x, out_dtype: Optional[torch.dtype] = None, silu_pair: bool = False) -> torch.Tensor:
        """``x`` is a tensor [M, K] or a :class:`LazyNorm`.  ``silu_pair``: the weight is gates then ups and the
        result is ``silu(gate) * up`` [M, N/2]."""
        if self.weight is None:
            raise RuntimeError(f"projection {self.names} used before its weights were loaded")
        fused = self._forward_skinny(x, out_dtype, silu_pair)
        if fused is not None:
            return fused
        if isinstance(x, LazyNorm):
            x = x.materialize()
        if silu_pair and x.dtype == torch.bfloat16 and x.shape[0] > 0:
            from . import gemm_dispatch
            gated = gemm_dispatch.bf16_gated_matmul_nt(x, self.weight)
            if gated is not None:
                return gated
        y = matmul_nt(x, self.weight, out_dtype if not silu_pair else None)
        if not silu_pair:
            return y
        act = torch.empty((y.shape[0], y.shape[1] // 2), dtype=y.dtype, device=y.device)
        kernels.silu_mul(y, act)
        return act

    def _forward_skinny(self, x, out_dtype, silu_pair) -> Optional[torch.Tensor]:
        """The few-rows kernel with the norm in its prologue and/or the gate in its epilogue, when it takes
        the shape; None otherwise."""
        w = self.weight
        if w.dtype != torch.bfloat16 or not w.is_contiguous():
            return None
        lazy = isinstance(x, LazyNorm)
        M = x.shape[0]
        N, K = w.shape
        if M == 0 or M > 16:
            return None
        out_dtype = out_dtype or torch.bfloat16
        if silu_pair and out_dtype != torch.bfloat16:
            return None
        out_cols = N // 2 if silu_pair else N
        from . import gemm_dispatch
        choice = gemm_dispatch.few_rows_kernel(M, N, K)
        if choice == "library":
            return None           # the library product (and the activation kernel after it) in forward()
        if choice == "wstream":
            # long K: the weight-streaming kernel (no norm prologue; the gate is in its epilogue)
            rows = x.materialize() if lazy else x
            if (not silu_pair or rows.dtype != torch.bfloat16 or rows.stride(1) != 1 or rows.stride(0) % 8 or w.stride(0) % 8
                    or not kernels.gemm_wstream_supports(M, N, K)):
                return None
            out = torch.empty((M, out_cols), dtype=torch.bfloat16, device=w.device)
            kernels.gemm_wstream(rows, w, out, silu_pair=True)
            return out
        if lazy and x._rows is None:
            stream = x.stream
            rms = x.norm.fusable_rms()
            if (rms is not None and stream.residual.is_contiguous()
                    and K <= gemm_dispatch.FUSED_NORM_MAX_K and kernels.gemm_skinny_supports(M, N, K, True)
                    and (stream.pending is None or stream.pending.is_contiguous())):
                out = torch.empty((M, out_cols), dtype=out_dtype, device=w.device)
                has_delta = stream.pending is not None
                kernels.gemm_skinny(w, out, residual=stream.residual, pending=stream.pending, norm_weight=rms[0],
                                    eps=rms[1], residual_out=stream.spare() if has_delta else None, silu_pair=silu_pair,
                                    warm=self.warm_next)
                if has_delta:
                    stream.swap()
                return out
        rows = x.materialize() if lazy else x
        if rows.dtype != torch.bfloat16 or rows.stride(1) != 1 or not kernels.gemm_skinny_supports(M, N, K, False):
            return None
        out = torch.empty((M, out_cols), dtype=out_dtype, device=w.device)
        kernels.gemm_skinny(w, out, act=rows, silu_pair=silu_pair, warm=self.warm_next)
        return out
