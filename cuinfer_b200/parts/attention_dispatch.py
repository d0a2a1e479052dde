"""Choice of the paged-attention kernel for a step.

float32 always runs the all-sizes kernel.  bfloat16: a step of single decoded tokens runs the split-KV kernel (its
TMA path where the cache layout allows and a CTA streams at least ``kernels.DECODE_TMA_MIN_KEYS`` keys, else its
cp.async path); any
other step runs the tcgen05 kernel (head size 128, heads per kv head dividing 128) or the mma.sync kernel (head
size 64 or 128); other head sizes fall back to the all-sizes kernel.  ``CUINFER_B200_ATTENTION=mma`` keeps prompt
portions off the tcgen05 kernel (for comparisons).
"""
from __future__ import annotations

import os

import torch

from .. import kernels
from .context import PagedKV, StepContext


_FORCE_MMA = os.environ.get("CUINFER_B200_ATTENTION", "") == "mma"


def paged_attention(qkv: torch.Tensor, out: torch.Tensor, kv: PagedKV, ctx: StepContext, num_heads: int,
                    num_kv_heads: int, head_dim: int, scale: float, window: int, warm: torch.Tensor | None = None) -> None:
    """``warm``: what the step reads right after the attention (the output projection's weight); the decode kernel
    asks for it to be fetched into the L2 when its stream of keys ends."""
    if (qkv.dtype == torch.bfloat16 and ctx.decode_only
            and kernels.paged_attention_decode_supports(head_dim, num_heads, num_kv_heads)):
        longest = max(1, ctx.max_seq_len)
        tma = kernels.decode_tma_takes(kv.group.page_size, head_dim, window)
        splits = kernels.decode_splits(ctx.num_requests, num_kv_heads, longest, kernels.decode_slots(head_dim), tma=tma,
                                       head_dim=head_dim)
        tma = tma and kernels.decode_uses_tma(longest, splits)
        kernels.paged_attention_decode(qkv, out, kv.cache, kv.group.block_table, ctx.seq_lens, num_heads,
                                       num_kv_heads, head_dim, scale, window, splits, tma=tma, warm=warm)
        return
    if qkv.dtype == torch.bfloat16 and not _FORCE_MMA and kernels.attention_tcgen05_supports(
            head_dim, num_heads, num_kv_heads, kv.group.page_size) and out.stride(0) % 8 == 0 and qkv.stride(0) % 8 == 0:
        lens = ctx.query_lens_for_launch()
        kernels.attention_tcgen05(qkv, out, kv.cache, kv.group.block_table, ctx.query_start_loc, ctx.seq_lens, lens,
                                  num_heads, num_kv_heads, head_dim, scale, window)
        return
    if qkv.dtype == torch.bfloat16 and kernels.paged_attention_prefill_supports(head_dim, num_heads, num_kv_heads):
        lens = ctx.query_lens_for_launch()
        kernels.paged_attention_prefill(qkv, out, kv.cache, kv.group.block_table, ctx.query_start_loc, ctx.seq_lens,
                                        lens, num_heads, num_kv_heads, head_dim, scale, window)
        return
    kernels.paged_attention_generic(
        qkv, out, kv.cache, kv.group.block_table, ctx.query_start_loc, ctx.seq_lens, ctx.token_request,
        num_heads, num_kv_heads, head_dim, scale, window)
