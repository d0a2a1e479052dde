"""A decoder built from a :class:`ModelSpec`: embedding, the layers in their run order, final norm, output head.

The reference's ``CausalLM`` (csrc/model/causal_lm.cpp:16-115) does the same for one fixed arrangement:
embedding gather (:74-80), ``L`` decoder layers (:81-86), then at the wanted positions only a gather,
the final norm and the output projection, with the head aliasing the embedding when the model ties them
(:35-38, :99-114).  Here logits come back in 32 bits.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import kernels
from .base import Block, Part, ResidualStream
from .context import StepContext
from .linear import Linear
from .registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS
from .spec import LayerSpec, ModelSpec, PagedCacheNeed, StateNeed, TensorSpec


def build_layer(layer: LayerSpec, hidden_size: int, dtype: torch.dtype) -> Block:
    mixer_name = layer.mixer.get("name", "self_attn")
    ffn_name = layer.feed_forward.get("name", "mlp")
    mixer = MIXERS.get(layer.mixer.kind)(layer.mixer, hidden_size=hidden_size, prefix=f"{layer.prefix}.{mixer_name}", dtype=dtype)
    ffn = FEED_FORWARDS.get(layer.feed_forward.kind)(layer.feed_forward, hidden_size=hidden_size,
                                                     prefix=f"{layer.prefix}.{ffn_name}", dtype=dtype)
    norm_cls = NORMS.get(layer.norm.kind)

    def make_norm(prefix: str):
        return norm_cls(layer.norm, hidden_size=hidden_size, prefix=prefix, dtype=dtype)

    return BLOCKS.get(layer.block.kind)(layer.block, mixer=mixer, feed_forward=ffn, make_norm=make_norm, prefix=layer.prefix)


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype) -> None:
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"model dtype must be bfloat16 or float32, got {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.hidden_size = spec.hidden_size
        self.vocab_size = spec.vocab_size
        self.order: Tuple[int, ...] = spec.run_order()
        self.cache_source: Dict[int, int] = dict(spec.cache_source)
        self.blocks: List[Block] = [build_layer(l, spec.hidden_size, dtype) for l in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, hidden_size=spec.hidden_size,
                                                          prefix=spec.final_norm_prefix, dtype=dtype)
        self.embedding: Optional[torch.Tensor] = None
        self.tied = spec.lm_head_name is None
        self.lm_head = Linear([spec.lm_head_name or spec.embedding_name], [spec.vocab_size], spec.hidden_size, dtype)
        self._bad_id_flag: Optional[torch.Tensor] = None

    # ---- weights ------------------------------------------------------------------------------
    def _embedding_spec(self) -> TensorSpec:
        return TensorSpec(self.spec.embedding_name, (self.vocab_size, self.hidden_size))

    def parts(self) -> List[Part]:
        out: List[Part] = []
        for block in self.blocks:
            out.extend(block.parts())
        out.append(self.final_norm)
        return out

    def tensors(self) -> List[TensorSpec]:
        specs = [self._embedding_spec()]
        for part in self.parts():
            specs.extend(part.tensors())
        if not self.tied:
            specs.extend(self.lm_head.tensors())
        seen: Dict[str, TensorSpec] = {}
        for s in specs:
            if s.name in seen and seen[s.name].shape != s.shape:
                raise ValueError(f"tensor {s.name} is expected with two shapes: {seen[s.name].shape} and {s.shape}")
            seen[s.name] = s
        return list(seen.values())

    def load(self, store) -> None:
        store.check(self.tensors())
        self.embedding = store.get(self._embedding_spec())
        if self.embedding.dtype != self.dtype:
            self.embedding = self.embedding.to(self.dtype)
        for part in self.parts():
            part.load(store)
        if self.tied:
            self.lm_head.tie(self.embedding)
        else:
            self.lm_head.load(store)
        self._bad_id_flag = torch.zeros(1, dtype=torch.int32, device=store.device)
        # hints for the L2 along the order in which the layers run: every layer is told which weight follows it
        runs = self.runs()
        for i, (_run, layer) in enumerate(runs):
            follower = self.blocks[runs[i + 1][1]].first_weight() if i + 1 < len(runs) else None
            self.blocks[layer].warm_after(follower)

    # ---- what the layers keep between steps ----------------------------------------------------
    def runs(self) -> List[Tuple[int, int]]:
        """(run index, layer index) in execution order."""
        return list(enumerate(self.order))

    def cache_needs(self) -> Dict[int, PagedCacheNeed]:
        """Paged cache of every run that owns one (runs that read another run's cache are left out)."""
        out: Dict[int, PagedCacheNeed] = {}
        for run, layer in self.runs():
            need = self.blocks[layer].mixer.cache_need()
            if need is None:
                if run in self.cache_source:
                    raise ValueError(f"run {run} is told to read run {self.cache_source[run]}'s cache but its mixer has none")
                continue
            if run in self.cache_source:
                src_need = self.blocks[self.order[self.cache_source[run]]].mixer.cache_need()
                if src_need is None or (src_need.num_kv_heads, src_need.head_dim) != (need.num_kv_heads, need.head_dim):
                    raise ValueError(f"run {run} cannot read run {self.cache_source[run]}'s cache: shapes differ")
                continue
            out[run] = need
        return out

    def state_needs(self) -> Dict[int, StateNeed]:
        out: Dict[int, StateNeed] = {}
        for run, layer in self.runs():
            need = self.blocks[layer].mixer.state_need()
            if need is not None:
                out[run] = need
        return out

    # ---- what the engine asks before it runs the model -----------------------------------------------
    @property
    def capturable(self) -> bool:
        """True when every part's and block's ``forward`` may be replayed from a CUDA graph (Part.capturable)."""
        return all(block.capturable for block in self.blocks) and all(part.capturable for part in self.parts())

    def workspace_bytes(self, tokens: int, rows: int) -> int:
        """Device memory a step of ``tokens`` rows with ``rows`` wanted logits needs beside weights and cache: the
        32-bit residual stream with its spare and a pending delta, the widest block's intermediate results, and the
        wanted rows with their logits (twice: the sampler works on a copy)."""
        residual = 3 * tokens * self.hidden_size * 4
        widest = max((block.workspace_bytes(tokens) for block in self.blocks), default=0)
        head = rows * (self.hidden_size * 8 + self.vocab_size * 8)
        return residual + widest + head

    # ---- compute -------------------------------------------------------------------------------------
    def forward(self, ctx: StepContext) -> ResidualStream:
        residual = torch.empty((ctx.num_tokens, self.hidden_size), dtype=torch.float32, device=ctx.token_ids.device)
        kernels.embedding_gather(ctx.token_ids, self.embedding, residual, self._bad_id_flag)
        stream = ResidualStream(residual)
        for run, layer in self.runs():
            self.blocks[layer].forward(stream, ctx, run)
        return stream

    def logits(self, stream: ResidualStream, indices: torch.Tensor) -> torch.Tensor:
        """32-bit logits ``[len(indices), vocab]`` of the rows ``indices`` of the step."""
        rows = torch.empty((indices.numel(), self.hidden_size), dtype=torch.float32, device=indices.device)
        kernels.gather_rows(stream.residual, stream.pending, indices, rows)
        normed = self.final_norm.norm_rows(rows)
        return self.lm_head.forward(normed, out_dtype=torch.float32)

    def saw_bad_token_id(self) -> bool:
        """True if a token id outside the vocabulary reached the embedding since the last call (it read as zeros)."""
        bad = bool(self._bad_id_flag.item())
        if bad:
            self._bad_id_flag.zero_()
        return bad
