"""Arrangements of a layer's parts around the residual stream.

``prenorm``: ``x += mixer(norm1(x)); x += feed_forward(norm2(x))`` — the reference's decoder layer
(csrc/model/causal_lm.cpp:138-188).  Each sub-layer's output stays pending until the next norm, which
adds it to the 32-bit residual and normalises in one pass (the reference fuses only the first add,
csrc/ops/residual_rms_norm_fused.cu:58-109); the last pending delta of the last layer is folded by
the model's final norm.  Spec: ``PartSpec("prenorm", norm_names=(first, second))``.
"""
from __future__ import annotations

from typing import Callable, List

from .base import Block, FeedForward, LazyNorm, Mixer, Norm, Part, ResidualStream
from .context import StepContext
from .registry import BLOCKS
from .spec import PartSpec


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    def __init__(self, spec: PartSpec, *, mixer: Mixer, feed_forward: FeedForward,
                 make_norm: Callable[[str], Norm], prefix: str) -> None:
        super().__init__(spec, mixer=mixer, feed_forward=feed_forward, make_norm=make_norm, prefix=prefix)
        first, second = spec.get("norm_names", ("input_layernorm", "post_attention_layernorm"))
        self.mixer_norm = make_norm(f"{prefix}.{first}")
        self.feed_forward_norm = make_norm(f"{prefix}.{second}")

    def parts(self) -> List[Part]:
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, stream: ResidualStream, ctx: StepContext, run: int) -> None:
        h = self._normed(stream, self.mixer_norm, self.mixer)
        stream.pending = self.mixer.forward(h, ctx, run)
        h = self._normed(stream, self.feed_forward_norm, self.feed_forward)
        stream.pending = self.feed_forward.forward(h, ctx)

    @staticmethod
    def _normed(stream: ResidualStream, norm: Norm, consumer: Part):
        """The normed rows for ``consumer``: computed now, or handed over uncomputed when the consumer can
        fold the norm into its first projection."""
        if getattr(consumer, "accepts_lazy_norm", False):
            return LazyNorm(stream, norm)
        return norm.add_norm(stream)
