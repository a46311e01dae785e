"""Arrangements of parts into a layer.  ``prenorm``: andre-fu/prism's decoder
layer (engine/executor.py:106-127): norm, mixer, residual add, norm,
feed-forward, residual add.  Each residual add is carried out by the norm
that follows it (the next block's first norm, or the final norm).
``parallel``: one norm whose output both the mixer and the feed-forward read;
their two results are added to the residual stream together."""

from __future__ import annotations

from typing import Optional

from .base import Block, PartSpec, build_part, register_part
from .. import ops


@register_part("block", "prenorm")
class PreNormBlock(Block):
    def __init__(self, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec, ff_norm: PartSpec):
        self.mixer_norm = self.add_child("mixer_norm", build_part("norm", mixer_norm))
        self.mixer = self.add_child("mixer", build_part("mixer", mixer))
        self.ff_norm = self.add_child("ff_norm", build_part("norm", ff_norm))
        self.feed_forward = self.add_child("feed_forward", build_part("feed_forward", feed_forward))

    def forward(self, ctx, residual, delta, cache):
        h = self.mixer_norm.forward(ctx, residual, delta)
        d = self.mixer.forward(ctx, h, cache)
        h = self.ff_norm.forward(ctx, residual, d)
        d = self.feed_forward.forward(ctx, h)
        return residual, d


@register_part("block", "parallel")
class ParallelBlock(Block):
    """``h = norm(x); x += mixer(h) + feed_forward(h)``.  The two results travel to the next norm as a
    float32 stack ``[2, T, H]`` and are added to the float32 residual there, so the sum is never rounded
    to 16 bits.  ``feed_forward`` None: the layer has a mixer only."""

    def __init__(self, mixer: PartSpec, norm: PartSpec, feed_forward: Optional[PartSpec] = None):
        self.norm = self.add_child("norm", build_part("norm", norm))
        self.mixer = self.add_child("mixer", build_part("mixer", mixer))
        self.feed_forward = (self.add_child("feed_forward", build_part("feed_forward", feed_forward))
                             if feed_forward is not None else None)

    def forward(self, ctx, residual, delta, cache):
        h = self.norm.forward(ctx, residual, delta)
        d_mix = self.mixer.forward(ctx, h, cache)
        if self.feed_forward is None:
            return residual, d_mix
        d_ff = self.feed_forward.forward(ctx, h)
        return residual, ops.stack_deltas(ctx, (d_mix, d_ff))
