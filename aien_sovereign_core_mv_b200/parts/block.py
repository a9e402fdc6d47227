"""Arrangements of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

from typing import Optional

import torch

from ..registry import register_block
from .. import kernels as K
from .base import Block, FeedForward, Mixer, Norm, Prenormed, RunBinding, StepContext, StreamCopy, add_to_residual


@register_block("prenorm")
class PreNormBlock(Block):
    """x -> norm -> mixer -> +x -> norm -> feed-forward -> +x
    (crates/aien-inference-abi/src/weights.rs:290-365).  Each residual sum is carried as a
    pending ``delta`` and added inside the next norm kernel; or, where the norm and the parts
    around it allow (``Norm.sink``), the product that ends a branch adds it and the product that
    follows finishes the norm, and no norm kernel runs between them."""

    norm_slots = ("norm_in", "norm_post")
    chains_norm = True

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norm_in: Norm, norm_post: Norm):
        self.mixer, self.feed_forward, self.norm_in, self.norm_post = mixer, feed_forward, norm_in, norm_post

    def parts(self):
        return {"norm_in": self.norm_in, "mixer": self.mixer, "norm_post": self.norm_post, "feed_forward": self.feed_forward}

    def workspace_bytes(self, lim):
        return sum(p.workspace_bytes(lim) for p in self.parts().values())

    def first_norm(self):
        return self.norm_in

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, run: RunBinding, next_norm: Optional[Norm] = None):
        h = self.norm_in.forward(ctx, x, delta)
        if isinstance(h, Prenormed) and not self.mixer.takes_prenormed:
            h = h.materialise(ctx)
        sink = self.norm_post.sink(ctx, x) if self.mixer.feeds_residual else None
        a = self.mixer.forward(ctx, h, run, sink=sink) if sink is not None else self.mixer.forward(ctx, h, run)
        h2 = self.norm_post.forward(ctx, x, a)
        if isinstance(h2, Prenormed) and not self.feed_forward.takes_prenormed:
            h2 = h2.materialise(ctx)
        sink = next_norm.sink(ctx, x) if (next_norm is not None and self.feed_forward.feeds_residual) else None
        return self.feed_forward.forward(ctx, h2, sink=sink) if sink is not None else self.feed_forward.forward(ctx, h2)


@register_block("branchnorm")
class BranchNormBlock(Block):
    """x -> x + norm_mixer(mixer(x)) -> x + norm_ff(feed_forward(x)): the sublayers read the
    stream itself and each norm stands on its sublayer's *output*.  Every sum is made here, in
    float32 (``Norm.add_normed``), so the block hands no pending sum on; it hands on the
    compute-dtype copy of the stream that the last sum's kernel wrote (``StreamCopy``), which the
    next block of this kind takes as its mixer's input.  A layer without a feed-forward is the
    kind "branchnorm_mixer"."""

    norm_slots = ("norm_mixer", "norm_ff")

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], norm_mixer: Norm, norm_ff: Optional[Norm] = None):
        if (feed_forward is None) != (norm_ff is None):
            raise ValueError("a branch-norm block has a feed-forward and its norm, or neither")
        self.mixer, self.feed_forward, self.norm_mixer, self.norm_ff = mixer, feed_forward, norm_mixer, norm_ff

    def parts(self):
        out = {"norm_mixer": self.norm_mixer, "mixer": self.mixer}
        if self.feed_forward is not None:
            out["norm_ff"] = self.norm_ff
            out["feed_forward"] = self.feed_forward
        return out

    def workspace_bytes(self, lim):
        return sum(p.workspace_bytes(lim) for p in self.parts().values()) + 3 * (lim.max_tokens * self.norm_mixer.size * lim.itemsize + 256)

    def _stream_copy(self, ctx: StepContext, x: torch.Tensor, delta):
        if isinstance(delta, StreamCopy):
            return delta.h
        add_to_residual(ctx, x, delta)             # whatever another kind of block left pending
        if ctx.dtype == torch.float32:
            return x
        h = ctx.workspace.take(tuple(x.shape), ctx.dtype)
        K.convert(x, h)
        return h

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, run: RunBinding):
        h = self._stream_copy(ctx, x, delta)
        a = self.mixer.forward(ctx, h, run)
        h = self.norm_mixer.add_normed(ctx, x, a, want_copy=True)
        if self.feed_forward is not None:
            f = self.feed_forward.forward(ctx, h)
            a, b = f if isinstance(f, tuple) else (f, None)          # a routed feed-forward returns (routed parts, shared output)
            h = self.norm_ff.add_normed(ctx, x, a, b, want_copy=True)
        return StreamCopy(h)


@register_block("branchnorm_mixer")
class BranchNormMixerBlock(BranchNormBlock):
    """The branch-norm block of a layer that has no feed-forward: x -> x + norm_mixer(mixer(x))."""

    norm_slots = ("norm_mixer",)

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], norm_mixer: Norm):
        if feed_forward is not None:
            raise ValueError("the block kind 'branchnorm_mixer' takes no feed-forward")
        super().__init__(mixer, None, norm_mixer, None)
