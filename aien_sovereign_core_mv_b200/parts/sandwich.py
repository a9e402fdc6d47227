"""A layer that norms every sublayer's input and its output, with a scaled residual sum, and an optional
per-token side input after the feed-forward."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from ..registry import make_part, register_block, register_side
from .base import Block, FeedForward, Mixer, Norm, NormedStream, Part, RunBinding, StepContext, add_to_residual
from .linear import linear


@register_side("gated_token_table")
class GatedTokenTable(Part):
    """y = W_proj (gelu_tanh(W_gate x) * e) with e = ``dim`` columns, from ``column`` on, of the row that a second
    embedding table holds for the token; x is the residual stream as it stands.  The table belongs to the model's
    embedding part (``Embedding.side_table``), which every layer's side input shares.  ``norm`` is the RMS norm (plain
    weight) that the block puts on y before it sums it into the stream."""

    def __init__(self, hidden_size: int, dim: int, column: int, eps: float):
        self.hidden_size, self.dim, self.column = int(hidden_size), int(dim), int(column)
        self.norm = make_part("norm", "rmsnorm", size=self.hidden_size, eps=float(eps))
        self.w_gate = self.w_proj = self.table = None

    def param_shapes(self):
        return {"gate": ((self.dim, self.hidden_size), "matrix"), "proj": ((self.hidden_size, self.dim), "matrix"),
                "norm": ((self.hidden_size,), "norm")}

    def bind(self, tensors):
        self.w_gate, self.w_proj = tensors["gate"].contiguous(), tensors["proj"].contiguous()
        self.norm.bind({"weight": tensors["norm"]})

    def tie_embedding(self, embedding) -> None:
        table = embedding.side_table() if hasattr(embedding, "side_table") else None
        if table is None or table.shape[1] < self.column + self.dim:
            raise ValueError("a layer's side input needs an embedding part with a side table wide enough for its columns")
        self.table = table

    def workspace_bytes(self, lim):
        return lim.max_tokens * (self.dim * 8 + self.hidden_size * 4) + 4096

    def forward(self, ctx: StepContext, hx: torch.Tensor) -> torch.Tensor:
        z = linear(ctx, hx, self.w_gate, out_dtype=torch.float32)
        g = ctx.workspace.take((ctx.num_tokens, self.dim), ctx.dtype)
        K.gelu_times_table(z, self.table, self.column, ctx.token_ids, g)
        return linear(ctx, g, self.w_proj, out_dtype=torch.float32)


@register_block("sandwich")
class SandwichBlock(Block):
    """x <- x + m * norm_out(mixer(norm_in(x))); x <- x + m * norm_ff_out(ff(norm_ff_in(x))); with a side input then
    x <- x + m * side.norm(side(x)).  ``residual_mult`` is m.  Every sum is made here, in float32, by the kernel that
    also makes what the next sublayer reads (its input norm, or the stream's compute-dtype copy for the side input), so
    one kernel runs between two sublayers.  The block hands the next block its first norm's output (``NormedStream``)
    when that block says which norm it starts with.  A layer without a feed-forward is the kind "sandwich_mixer"."""

    norm_slots = ("norm_in", "norm_out", "norm_ff_in", "norm_ff_out")
    chains_norm = True

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], norm_in: Norm, norm_out: Norm,
                 norm_ff_in: Optional[Norm] = None, norm_ff_out: Optional[Norm] = None, residual_mult: float = 1.0,
                 side: Optional[dict] = None):
        if (feed_forward is None) != (norm_ff_in is None) or (feed_forward is None) != (norm_ff_out is None):
            raise ValueError("a sandwich block has a feed-forward and its two norms, or none of the three")
        if not hasattr(norm_out, "add_normed_scaled") or (norm_ff_out is not None and not hasattr(norm_ff_out, "add_normed_scaled")):
            raise ValueError("the output norms of a sandwich block must offer add_normed_scaled")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.norm_in, self.norm_out, self.norm_ff_in, self.norm_ff_out = norm_in, norm_out, norm_ff_in, norm_ff_out
        self.mult = float(residual_mult)
        self.side = None
        if side:
            params = {k: v for k, v in dict(side).items() if k != "kind"}
            self.side = make_part("side", side["kind"], **params)

    def parts(self):
        out = {"norm_in": self.norm_in, "mixer": self.mixer, "norm_out": self.norm_out}
        if self.feed_forward is not None:
            out.update({"norm_ff_in": self.norm_ff_in, "feed_forward": self.feed_forward, "norm_ff_out": self.norm_ff_out})
        if self.side is not None:
            out["side"] = self.side
        return out

    def workspace_bytes(self, lim):
        return sum(p.workspace_bytes(lim) for p in self.parts().values()) + 4 * (lim.max_tokens * self.norm_in.size * lim.itemsize + 256)

    def first_norm(self):
        return self.norm_in

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, run: RunBinding, next_norm: Optional[Norm] = None):
        if isinstance(delta, NormedStream) and delta.norm is self.norm_in:
            h = delta.h
        else:
            add_to_residual(ctx, x, delta)
            h = self.norm_in.forward(ctx, x, None)
        # what follows each sum: the feed-forward's input norm, the side input's copy of the stream, the next block's norm
        stages = [(self.norm_out, lambda hh: self.mixer.forward(ctx, hh, run))]
        if self.feed_forward is not None:
            stages.append((self.norm_ff_out, lambda hh: self.feed_forward.forward(ctx, hh)))
        if self.side is not None:
            stages.append((self.side.norm, lambda hh: self.side.forward(ctx, hh)))
        for i, (post, run_sublayer) in enumerate(stages):
            a = run_sublayer(h)
            last = i + 1 == len(stages)
            if last:
                h = post.add_normed_scaled(ctx, x, a, self.mult, then=next_norm)
            elif stages[i + 1][0] is self.norm_ff_out:
                h = post.add_normed_scaled(ctx, x, a, self.mult, then=self.norm_ff_in)
            else:
                h = post.add_normed_scaled(ctx, x, a, self.mult, want_copy=True)
        return NormedStream(h, next_norm) if (next_norm is not None and h is not None) else None


@register_block("sandwich_mixer")
class SandwichMixerBlock(SandwichBlock):
    """The sandwich block of a layer that has no feed-forward."""

    norm_slots = ("norm_in", "norm_out")

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], norm_in: Norm, norm_out: Norm,
                 residual_mult: float = 1.0, side: Optional[dict] = None):
        if feed_forward is not None:
            raise ValueError("the block kind 'sandwich_mixer' takes no feed-forward")
        super().__init__(mixer, None, norm_in, norm_out, None, None, residual_mult, side)
