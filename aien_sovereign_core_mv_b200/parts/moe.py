"""Routed feed-forward: a router, small experts, an optional shared expert."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from ..registry import register_feed_forward
from .base import FeedForward, StepContext
from .linear import linear


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    """Every token uses ``top`` of ``num_experts`` experts.  Router logits z = W_r h and the scores
    s = softmax(z) over all experts are float32.  With ``group_count`` > 1 the experts form that
    many equal groups of neighbours, a group scores its best expert and only experts of the best
    ``group_keep`` groups can be chosen.  The chosen experts' outputs are summed with their scores
    as weights (``renormalise``: divided by the sum of the chosen scores).  An expert is
    W_down f(W_up h) without biases and without a gate, f the gelu in its erf form ("gelu") or its
    tanh form ("gelu_tanh").  ``shared_ff`` > 0: one more expert of that hidden size runs for
    every token and is added.

    ``forward`` returns ``(parts, shared)``: the weighted outputs of the chosen experts as parts
    [top, T, H], one per choice (float32, or bfloat16 from the grouped tensor-core products), and
    the shared expert's output (or None); whoever takes the branch adds them in that order, in float32.  Expert tensors are stacked [E, ...] when they arrive."""

    def __init__(self, hidden_size: int, expert_ff: int, num_experts: int, top: int, group_count: int = 1, group_keep: int = 1,
                 shared_ff: int = 0, act: str = "gelu", shared_act: Optional[str] = None, renormalise: bool = False):
        self.hidden_size, self.expert_ff, self.num_experts, self.top = int(hidden_size), int(expert_ff), int(num_experts), int(top)
        self.group_count, self.group_keep = int(group_count or 1), int(group_keep or 1)
        self.shared_ff = int(shared_ff or 0)
        if act not in K.ACT_KINDS or (shared_act or act) not in K.ACT_KINDS:
            raise ValueError(f"expert activation {act!r} / {shared_act!r}: one of {sorted(K.ACT_KINDS)}")
        self.act, self.shared_act = K.ACT_KINDS[act], K.ACT_KINDS[shared_act or act]
        self.renormalise = bool(renormalise)
        E, G = self.num_experts, self.group_count
        if E <= 0 or G <= 0 or E % G:
            raise ValueError(f"{E} experts do not form {G} equal groups")
        if not (0 < self.group_keep <= G):
            raise ValueError(f"group_keep {self.group_keep} of {G} groups")
        if not (0 < self.top <= self.group_keep * (E // G)):
            raise ValueError(f"top {self.top} exceeds the {self.group_keep * (E // G)} experts that stay eligible")
        self.w_router = self.w_up = self.w_down = self.w_shared_up = self.w_shared_down = self.expert_count = None

    def param_shapes(self):
        H, F = self.hidden_size, self.expert_ff
        shapes = {"router": ((self.num_experts, H), "matrix")}
        for e in range(self.num_experts):
            shapes[f"experts.{e}.up"] = ((F, H), "matrix")
            shapes[f"experts.{e}.down"] = ((H, F), "matrix")
        if self.shared_ff:
            shapes["shared.up"] = ((self.shared_ff, H), "matrix")
            shapes["shared.down"] = ((H, self.shared_ff), "matrix")
        return shapes

    def bind(self, tensors):
        # Router logits are float32 sums.  A float32 engine keeps the matrix in float32 and multiplies on the CUDA
        # cores; a bfloat16 engine multiplies the stored bfloat16 matrix by the bfloat16 copy of the stream on the
        # products it uses everywhere (every product of two bfloat16 numbers is exact in float32; the sums are float32).
        self.w_router = tensors["router"].contiguous()
        ups = [tensors[f"experts.{e}.up"] for e in range(self.num_experts)]
        downs = [tensors[f"experts.{e}.down"] for e in range(self.num_experts)]
        if len({t.dtype for t in ups + downs}) > 1:
            ups, downs = [t.float() for t in ups], [t.float() for t in downs]
        self.w_up = torch.stack(ups, dim=0).contiguous()                # [E, F, H]
        self.w_down = torch.stack(downs, dim=0).contiguous()            # [E, H, F]
        # choices per expert: the router's kernel counts, the plan of the grouped products reads and zeroes them again
        self.expert_count = torch.zeros(self.num_experts, dtype=torch.int32, device=self.w_up.device)
        if self.shared_ff:
            self.w_shared_up = tensors["shared.up"].contiguous()
            self.w_shared_down = tensors["shared.down"].contiguous()

    def workspace_bytes(self, lim):
        T = lim.max_tokens
        return T * (self.num_experts * 4 + self.top * 8 + self.top * self.expert_ff * lim.itemsize + self.top * self.hidden_size * 4
                    + self.shared_ff * lim.itemsize + self.hidden_size * 4) + 16384 + 2 * K.PARTIALS_MAX_BYTES \
            + K.moe_workspace_bytes(lim, self.num_experts, self.top, self.hidden_size, self.expert_ff)

    def forward(self, ctx: StepContext, h: torch.Tensor):
        T, top = ctx.num_tokens, self.top
        ws = ctx.workspace
        if h.dtype == torch.bfloat16 and self.w_router.dtype == torch.bfloat16:
            z = linear(ctx, h, self.w_router, out_dtype=torch.float32)
        else:
            z = ws.take((T, self.num_experts), torch.float32)
            K.gemm_simple(h, self.w_router, z)                          # float32 operands, float32 sums
        ids = ws.take((T, top), torch.int32)
        wts = ws.take((T, top), torch.float32)
        counts = self.expert_count if K.moe_takes_grouped(h, self.w_up, self.w_down) else None
        K.moe_route(z, self.group_count, self.group_keep, top, self.renormalise, ids, wts, counts)
        parts = K.moe_experts(ctx, h, self.w_up, self.w_down, ids, wts, top, self.act, counts)
        shared = None
        if self.shared_ff:
            a = linear(ctx, h, self.w_shared_up, act=self.shared_act)          # the activation in the product's epilogue
            # beside bfloat16 routed parts (the grouped products) the shared expert's output is bfloat16 too; else float32
            shared = linear(ctx, a, self.w_shared_down, out_dtype=torch.bfloat16 if counts is not None else torch.float32, may_defer_sum=True)
        return parts, shared
