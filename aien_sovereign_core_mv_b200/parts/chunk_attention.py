"""Grouped-query attention with a chunk mask, a softmax sink and keys that double as values."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from ..registry import register_mixer
from .base import CacheNeed, Mixer, Position, RunBinding, StepContext
from .linear import linear


@register_mixer("chunked_sink_attention")
class ChunkedSinkAttention(Mixer):
    """One product over the stacked rows q | k (there is no value projection when
    ``values_from_keys``: a value is the first ``value_dim`` numbers of its key as projected,
    before rotation and norm), rotation of neighbouring pairs over the first ``rotary_dim``
    dimensions, then (``unit_qk``) q and k divided by their root mean square per head, a norm
    without a weight.  Scores are q.k * ``scale``.  Masks: causal, and with ``chunk`` > 0 a token
    sees only the keys of its own chunk of that many positions (chunks counted from position 0 of
    the sequence, whatever way the prompt was cut); ``window`` > 0 bounds the keys as well.  With
    ``sink`` every head has one learned number whose exponential joins the softmax denominator:
    it has no key and no value, is not scaled, and counts once.  Rotation, norm, scores and
    softmax are float32 in both engine precisions.

    The cache keeps two planes per token, the prepared key and the value; with a chunk mask the
    pages before the chunk of the next token are given back (cache kind "chunk")."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position: Position,
                 value_dim: Optional[int] = None, scale: Optional[float] = None, chunk: int = 0, window: int = 0,
                 sink: bool = False, unit_qk: bool = True, unit_eps: float = 1e-6, values_from_keys: bool = True):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if head_dim % 2 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim}: the attention kernels take even sizes up to 256")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.value_dim = int(value_dim if value_dim is not None else head_dim)
        if not (0 < self.value_dim <= self.head_dim) and values_from_keys:
            raise ValueError(f"value_dim {self.value_dim}: a value taken from its key cannot be longer than the key ({self.head_dim})")
        if self.value_dim > 256:
            raise ValueError(f"value_dim {self.value_dim}: the attention kernels take sizes up to 256")
        if getattr(position, "pairing", "interleaved") != "interleaved":
            raise ValueError("this mixer rotates neighbouring pairs (2i with 2i+1): give it a position part with pairing='interleaved'")
        self.position = position
        self.scale = float(scale) if scale is not None else self.head_dim ** -0.5
        self.chunk, self.window = int(chunk or 0), int(window or 0)
        if self.chunk < 0 or self.window < 0:
            raise ValueError("chunk and window must not be negative")
        self.sink, self.unit_qk, self.unit_eps = bool(sink), bool(unit_qk), float(unit_eps)
        self.values_from_keys = bool(values_from_keys)
        self.q_dim, self.k_dim, self.v_dim = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim, self.num_kv_heads * self.value_dim
        self.o_in = self.num_heads * self.value_dim
        self.w_qk = self.w_o = self.sinks = None

    # ---- tensors
    def param_shapes(self):
        H = self.hidden_size
        shapes = {"q_proj": ((self.q_dim, H), "matrix"), "k_proj": ((self.k_dim, H), "matrix"), "o_proj": ((H, self.o_in), "matrix")}
        if not self.values_from_keys:
            shapes["v_proj"] = ((self.v_dim, H), "matrix")
        if self.sink:
            shapes["sink"] = ((self.num_heads,), "vector")
        return shapes

    def bind(self, tensors):
        rows = [tensors["q_proj"], tensors["k_proj"]] + ([] if self.values_from_keys else [tensors["v_proj"]])
        if len({t.dtype for t in rows}) > 1:
            rows = [t.float() for t in rows]
        self.w_qk = torch.cat(rows, dim=0).contiguous()                 # rows q | k (| v)
        self.w_o = tensors["o_proj"].contiguous()
        if self.sink:
            self.sinks = tensors["sink"].float().contiguous()           # the softmax is float32

    def cache_need(self):
        planes = (("k", (self.num_kv_heads, self.head_dim)), ("v", (self.num_kv_heads, self.value_dim)))
        if self.chunk > 0 and (self.window == 0 or self.window >= self.chunk):
            return CacheNeed("chunk", self.chunk, planes)
        if self.window > 0:
            return CacheNeed("window", self.window, planes)
        return CacheNeed("full", 0, planes)

    def workspace_bytes(self, lim):
        rows = self.q_dim + self.k_dim + (0 if self.values_from_keys else self.v_dim)
        return lim.max_tokens * (rows * 4 + self.q_dim * lim.itemsize + self.o_in * lim.itemsize + self.hidden_size * 4) + 8192 \
            + 2 * K.PARTIALS_MAX_BYTES + K.chunk_attention_workspace_bytes(lim, self.num_heads, self.value_dim, self.chunk)

    # ---- one step
    def forward(self, ctx: StepContext, h: torch.Tensor, run: RunBinding):
        T = ctx.num_tokens
        group = ctx.groups[run.group]
        k_cache, v_cache = group.storage["k"][run.slot], group.storage["v"][run.slot]
        if run.writes:
            qk = linear(ctx, h, self.w_qk, out_dtype=torch.float32, may_defer_sum=True)          # float32 into the rotation and norm
            q, k = qk[..., :self.q_dim], qk[..., self.q_dim:self.q_dim + self.k_dim]
            v = None if self.values_from_keys else qk[..., self.q_dim + self.k_dim:]
        else:
            q = linear(ctx, h, self.w_qk[:self.q_dim], out_dtype=torch.float32, may_defer_sum=True)
            k = v = None
        rot = self.position.rotary(ctx)
        cos, sin, rdim = rot if rot is not None else (None, None, 0)
        q_out = ctx.workspace.take((T, self.q_dim), ctx.dtype)
        K.qk_rope_pairs_unit_kv_write(q, k, v, self.head_dim, self.value_dim, self.unit_qk, self.unit_eps, cos, sin, rdim,
                                      group.slot_map if k is not None else None, k_cache if k is not None else None,
                                      v_cache if k is not None else None, q_out)
        out = ctx.workspace.take((T, self.o_in), ctx.dtype)
        K.chunk_sink_attention(ctx, q_out, k_cache, v_cache, group, out, self.num_heads, self.num_kv_heads, self.head_dim,
                               self.value_dim, self.window, self.chunk, self.sinks, self.scale)
        return linear(ctx, out, self.w_o, out_dtype=torch.float32, may_defer_sum=True)
