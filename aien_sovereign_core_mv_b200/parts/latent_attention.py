"""Attention whose keys and values are made from one cached latent per token."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from ..registry import register_mixer
from .base import CacheNeed, Mixer, Position, RunBinding, StepContext
from .linear import linear


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    """Queries through a latent: c_q = RMSnorm(W_dq h) (weight ``dq_norm``), q = W_uq c_q, per head ``head_dim``
    unrotated then ``rot_dim`` rotated numbers.  Keys and values through a latent: W_dkv h has ``kv_rank`` + ``rot_dim``
    rows; the first kv_rank, RMS-normed (weight ``dkv_norm``), are the latent c, the rest one rotated key part shared by
    all heads.  Per head the unrotated key is W_uk c and the value W_uv c; score = (q_unrot . k_unrot + q_rot . k_rot) *
    ``scale``; causal, optionally only the last ``window`` positions (the token itself included); optionally a learned
    sink per head in the softmax denominator; W_o on the heads.  The rotation turns neighbouring pairs of the first
    ``rotary_dim`` numbers of the rotated part (the position part's table).

    The cache keeps one row [c | k_rot] per token and nothing per head.  The kernels never build a head's keys or
    values: W_uk is applied to the query (q_lat = W_uk,h^T q_unrot) and W_uv to the weighted sum of latents, so a cached
    row serves every head as key and as value.  ``own_cache`` False: the layer has no W_dkv and attends over the rows
    another layer wrote (its run binding names that layer's planes).  ``cache_window``: how many positions the cache
    must keep, when layers that share it have different windows (default: ``window``)."""

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, value_dim: int, kv_rank: int, q_rank: int,
                 position: Position, scale: Optional[float] = None, window: int = 0, cache_window: Optional[int] = None,
                 sink: bool = False, norm_eps: float = 1e-6, own_cache: bool = True):
        self.hidden_size, self.num_heads, self.head_dim, self.rot_dim = int(hidden_size), int(num_heads), int(head_dim), int(rot_dim)
        self.value_dim, self.kv_rank, self.q_rank = int(value_dim), int(kv_rank), int(q_rank)
        if min(self.num_heads, self.head_dim, self.value_dim, self.kv_rank, self.q_rank) <= 0 or self.rot_dim < 0:
            raise ValueError("latent attention: heads, head_dim, value_dim, kv_rank and q_rank must be positive")
        if self.rot_dim and getattr(position, "pairing", "interleaved") != "interleaved":
            raise ValueError("this mixer rotates neighbouring pairs (2i with 2i+1): give it a position part with pairing='interleaved'")
        self.position = position
        self.rotary_dim = int(getattr(position, "rotary_dim", 0) or 0) if self.rot_dim else 0
        if self.rotary_dim > self.rot_dim:
            raise ValueError(f"the position part rotates {self.rotary_dim} numbers, the rotated part has {self.rot_dim}")
        self.scale = float(scale) if scale is not None else (self.head_dim + self.rot_dim) ** -0.5
        self.window = int(window or 0)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        if self.window < 0 or (self.window == 0) != (self.cache_window == 0) or self.cache_window < self.window:
            raise ValueError("cache_window must cover window (0 for both: every earlier position is seen)")
        self.sink, self.norm_eps, self.own_cache = bool(sink), float(norm_eps), bool(own_cache)
        self.q_head = self.head_dim + self.rot_dim
        self.row = self.kv_rank + self.rot_dim
        self.w_down = self.w_uq = self.w_uk_t = self.w_uv = self.w_o = self.dq_norm = self.dkv_norm = self.sinks = None

    # ---- tensors
    def param_shapes(self):
        H, n = self.hidden_size, self.num_heads
        shapes = {"dq_proj": ((self.q_rank, H), "matrix"), "dq_norm": ((self.q_rank,), "norm"),
                  "uq_proj": ((n * self.q_head, self.q_rank), "matrix"), "uk_proj": ((n * self.head_dim, self.kv_rank), "matrix"),
                  "uv_proj": ((n * self.value_dim, self.kv_rank), "matrix"), "o_proj": ((H, n * self.value_dim), "matrix")}
        if self.own_cache:
            shapes.update({"dkv_proj": ((self.row, H), "matrix"), "dkv_norm": ((self.kv_rank,), "norm")})
        if self.sink:
            shapes["sink"] = ((n,), "vector")
        return shapes

    def bind(self, tensors):
        rows = [tensors["dq_proj"]] + ([tensors["dkv_proj"]] if self.own_cache else [])
        if len({t.dtype for t in rows}) > 1:
            rows = [t.float() for t in rows]
        self.w_down = torch.cat(rows, dim=0).contiguous()              # rows query latent | key/value latent | shared key part
        self.w_uq, self.w_o = tensors["uq_proj"].contiguous(), tensors["o_proj"].contiguous()
        n = self.num_heads
        # per head [kv_rank, head_dim]: the matrix that takes a head's unrotated query to the latent
        self.w_uk_t = tensors["uk_proj"].view(n, self.head_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors["uv_proj"].view(n, self.value_dim, self.kv_rank).contiguous()
        self.dq_norm = tensors["dq_norm"].contiguous()
        if self.own_cache:
            self.dkv_norm = tensors["dkv_norm"].to(self.dq_norm.dtype).contiguous()
        if self.sink:
            self.sinks = tensors["sink"].float().contiguous()           # the softmax is float32

    def cache_need(self):
        planes = (("latent", (self.row,)),)
        return CacheNeed("window", self.cache_window, planes) if self.cache_window > 0 else CacheNeed("full", 0, planes)

    def workspace_bytes(self, lim):
        n = self.num_heads
        per_token = (self.q_rank + self.row) * 4 + self.q_rank * lim.itemsize + n * self.q_head * 4 + n * self.row * 4 \
            + n * self.kv_rank * lim.itemsize + n * self.value_dim * lim.itemsize + self.hidden_size * 4
        # the partial results of a step with few tiles: tokens * heads * ksplit rows, which latent_attention_tc_ksplit keeps
        # below 296 tiles' worth of 64 rows
        split = 296 * K.LATENT_TC_TILE * (self.kv_rank + 2) * 4
        return lim.max_tokens * per_token + 16384 + split + K.PARTIALS_MAX_BYTES

    # ---- one step
    def forward(self, ctx: StepContext, h: torch.Tensor, run: RunBinding):
        T, n, ws = ctx.num_tokens, self.num_heads, ctx.workspace
        group = ctx.groups[run.group]
        cache = group.storage["latent"][run.slot]                       # [tokens of the pool, kv_rank + rot_dim]
        writes = run.writes and self.own_cache
        if run.writes and not self.own_cache:
            raise RuntimeError("a latent-attention layer without its own key/value projection was bound to write a cache")
        w_down = self.w_down if writes else self.w_down[:self.q_rank]
        d = linear(ctx, h, w_down, out_dtype=torch.float32)
        rot = self.position.rotary(ctx) if self.rotary_dim else None
        cos, sin, rdims = rot if rot is not None else (None, None, 0)
        cq = ws.take((T, self.q_rank), ctx.dtype)
        K.latent_prepare(d, self.q_rank, self.dq_norm, self.norm_eps, cq, self.q_rank, self.kv_rank, self.rot_dim, rdims,
                         self.dkv_norm, cos, sin, group.slot_map if writes else None, cache if writes else None)
        tc = K.latent_attention_tc_supports(cache.dtype, self.kv_rank, self.rot_dim) and ctx.dtype == torch.bfloat16
        # per head: unrotated | rotated part, before rotation; an operand of the tensor-core products where those run
        q = linear(ctx, cq, self.w_uq, out_dtype=torch.bfloat16 if tc else torch.float32)
        qf = ws.take((T, n * self.row), torch.bfloat16 if tc else torch.float32)    # per head: the query in the latent | rotated part
        K.head_project(q, self.q_head, 0, self.w_uk_t, qf, self.row, 0)
        if self.rot_dim:
            K.rotate_pairs_rows(q, self.q_head, self.head_dim, qf, self.row, self.kv_rank, n, self.rot_dim, rdims, cos, sin)
        mixed = ws.take((T, n * self.kv_rank), ctx.dtype)
        if tc:
            small = K.latent_attention_tc_small_tiles(ctx.decode_only, self.kv_rank)
            ksplit = K.latent_attention_tc_ksplit(T, ctx.num_seqs, n, ctx.max_ctx_len, self.window, small)
            scratch = ws.take((K.latent_attention_tc_scratch(T, n, self.kv_rank, ksplit),), torch.float32) if ksplit > 1 else None
            K.latent_attention_tc(qf, cache, group.block_table, group.max_blocks, ctx.q_start, ctx.positions, mixed, ctx.num_seqs, n,
                                  self.kv_rank, self.rot_dim, group.page_size, self.window, self.scale, self.sinks, ksplit, scratch, small)
        else:
            K.latent_attention(qf, cache, group.block_table, group.max_blocks, ctx.seq_of_token, ctx.positions, mixed, n, self.kv_rank,
                               self.rot_dim, group.page_size, self.window, self.scale, self.sinks)
        o = ws.take((T, n * self.value_dim), ctx.dtype)
        K.head_project(mixed, self.kv_rank, 0, self.w_uv, o, self.value_dim, 0)
        return linear(ctx, o, self.w_o, out_dtype=torch.float32, may_defer_sum=True)     # the branch norm adds partial products
