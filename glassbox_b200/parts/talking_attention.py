"""Causal grouped-query softmax attention whose heads exchange their weights after the softmax.

h -> one stacked product gives q (heads x head_dim), k (kv heads x head_dim), v (kv heads x value_dim) as float32 sums ->
biases are added, the leading channels of every query and key head are rotated (channel i with channel i + rot/2; the (cos,
sin) table carries a stretching of the frequencies and its factor, if the position spec has one), k and v go into the paged
cache at the row's slot (all rows of the step before any attention) -> per (row, head g), over the row's visible keys of its
own request: s_j = q . k_j * scale, capped as cap * tanh(s_j / cap), weights w_g(j) = exp(s_j) / (1 + sum_j' exp(s_j')): the
added one is a key of score 0 without a value -> head h's output is sum_j (sum_g talk[h, g] w_g(j)) v_c(h)(j), with c(h) the
key/value head of h -> residual (+)= out Wo^T.

The mix of the weights is linear, so it is taken out of the sum over keys: O[g, c] = sum_j w_g(j) v_c(j) is formed for every
query head g and every key/value head c in one pass with a running maximum per head (each head's softmax stays its own),
and out_h = sum_g talk[h, g] O[g, c(h)] is a small second kernel. Biases, angles, scores, weights, the sums over keys and the
mix are float32 whatever the activation dtype; the cache holds the activation dtype.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.binding import ParamSpec
from .base import Mixer, PagedKvSpec, build_part, register_part
from .linear import linear


def pick_kernel(dtype, single_tokens: bool, heads: int, kv_heads: int, dim: int, vdim: int, value_heads: int) -> str:
    """Which attention kernel a step takes: "decode" (single decoded tokens, a block of warps per (row, head) that share the
    row's keys), "tiles" (prompt portions in bfloat16 on the tensor cores) or "rows" (one warp per (row, head): float32
    portions, sizes the others are not built for)."""
    if single_tokens and kernels.talking_attention_decode_supported(dtype, heads, kv_heads, vdim, value_heads):
        return "decode"
    if not single_tokens and kernels.talking_attention_tiles_supported(dtype, dim, vdim, value_heads):
        return "tiles"
    return "rows"


class TalkingAttention(Mixer):
    accepts_deferred_input = True
    launches_through_kernels_only = True
    can_overwrite_output = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        s = spec
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ValueError(f"num_heads {s.num_heads} is not a multiple of num_kv_heads {s.num_kv_heads}")
        if not 0 < s.head_dim <= 256 or not 0 < s.value_dim <= 256:
            raise ValueError(f"head_dim {s.head_dim} and value_dim {s.value_dim} must lie in 1..256")
        if s.talk and s.num_kv_heads * s.value_dim > 2048:
            raise ValueError(f"{s.num_kv_heads} key/value heads of {s.value_dim} channels: mixing the heads takes at most 2048 in all")
        if s.softcap is not None and not s.softcap > 0:
            raise ValueError(f"softcap {s.softcap} must be positive")
        if s.window is not None and s.window <= 0:
            raise ValueError(f"window {s.window} must be positive")
        self.hidden_size = hidden_size
        self.H, self.G, self.D, self.V = s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim
        self.in_cols = (self.H + self.G) * self.D + self.G * self.V
        self.position = build_part("position", s.position)
        self.rot = self.position.rotary_dim
        if self.rot > self.D:
            raise ValueError(f"{self.rot} rotated channels are more than head_dim {self.D}")
        if self.rot and getattr(self.position, "pairing", "half") != "half":
            raise ValueError("this mixer rotates channel i with channel i + rot/2 (pairing 'half')")

    def param_specs(self):
        d, s = self.hidden_size, self.spec
        pieces = (self.H * self.D, self.G * self.D, self.G * self.V)
        specs = {"w_in": ParamSpec((self.in_cols, d), pieces=pieces), "wo": ParamSpec((d, self.H * self.V))}
        if s.bias:
            specs["b_in"] = ParamSpec((self.in_cols,), role="gain", pieces=pieces, init=(0.0, 0.3))
        if s.talk:
            specs["talk"] = ParamSpec((self.H, self.H), role="gain", init=(1.0 / self.H, 0.5 / self.H))
        return specs

    def cache_spec(self):
        return PagedKvSpec(self.G, self.D, self.spec.window, value_dim=self.V)

    def forward(self, ctx, h, residual, cache, writes_cache: bool) -> None:
        n, s, p = h.shape[0], self.spec, self.params
        ld = -(-self.in_cols // 4) * 4                      # rows of the float32 buffer start 16-byte aligned
        proj = ctx.scratch("tk_proj", (n, ld), torch.float32)[:, :self.in_cols]
        linear(ctx, h, p["w_in"], proj)
        q = ctx.scratch("tk_q", (n, self.H * self.D))
        table = self.position.fused_table(ctx.device) if self.rot else None
        kernels.bias_rope_write(proj, p.get("b_in"), table, ctx.positions, cache.slots, q, cache.k, cache.v, self.H, self.G, self.D,
                                self.V, self.rot, cache.page_size, writes_cache, ctx.status)
        value_heads = self.G if s.talk else 1
        cols = self.H * value_heads * self.V
        how = pick_kernel(q.dtype, ctx.decode_only, self.H, self.G, self.D, self.V, value_heads)
        common = dict(heads=self.H, kv_heads=self.G, dim=self.D, vdim=self.V, value_heads=value_heads, page_size=cache.page_size,
                      scale=s.scale, softcap=s.softcap, unit_sink=s.unit_sink, window=s.window, status=ctx.status)
        shares, ml = 1, None
        if how == "decode":
            # few rows: the keys of a row are cut into shares, so that the blocks fill the chip; the mix merges the shares
            reach = min(ctx.max_context, s.window) if s.window else ctx.max_context
            shares = kernels.talking_decode_shares(n, self.H, self.G, self.V, value_heads, reach)
            wide = ctx.scratch("tk_wide_shares", (n, shares * cols), torch.float32, grow=True)
            ml = ctx.scratch("tk_ml", (n, shares * self.H * 2), torch.float32, grow=True) if shares > 1 else None
            kernels.talking_attention_decode(q, wide, cache.k, cache.v, cache.block_tables, ctx.row_seq, ctx.positions, shares=shares, ml=ml,
                                             **common)
        else:
            wide = ctx.scratch("tk_wide", (n, cols), torch.float32)
            if how == "tiles":
                kernels.talking_attention_tiles(q, wide, cache.k, cache.v, cache.block_tables, ctx.seq_first_row, ctx.seq_start_pos,
                                                ctx.max_rows_per_seq, **common)
            else:
                kernels.talking_attention_rows(q, wide, cache.k, cache.v, cache.block_tables, ctx.row_seq, ctx.positions, **common)
        att = ctx.scratch("att", (n, self.H * self.V))
        kernels.talk_combine(wide, p.get("talk"), att, ctx.positions, self.H, self.G, self.V, value_heads, shares=shares, ml=ml,
                             unit_sink=s.unit_sink)
        linear(ctx, att, p["wo"], residual, accumulate=not getattr(ctx, "overwrite_output", False))


register_part("mixer", "talking_attention", TalkingAttention, replace=True)
