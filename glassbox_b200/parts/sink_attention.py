"""Causal grouped-query softmax attention whose positions enter as a bias on the distance, with a sink in the softmax.

x -> one stacked product gives q (heads x head_dim), k (kv heads x head_dim), v (kv heads x value_dim) and one gate logit
per head as float32 sums -> every query and key head is RMS-normed over head_dim (one gain shared by the query heads, one by
the key heads); nothing is rotated -> values: a "source" layer leaves its v rows in a float32 buffer that lives for the
step, a "mixed" layer replaces its v by (1 - lambda) v + lambda v_source of the same token; k and the (mixed) v go into the
paged cache at the row's slot (all rows of the step before any attention) -> per (row, head), over the row's visible keys j
of its own request: s_j = q . k_j * scale - r1_h * ln(1 + r2_h * (i - j)), weights exp(s_j - m) / (sum_j exp(s_j - m) +
exp(sink_h - m)): the sink adds to the denominator and to nothing else -> the head's output times sigmoid(gate logit) ->
residual += out Wo^T. A window w lets position p see keys p-w+1 .. p; pages behind the window of every future query go
back to the pool, as for any windowed paged group. Norms, distances, logarithms, scores, weights, the sums over keys, the
value mix and the gate are float32 whatever the activation dtype; the cache holds the activation dtype.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.binding import ParamSpec
from .base import Mixer, PagedKvSpec, register_part
from .linear import linear

#: name of the step's buffer in which a "source" layer leaves its values for the "mixed" layers after it
VALUE_SOURCE = "value_mix_source"


class SinkAttention(Mixer):
    launches_through_kernels_only = True
    can_overwrite_output = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        s = spec
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ValueError(f"num_heads {s.num_heads} is not a multiple of num_kv_heads {s.num_kv_heads}")
        if not 0 < s.head_dim <= 256 or not 0 < s.value_dim <= 256:
            raise ValueError(f"head_dim {s.head_dim} and value_dim {s.value_dim} must lie in 1..256")
        if s.window is not None and s.window <= 0:
            raise ValueError(f"window {s.window} must be positive")
        if s.value_mix not in ("none", "source", "mixed"):
            raise ValueError(f"value_mix {s.value_mix!r} must be 'none', 'source' or 'mixed'")
        self.hidden_size = hidden_size
        self.H, self.G, self.D, self.V = s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim
        self.gate_col = (self.H + self.G) * self.D + self.G * self.V
        self.in_cols = self.gate_col + (self.H if s.output_gate else 0)

    def param_specs(self):
        d, s = self.hidden_size, self.spec
        pieces = (self.H * self.D, self.G * self.D, self.G * self.V) + ((self.H,) if s.output_gate else ())
        specs = {"w_in": ParamSpec((self.in_cols, d), pieces=pieces), "wo": ParamSpec((d, self.H * self.V))}
        if s.qk_norm_eps is not None:
            specs["q_norm"] = ParamSpec((self.D,), role="gain")
            specs["k_norm"] = ParamSpec((self.D,), role="gain")
        if s.distance_bias:
            specs["r1"] = ParamSpec((self.H,), role="gain", init=(0.5, 0.2))
            specs["r2"] = ParamSpec((self.H,), role="gain", init=(0.3, 0.05))
        if s.sink:
            specs["sink"] = ParamSpec((self.H,), role="gain", init=(0.0, 1.0))
        if s.value_mix == "mixed":
            specs["value_mix"] = ParamSpec((), role="gain", init=(0.4, 0.1))
        return specs

    def cache_spec(self):
        return PagedKvSpec(self.G, self.D, self.spec.window, value_dim=self.V)

    def forward(self, ctx, h, residual, cache, writes_cache: bool) -> None:
        n, s = h.shape[0], self.spec
        ld = -(-self.in_cols // 4) * 4                      # rows of the float32 buffer start 16-byte aligned
        proj = ctx.scratch("sk_proj", (n, ld), torch.float32)[:, :self.in_cols]
        linear(ctx, h, self.params["w_in"], proj)
        q = ctx.scratch("sk_q", (n, self.H * self.D))
        source = ctx.scratch(VALUE_SOURCE, (n, self.G * self.V), torch.float32) if s.value_mix != "none" else None
        kernels.qk_norm_rope_write(proj[:, :self.gate_col], self.params.get("q_norm"), self.params.get("k_norm"), None, ctx.positions,
                                   cache.slots, q, cache.k, cache.v, self.H, self.G, self.D, self.V, 0, s.qk_norm_eps or 0.0,
                                   cache.page_size, writes_cache, ctx.status,
                                   values_out=source if s.value_mix == "source" else None,
                                   values_in=source if s.value_mix == "mixed" else None, value_mix=self.params.get("value_mix"))
        att = ctx.scratch("att", (n, self.H * self.V))
        self.attend(ctx, q, att, cache, proj[:, self.gate_col:] if s.output_gate else None)
        linear(ctx, att, self.params["wo"], residual, accumulate=not getattr(ctx, "overwrite_output", False))

    def attend(self, ctx, q, att, cache, gate) -> None:
        """Single decoded tokens in bfloat16, where key and value size are equal and one the split-key tensor-core
        kernel is built for, take that kernel's instantiation with the bias, the sink and the gate; other single tokens take
        the kernel that shares a row's keys between the warps of a block; prompt portions in bfloat16 run on the tensor
        cores: on the tcgen05 flash kernel's instantiation with the three terms where key and value size are the one it is
        built for, else on the tile kernel at the head sizes that one is built for; everything else (float32 portions, other
        sizes) takes the one-warp-per-(row, head) kernel."""
        p, s = self.params, self.spec
        if (ctx.decode_only and self.D == self.V and q.shape[0] <= 65535
                and kernels.attention_decode_mma_supported(q.dtype, self.H, self.G, self.D, cache.page_size)):
            n = q.shape[0]
            reach = min(ctx.max_context, s.window) if s.window else ctx.max_context      # keys a row can see
            splits, block_keys, warps = kernels.decode_mma_plan(n, self.G, self.D, reach)
            part_acc = ctx.scratch("decode_part_acc", (n, self.H * warps * splits * self.D), torch.float32, grow=True)
            part_ml = ctx.scratch("decode_part_ml", (n, self.H * warps * splits * 2), torch.float32, grow=True)
            counters = ctx.zeros_once("decode_counters", ctx.max_rows * self.H, torch.int32)
            kernels.attention_decode_mma(q, att, cache.k, cache.v, cache.block_tables, ctx.row_seq, ctx.positions, self.H, self.G,
                                         self.D, cache.page_size, s.scale, s.window, splits, part_acc, part_ml, counters, ctx.status,
                                         block_keys, warps, sink_terms=(p.get("r1"), p.get("r2"), p.get("sink"), gate))
            return
        common = dict(r1=p.get("r1"), r2=p.get("r2"), sink=p.get("sink"), gate=gate, heads=self.H, kv_heads=self.G, dim=self.D,
                      vdim=self.V, page_size=cache.page_size, scale=s.scale, window=s.window, status=ctx.status)
        if ctx.decode_only and kernels.sink_attention_decode_supported(q.dtype, self.V):
            kernels.sink_attention_decode(q, att, cache.k, cache.v, cache.block_tables, ctx.row_seq, ctx.positions, **common)
            return
        if (not ctx.decode_only and self.D == self.V
                and kernels.attention_prefill_tc_supported(q, att, self.H, self.G, self.D, cache.page_size)):
            kernels.attention_prefill_tc(q, att, cache.k, cache.v, cache.block_tables, ctx.seq_first_row, ctx.seq_start_pos,
                                         ctx.max_rows_per_seq, self.H, self.G, self.D, cache.page_size, s.scale, s.window, ctx.status,
                                         sink_terms=(p.get("r1"), p.get("r2"), p.get("sink"), gate))
            return
        if not ctx.decode_only and kernels.sink_attention_tiles_supported(q.dtype, self.D, self.V):
            kernels.sink_attention_tiles(q, att, cache.k, cache.v, cache.block_tables, ctx.seq_first_row, ctx.seq_start_pos,
                                         ctx.max_rows_per_seq, **common)
            return
        kernels.sink_attention_rows(q, att, cache.k, cache.v, cache.block_tables, ctx.row_seq, ctx.positions, **common)


register_part("mixer", "sink_attention", SinkAttention, replace=True)
