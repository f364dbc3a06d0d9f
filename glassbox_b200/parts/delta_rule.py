"""A gated delta-rule mixer with one decay per head and key channel.

h -> one stacked product gives q and k (num_kv_heads x key_dim each), v (num_heads x value_dim), the inputs of the two
low-rank maps (decay, output gate) and beta's logits. q, k, v pass a short causal convolution along the request's
tokens (its last taps - 1 inputs live in the request's state slot) and SiLU; q and k become unit vectors per head, q
also times key_dim^(-1/2). Per head, with S [key_dim, value_dim] from the request's state slot, token by token:

    S <- diag(g) S,  g = exp(-exp(A_log) * softplus(W_a2 (W_a1 h) + dt_bias))   (one decay per key channel)
    u = beta (v - S^T k),  beta = sigmoid(W_b h)
    S <- S + k u^T
    o = S^T q                                                                   (the read-out sees the token's own write)

o is RMS-normed per head (gain shared by heads), times sigmoid(W_g2 (W_g1 h)), and projected by W_o. The state, the
decays, beta, the unit vectors and the norm are float32 whatever the activation dtype: the stacked product and the two
second-level products write float32.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.binding import ParamSpec
from .base import Mixer, StateSpec, register_part
from .linear import linear


#: With few requests a decode step is a chain of short kernels and every launch saved counts: the fused form (three
#: launches fewer per layer) wins. With many, every block of the fused form reads its head's slice of the two low-rank
#: matrices again, half as many bytes as S itself, and the products done once for all rows win. Measured, ms per step
#: fused / not, 8 layers: width 1024 batch 1 0.335 / 0.360, batch 8 0.390 / 0.452, batch 64 0.834 / 0.820; width 2048
#: batch 64 1.568 / 1.482.
FUSE_DECODE_MAX_ROWS = 16


class ChannelDelta(Mixer):
    accepts_deferred_input = True
    launches_through_kernels_only = True
    can_overwrite_output = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        s = spec
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ValueError(f"num_heads {s.num_heads} is not a multiple of num_kv_heads {s.num_kv_heads}")
        if not 0 < s.key_dim <= 1024 or s.value_dim <= 0:
            raise ValueError(f"key_dim {s.key_dim} must lie in 1..1024 and value_dim {s.value_dim} be positive")
        if not 1 <= s.conv_taps <= 64:
            raise ValueError(f"conv_taps {s.conv_taps} must lie in 1..64")
        if s.decay_rank <= 0 or s.gate_rank <= 0:
            raise ValueError("the low-rank maps of the decay and of the gate need a positive rank")
        self.hidden_size = hidden_size
        self.H, self.KH, self.dk, self.dv, self.taps = s.num_heads, s.num_kv_heads, s.key_dim, s.value_dim, s.conv_taps
        self.qk_cols, self.v_cols = self.KH * self.dk, self.H * self.dv
        self.conv_cols = 2 * self.qk_cols + self.v_cols
        # columns of the stacked product: q | k | v | decay map input | gate map input | beta logits
        self.a1_at = self.conv_cols
        self.g1_at = self.a1_at + s.decay_rank
        self.b_at = self.g1_at + s.gate_rank
        self.in_cols = self.b_at + self.H
        self.state_numbers = self.H * self.dk * self.dv
        self.conv_state_at = self.state_numbers

    def param_specs(self):
        d, s = self.hidden_size, self.spec
        return {
            "w_in": ParamSpec((self.in_cols, d), pieces=(self.qk_cols, self.qk_cols, self.v_cols, s.decay_rank, s.gate_rank, self.H)),
            "conv": ParamSpec((self.conv_cols, self.taps), role="gain", pieces=(self.qk_cols, self.qk_cols, self.v_cols)),
            "w_a2": ParamSpec((self.H * self.dk, s.decay_rank)),
            "w_g2": ParamSpec((self.v_cols, s.gate_rank)),
            "dt_bias": ParamSpec((self.H * self.dk,), role="gain"),
            "a_log": ParamSpec((self.H,), role="gain"),
            "out_norm": ParamSpec((self.dv,), role="gain"),
            "wo": ParamSpec((d, self.v_cols)),
        }

    def cache_spec(self):
        """One float32 row per request: S [heads, key_dim, value_dim], then the convolutions' last taps - 1 inputs
        [taps - 1, q | k | v channels]."""
        return StateSpec((self.state_numbers + (self.taps - 1) * self.conv_cols,), torch.float32)

    def forward(self, ctx, h, residual, cache, writes_cache: bool) -> None:
        n = h.shape[0]
        s = self.spec
        f32 = torch.float32
        ld = -(-self.in_cols // 4) * 4                      # rows of the float32 buffers start 16-byte aligned
        proj = ctx.scratch("delta_proj", (n, ld), f32)[:, :self.in_cols]
        linear(ctx, h, self.params["w_in"], proj)
        state = cache.state
        att = ctx.scratch("att", (n, self.v_cols))
        beta = proj[:, self.b_at:self.b_at + self.H]
        decode = ctx.decode_only and kernels.channel_delta_decode_supported(self.dk, self.dv)
        if decode and n <= FUSE_DECODE_MAX_ROWS and kernels.DeltaDecodeFusion.supported(self.params["w_a2"], self.params["w_g2"]):
            # one token per request: convolutions, low-rank products, recurrence, read-out norm and gate in one kernel
            # that reads and writes S once, in whole rows; then the convolutions' last inputs move up by one
            fusion = kernels.DeltaDecodeFusion(proj, self.params["conv"], self.conv_state_at, self.a1_at, self.params["w_a2"],
                                               self.params["w_g2"])
            kernels.channel_delta_decode(None, beta, None, self.params["dt_bias"], self.params["a_log"], state, None,
                                         self.params["out_norm"], s.norm_eps, att, ctx.seq_first_row, ctx.seq_start_pos,
                                         ctx.seq_slots, self.H, self.KH, self.dk, self.dv, writes_cache, ctx.status, fusion=fusion)
            if writes_cache and self.taps > 1:
                kernels.short_conv_state(proj[:, :self.conv_cols], state, self.conv_state_at, self.taps, ctx.seq_first_row,
                                         ctx.seq_start_pos, ctx.seq_slots)
        else:
            decay = ctx.scratch("delta_decay", (n, self.H * self.dk), f32)
            gate = ctx.scratch("delta_gate", (n, self.v_cols), f32)
            linear(ctx, proj[:, self.a1_at:self.a1_at + s.decay_rank], self.params["w_a2"], decay)
            linear(ctx, proj[:, self.g1_at:self.g1_at + s.gate_rank], self.params["w_g2"], gate)
            qkv = ctx.scratch("delta_qkv", (n, self.conv_cols), f32)
            kernels.short_conv(proj[:, :self.conv_cols], self.params["conv"], qkv, state, self.conv_state_at, ctx.row_seq,
                               ctx.positions, ctx.seq_first_row, ctx.seq_start_pos, ctx.seq_slots, writes_cache, ctx.status)
            if decode:
                kernels.channel_delta_decode(qkv, beta, decay, self.params["dt_bias"], self.params["a_log"], state, gate,
                                             self.params["out_norm"], s.norm_eps, att, ctx.seq_first_row, ctx.seq_start_pos,
                                             ctx.seq_slots, self.H, self.KH, self.dk, self.dv, writes_cache, ctx.status)
            else:
                o = ctx.scratch("delta_o", (n, self.v_cols), f32)
                kernels.channel_delta(qkv, beta, decay, self.params["dt_bias"], self.params["a_log"], state, o, ctx.seq_first_row,
                                      ctx.seq_start_pos, ctx.seq_slots, self.H, self.KH, self.dk, self.dv, writes_cache, ctx.status)
                kernels.gated_head_norm(o, gate, self.params["out_norm"], att, self.H, s.norm_eps)
        linear(ctx, att, self.params["wo"], residual, accumulate=not getattr(ctx, "overwrite_output", False))


register_part("mixer", "channel_delta", ChannelDelta, replace=True)


class HeadDelta(Mixer):
    """The gated delta rule with ONE decay per head and token, g = exp(-exp(A_log_h) * softplus(w_a_h . x + dt_bias_h)), whose
    decay and output gate are plain projections of the input: one stacked product gives q | k | v | decay logits (heads) |
    beta logits (heads) | gate logits (heads x value_dim) as float32 sums; the rest is ``ChannelDelta``'s path on the same
    kernels (convolutions and SiLU of q, k, v with their last inputs in the request's slot, unit vectors, the recurrence,
    the read-out's RMS norm per head with a gain shared by the heads), with silu(gate) or sigmoid(gate) on the way out."""
    accepts_deferred_input = True
    launches_through_kernels_only = True
    can_overwrite_output = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        s = spec
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ValueError(f"num_heads {s.num_heads} is not a multiple of num_kv_heads {s.num_kv_heads}")
        if not 0 < s.key_dim <= 1024 or s.value_dim <= 0:
            raise ValueError(f"key_dim {s.key_dim} must lie in 1..1024 and value_dim {s.value_dim} be positive")
        if not 1 <= s.conv_taps <= 64:
            raise ValueError(f"conv_taps {s.conv_taps} must lie in 1..64")
        if s.gate not in ("silu", "sigmoid"):
            raise ValueError(f"gate {s.gate!r} must be 'silu' or 'sigmoid'")
        self.hidden_size = hidden_size
        self.H, self.KH, self.dk, self.dv, self.taps = s.num_heads, s.num_kv_heads, s.key_dim, s.value_dim, s.conv_taps
        self.qk_cols, self.v_cols = self.KH * self.dk, self.H * self.dv
        self.conv_cols = 2 * self.qk_cols + self.v_cols
        self.a_at = self.conv_cols
        self.b_at = self.a_at + self.H
        self.g_at = self.b_at + self.H
        self.in_cols = self.g_at + self.v_cols
        self.state_numbers = self.H * self.dk * self.dv
        self.conv_state_at = self.state_numbers

    def param_specs(self):
        d = self.hidden_size
        return {
            "w_in": ParamSpec((self.in_cols, d), pieces=(self.qk_cols, self.qk_cols, self.v_cols, self.H, self.H, self.v_cols)),
            "conv": ParamSpec((self.conv_cols, self.taps), role="gain", pieces=(self.qk_cols, self.qk_cols, self.v_cols),
                              init=(0.0, 0.5)),
            "dt_bias": ParamSpec((self.H,), role="gain", init=(0.0, 1.0)),
            "a_log": ParamSpec((self.H,), role="gain", init=(-1.0, 1.0)),
            "out_norm": ParamSpec((self.dv,), role="gain"),
            "wo": ParamSpec((d, self.v_cols)),
        }

    def cache_spec(self):
        """One float32 row per request: S [heads, key_dim, value_dim], then the convolutions' last taps - 1 inputs
        [taps - 1, q | k | v channels]."""
        return StateSpec((self.state_numbers + (self.taps - 1) * self.conv_cols,), torch.float32)

    def forward(self, ctx, h, residual, cache, writes_cache: bool) -> None:
        n = h.shape[0]
        s, p = self.spec, self.params
        f32 = torch.float32
        ld = -(-self.in_cols // 4) * 4                      # rows of the float32 buffers start 16-byte aligned
        proj = ctx.scratch("delta_proj", (n, ld), f32)[:, :self.in_cols]
        linear(ctx, h, p["w_in"], proj)
        state = cache.state
        decay = proj[:, self.a_at:self.a_at + self.H]
        beta = proj[:, self.b_at:self.b_at + self.H]
        gate = proj[:, self.g_at:self.g_at + self.v_cols]
        qkv = ctx.scratch("delta_qkv", (n, self.conv_cols), f32)
        kernels.short_conv(proj[:, :self.conv_cols], p["conv"], qkv, state, self.conv_state_at, ctx.row_seq, ctx.positions,
                           ctx.seq_first_row, ctx.seq_start_pos, ctx.seq_slots, writes_cache, ctx.status)
        att = ctx.scratch("att", (n, self.v_cols))
        silu = s.gate == "silu"
        if ctx.decode_only and kernels.channel_delta_decode_supported(self.dk, self.dv):
            kernels.channel_delta_decode(qkv, beta, decay, p["dt_bias"], p["a_log"], state, gate, p["out_norm"], s.norm_eps, att,
                                         ctx.seq_first_row, ctx.seq_start_pos, ctx.seq_slots, self.H, self.KH, self.dk, self.dv,
                                         writes_cache, ctx.status, decay_per_head=True, gate_silu=silu)
        else:
            o = ctx.scratch("delta_o", (n, self.v_cols), f32)
            kernels.channel_delta(qkv, beta, decay, p["dt_bias"], p["a_log"], state, o, ctx.seq_first_row, ctx.seq_start_pos,
                                  ctx.seq_slots, self.H, self.KH, self.dk, self.dv, writes_cache, ctx.status, decay_per_head=True)
            kernels.gated_head_norm(o, gate, p["out_norm"], att, self.H, s.norm_eps, gate_silu=silu)
        linear(ctx, att, p["wo"], residual, accumulate=not getattr(ctx, "overwrite_output", False))


register_part("mixer", "head_delta", HeadDelta, replace=True)
