"""Linear attention with one fixed decay per head.

h -> one stacked product gives q, k (heads x head_dim each), v (heads x value_dim) and the output gate's logits (heads x
value_dim) as float32 sums -> q, k and v pass SiLU -> per head, with S [head_dim, value_dim] from the request's state slot,
token by token:

    S <- decay_h S + k v^T
    o = S^T q                                         (no other scale)

-> the heads' read-outs are RMS-normed together (one gain per channel of the concatenation), times sigmoid(gate), projected by
W_o. The state, SiLU, the read-out, its norm and the gate are float32 whatever the activation dtype. The recurrence runs on
the delta rule's kernel with the correction towards the value switched off: it is the same walk over tokens with S in
registers, without beta, unit vectors and the dot product with the key.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.binding import ParamSpec
from .base import Mixer, StateSpec, register_part
from .linear import linear


class DecayLinearAttention(Mixer):
    accepts_deferred_input = True
    launches_through_kernels_only = True
    can_overwrite_output = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        s = spec
        if s.num_heads <= 0 or not 0 < s.head_dim <= 1024 or s.value_dim <= 0:
            raise ValueError(f"heads {s.num_heads}, head_dim {s.head_dim} (1..1024) and value_dim {s.value_dim} must be positive")
        if len(s.decay) != s.num_heads or not all(0.0 <= float(g) <= 1.0 for g in s.decay):
            raise ValueError(f"decay must hold one number in [0, 1] per head ({s.num_heads}), got {list(s.decay)!r}")
        self.hidden_size = hidden_size
        self.H, self.dk, self.dv = s.num_heads, s.head_dim, s.value_dim
        self.qk_cols, self.v_cols = self.H * self.dk, self.H * self.dv
        self.gate_at = 2 * self.qk_cols + self.v_cols
        self.in_cols = self.gate_at + self.v_cols
        self._decay = None

    def param_specs(self):
        d = self.hidden_size
        return {"w_in": ParamSpec((self.in_cols, d), pieces=(self.qk_cols, self.qk_cols, self.v_cols, self.v_cols)),
                "out_norm": ParamSpec((self.v_cols,), role="gain"),
                "wo": ParamSpec((d, self.v_cols))}

    def cache_spec(self):
        """One float32 row per request: S [heads, head_dim, value_dim]."""
        return StateSpec((self.H * self.dk * self.dv,), torch.float32)

    def forward(self, ctx, h, residual, cache, writes_cache: bool) -> None:
        n = h.shape[0]
        f32 = torch.float32
        if self._decay is None or self._decay.device != ctx.device:
            self._decay = torch.tensor([float(g) for g in self.spec.decay], dtype=f32, device=ctx.device)
        ld = -(-self.in_cols // 4) * 4                      # rows of the float32 buffer start 16-byte aligned
        proj = ctx.scratch("lin_proj", (n, ld), f32)[:, :self.in_cols]
        linear(ctx, h, self.params["w_in"], proj)
        o = ctx.scratch("lin_o", (n, self.v_cols), f32)
        args = (proj[:, :self.gate_at], self._decay, cache.state, o, ctx.seq_first_row, ctx.seq_start_pos, ctx.seq_slots, self.H, self.dk,
                self.dv, writes_cache, ctx.status)
        if ctx.decode_only and kernels.channel_delta_decode_supported(self.dk, self.dv):
            # single tokens: the form that reads and writes S once, in whole rows
            kernels.decay_linear_attention_decode(*args, silu_inputs=True)
        elif kernels.linear_piece_rows(ctx.max_rows_per_seq, self.H, self.dk, self.dv):
            # a long portion: its pieces walk side by side, their states are chained afterwards (the decay is a constant)
            piece_rows = kernels.linear_piece_rows(ctx.max_rows_per_seq, self.H, self.dk, self.dv)
            pieces = kernels.linear_pieces_needed(n, ctx.seq_start_pos.shape[0], piece_rows)
            meta = ctx.scratch("lin_piece_meta", (1, 4 * pieces + 2 * ctx.seq_start_pos.shape[0] + 1), torch.int32, grow=True)
            piece_state = ctx.scratch("lin_piece_state", (pieces, self.H * self.dk * self.dv), f32, grow=True)
            kernels.decay_linear_attention_pieces(*args, meta.view(-1), piece_state, silu_inputs=True, piece_rows=piece_rows)
        else:
            kernels.decay_linear_attention(*args, silu_inputs=True)
        att = ctx.scratch("att", (n, self.v_cols))
        # the norm runs over the concatenated heads: one "head" of heads * value_dim channels
        kernels.gated_head_norm(o, proj[:, self.gate_at:], self.params["out_norm"], att, 1, self.spec.norm_eps)
        linear(ctx, att, self.params["wo"], residual, accumulate=not getattr(ctx, "overwrite_output", False))


register_part("mixer", "decay_linear_attention", DecayLinearAttention, replace=True)
