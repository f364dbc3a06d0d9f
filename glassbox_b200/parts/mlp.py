"""Dense gated feed-forward (SwiGLU): residual += (silu(h Wgate^T) * (h Wup^T)) Wdown^T, gate rows
then up rows stacked in one matrix, SiLU as g / (1 + exp(-g)), no bias
(crates/glassbox-core/src/model.rs:327-344; stacking crates/glassbox-core/src/load.rs:62-65)."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.binding import ParamSpec
from .base import FeedForward, register_part
from .linear import clamped_glu_linear, gated_linear, linear, relu2_linear


class SwiGlu(FeedForward):
    accepts_deferred_input = True
    launches_through_kernels_only = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        self.hidden_size = hidden_size
        self.inter = spec.intermediate_size

    def param_specs(self):
        d, i = self.hidden_size, self.inter
        return {"w_gate_up": ParamSpec((2 * i, d), pieces=(i, i)), "w_down": ParamSpec((d, i))}

    def forward(self, ctx, h, residual) -> None:
        n = h.shape[0]
        act = ctx.scratch("act", (n, self.inter))
        if not gated_linear(ctx, h, self.params["w_gate_up"], act):
            gate_up = ctx.scratch("gate_up", (n, 2 * self.inter))
            linear(ctx, h, self.params["w_gate_up"], gate_up)
            kernels.swiglu(gate_up, act)
        linear(ctx, act, self.params["w_down"], residual, accumulate=True)


class GeluGlu(FeedForward):
    """Dense gated feed-forward whose gate passes the tanh form of GELU: residual += (gelu_tanh(h Wgate^T) * (h Wup^T)) Wdown^T,
    gate rows then up rows stacked in one matrix, no bias. The unit is formed in float32 from the float32 sums of the first
    product."""
    accepts_deferred_input = True
    launches_through_kernels_only = True
    can_overwrite_output = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        self.hidden_size = hidden_size
        self.inter = spec.intermediate_size

    def param_specs(self):
        d, i = self.hidden_size, self.inter
        return {"w_gate_up": ParamSpec((2 * i, d), pieces=(i, i)), "w_down": ParamSpec((d, i))}

    def forward(self, ctx, h, residual) -> None:
        n = h.shape[0]
        act = ctx.scratch("act", (n, self.inter))
        if not gated_linear(ctx, h, self.params["w_gate_up"], act, unit="gelu_tanh"):
            gate_up = ctx.scratch("gate_up32", (n, 2 * self.inter), torch.float32)
            linear(ctx, h, self.params["w_gate_up"], gate_up)
            kernels.gelu_glu(gate_up, act)
        linear(ctx, act, self.params["w_down"], residual, accumulate=not getattr(ctx, "overwrite_output", False))


class SquaredRelu(FeedForward):
    """Dense feed-forward without a gate: residual += (relu(h Wup^T))^2 Wdown^T, no bias."""
    accepts_deferred_input = True
    launches_through_kernels_only = True
    can_overwrite_output = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        self.hidden_size = hidden_size
        self.inter = spec.intermediate_size

    def param_specs(self):
        d, i = self.hidden_size, self.inter
        return {"w_up": ParamSpec((i, d)), "w_down": ParamSpec((d, i))}

    def forward(self, ctx, h, residual) -> None:
        n = h.shape[0]
        act = ctx.scratch("act", (n, self.inter))
        if not relu2_linear(ctx, h, self.params["w_up"], act):
            up = ctx.scratch("ffn_up", (n, self.inter))
            linear(ctx, h, self.params["w_up"], up)
            kernels.relu2(up, act)
        linear(ctx, act, self.params["w_down"], residual, accumulate=not getattr(ctx, "overwrite_output", False))


class ClampedGlu(FeedForward):
    """Dense gated feed-forward with clamped branches: g = min(x Wgate^T + b_gate, limit), u = clamp(x Wup^T + b_up, -limit,
    limit), residual += (g * sigmoid(slope * g) * (u + 1)) Wdown^T + b_down. Gate rows then up rows stacked in one matrix
    (and one bias vector). The clamps, the sigmoid and the product are formed in float32 from the float32 sums of the first
    product. A wiring that norms the branch takes the down projection's bias over (``ctx.accepts_output_bias``) and adds
    it on its way over the rows; otherwise a small kernel adds it."""
    launches_through_kernels_only = True
    can_overwrite_output = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        if not spec.limit > 0:
            raise ValueError(f"limit {spec.limit} must be positive")
        self.hidden_size = hidden_size
        self.inter = spec.intermediate_size

    def param_specs(self):
        d, i = self.hidden_size, self.inter
        specs = {"w_gate_up": ParamSpec((2 * i, d), pieces=(i, i)), "w_down": ParamSpec((d, i))}
        if self.spec.bias:
            specs["b_gate_up"] = ParamSpec((2 * i,), role="gain", pieces=(i, i), init=(0.0, 0.5))
            specs["b_down"] = ParamSpec((d,), role="gain", init=(0.0, 0.5))
        return specs

    def forward(self, ctx, h, residual) -> None:
        n, s, p = h.shape[0], self.spec, self.params
        act = ctx.scratch("act", (n, self.inter))
        if not clamped_glu_linear(ctx, h, p["w_gate_up"], p.get("b_gate_up"), s.limit, s.slope, act):
            gate_up = ctx.scratch("gate_up32", (n, 2 * self.inter), torch.float32)
            linear(ctx, h, p["w_gate_up"], gate_up)
            kernels.clamped_glu(gate_up, p.get("b_gate_up"), s.limit, s.slope, act)
        overwrite = getattr(ctx, "overwrite_output", False)
        linear(ctx, act, p["w_down"], residual, accumulate=not overwrite)
        if "b_down" in p:
            if overwrite and getattr(ctx, "accepts_output_bias", False):
                ctx.output_bias = p["b_down"]
            else:
                kernels.add_bias(residual, p["b_down"])


register_part("ffn", "clamped_glu", ClampedGlu, replace=True)
register_part("ffn", "swiglu", SwiGlu, replace=True)
register_part("ffn", "gelu_glu", GeluGlu, replace=True)
register_part("ffn", "relu2", SquaredRelu, replace=True)
