"""A routed feed-forward: a mixture of small squared-ReLU experts, of which each token uses a few, beside an optional
shared expert that every token uses.

Router: logits = W_router h in float32, scores s = sigmoid(logits). An expert is *chosen* by s + correction (a stored
number per expert), but *weighs* s * route_scale: the correction steers the choice only. The experts form `num_groups`
equal runs of neighbours; a run scores the sum of its two largest choice scores, and only experts of the `keep_groups`
best runs can be chosen (the others count as minus infinity; choice scores may be negative). The `top_k` largest remaining
choice scores win, the lowest index among equals. The weights are not renormalised.

With `scoring` "softmax_chosen" the router is plainer: logits = W_router h + router_bias in float32, the `top_k` largest
logits win (the lowest index among equals), and the weights are the softmax over the chosen logits alone.

Expert: W_down relu(W_up h)^2, no biases; or, with `activation` "clamped_glu", W_down (g * sigmoid(slope * g) * (u + 1)) with
g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit): the up parameter then holds, per expert, gate row f and up row
f as neighbours (rows 2f and 2f + 1), so that a product's neighbouring outputs are the two inputs of one unit. Output: sum over the chosen experts of weight * expert(h), plus, if there is a
shared expert, sigmoid(w_gate . h) * shared(h) (one gate number per token; without a gate the shared output is added as
it is). The experts' matrices are stacked by rows into two parameters, so a kernel finds expert e at row e * size.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.binding import ParamSpec
from .base import FeedForward, register_part
from .linear import linear, relu2_linear


#: up to this many rows the experts run as weight-streaming kernels per (row, choice); above it (bfloat16) as grouped
#: tensor-core products over the pairs sorted by expert
GROUPED_ABOVE_ROWS = 16


class RoutedExperts(FeedForward):
    launches_through_kernels_only = True
    can_overwrite_output = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        s = spec
        if s.num_experts <= 0 or not 0 < s.top_k <= s.num_experts or s.expert_size <= 0:
            raise ValueError(f"{s.num_experts} experts of {s.expert_size}, {s.top_k} per token: not a mixture")
        if s.num_groups < 1 or s.num_experts % s.num_groups or not 1 <= s.keep_groups <= s.num_groups:
            raise ValueError(f"{s.num_experts} experts do not form {s.num_groups} equal groups of which {s.keep_groups} are kept")
        if s.keep_groups * (s.num_experts // s.num_groups) < s.top_k:
            raise ValueError(f"{s.keep_groups} groups of {s.num_experts // s.num_groups} experts cannot supply {s.top_k} per token")
        if s.scoring not in ("sigmoid", "softmax_chosen") or s.activation not in ("relu2", "clamped_glu"):
            raise ValueError(f"scoring {s.scoring!r} / activation {s.activation!r} are not known")
        if s.scoring == "softmax_chosen" and (s.num_groups != 1 or s.correction):
            raise ValueError("softmax weights over the chosen logits go with neither groups nor a choice correction")
        if s.activation == "clamped_glu" and not s.limit > 0:
            raise ValueError(f"limit {s.limit} must be positive")
        self.hidden_size = hidden_size
        self.E, self.top, self.ff, self.shared = s.num_experts, s.top_k, s.expert_size, s.shared_size
        self.glu = s.activation == "clamped_glu"

    def param_specs(self):
        d, E, ff = self.hidden_size, self.E, self.ff
        up_rows = 2 * ff if self.glu else ff            # gated: an expert's gate matrix, then its up matrix
        specs = {"router": ParamSpec((E, d), role="gain", init=(0.0, 0.1)),
                 "w_up": ParamSpec((E * up_rows, d), pieces=(ff,) * (E * up_rows // ff)),
                 "w_down": ParamSpec((E * d, ff), pieces=(d,) * E)}
        if self.spec.router_bias:
            specs["router_bias"] = ParamSpec((E,), role="gain", init=(0.0, 0.1))
        if self.spec.correction:
            specs["correction"] = ParamSpec((E,), role="gain", init=(0.0, 0.1))
        if self.shared:
            specs["shared_up"] = ParamSpec((self.shared, d))
            specs["shared_down"] = ParamSpec((d, self.shared))
            if self.spec.shared_gate:
                specs["shared_gate"] = ParamSpec((1, d), role="gain", init=(0.0, 0.05))
        return specs

    def bind(self, params) -> None:
        super().bind(params)
        if self.glu:
            # [expert, gate | up, f, :] -> [expert, f, gate | up, :]: the two inputs of unit f become neighbouring rows
            w = self.params["w_up"]
            self.params["w_up"] = w.view(self.E, 2, self.ff, w.shape[1]).permute(0, 2, 1, 3).contiguous().view(w.shape)

    def forward(self, ctx, h, residual) -> None:
        n, d, s = h.shape[0], self.hidden_size, self.spec
        p = self.params
        unit = (s.limit, s.glu_slope) if self.glu else None
        choice = ctx.scratch("moe_choice", (n, self.top), torch.int32)
        weight = ctx.scratch("moe_weight", (n, self.top), torch.float32)
        gate = ctx.scratch("moe_gate", (n, 1), torch.float32) if "shared_gate" in p else None
        kernels.moe_route(h, p["router"], p.get("correction"), p.get("shared_gate"), ctx.positions, self.top, s.num_groups,
                          s.keep_groups, s.route_scale, choice, weight, gate, router_bias=p.get("router_bias"),
                          softmax_chosen=s.scoring == "softmax_chosen")
        shared_out = None
        if self.shared:
            # the shared expert is a dense squared-ReLU feed-forward: the framework's products, activation in the epilogue
            act = ctx.scratch("act", (n, self.shared))
            if not relu2_linear(ctx, h, p["shared_up"], act):
                up = ctx.scratch("ffn_up", (n, self.shared))
                linear(ctx, h, p["shared_up"], up)
                kernels.relu2(up, act)
            shared_out = ctx.scratch("moe_shared", (n, d), torch.float32)
            linear(ctx, act, p["shared_down"], shared_out)
        pair = ctx.scratch("moe_pair", (n, self.top * d), torch.float32)
        if n > GROUPED_ABOVE_ROWS and kernels.moe_grouped_supported(h.dtype, d, self.ff):
            # many rows: the pairs sorted by expert, one grouped product per half on the tensor cores
            tables = ctx.zeros_once(f"moe_tables_{self.E}_{self.top}", 2 * (self.E + 1) + ctx.max_rows * self.top, torch.int32)
            act = ctx.scratch("moe_act", (n, self.top * self.ff))
            kernels.moe_experts_grouped(h, p["w_up"], p["w_down"], self.E, choice, ctx.positions, tables, act, pair, unit=unit)
        else:
            # few rows (or float32): the chosen experts' matrices streamed once per (row, choice), many blocks each
            act = ctx.scratch("moe_act32", (n, self.top * self.ff), torch.float32)
            kernels.moe_expert_halves(h, p["w_up"], p["w_down"], self.E, choice, ctx.positions, act, pair, unit=unit)
        if getattr(ctx, "overwrite_output", False) and getattr(ctx, "accepts_weighted_rows", False):
            # whoever wired this branch forms the weighted sum itself, on its way over the rows (one launch and one trip
            # to memory less): the output is handed over as its parts
            ctx.weighted_rows = kernels.WeightedRows(pair, weight, shared_out, gate)
            return
        kernels.moe_combine(pair, weight, shared_out, gate, ctx.positions, residual,
                            accumulate=not getattr(ctx, "overwrite_output", False))


register_part("ffn", "routed_experts", RoutedExperts, replace=True)
