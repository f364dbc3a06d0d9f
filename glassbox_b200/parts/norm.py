"""Norms. RMSNorm: out_j = w_j * (x_j / sqrt(mean(x^2) + eps)), statistics in float32, no mean
subtraction, no bias, the gain used as stored (crates/glassbox-core/src/model.rs:94-100)."""
from __future__ import annotations

from .. import kernels
from ..weights.binding import ParamSpec
from .base import Norm, register_part


class RmsNorm(Norm):
    launches_through_kernels_only = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        self.eps = float(spec.eps)
        self.hidden_size = hidden_size

    def param_specs(self):
        return {"weight": ParamSpec((self.hidden_size,), role="gain")}

    def forward(self, ctx, x, out, rows=None) -> None:
        kernels.rmsnorm(x, self.params["weight"], out, self.eps, rows)

    def as_rms(self):
        return self.params["weight"], self.eps

    def add_normed(self, ctx, y, x, bias=None, copy=None) -> None:
        kernels.rmsnorm_add(y, self.params["weight"], x, self.eps, bias=bias, copy=copy)


class UnitOffsetRmsNorm(RmsNorm):
    """RMSNorm whose weight is stored around zero: out_j = (1 + w_j) * (x_j / sqrt(mean(x^2) + eps)). The gain 1 + w is
    formed once, in float32, when the weights arrive; from then on this is an RMSNorm with that gain, and everything
    that folds or fuses an RMSNorm takes it as one."""

    def bind(self, params) -> None:
        super().bind(params)
        self.params["weight"] = (self.params["weight"].float() + 1.0).contiguous()


class ResidualItself(Norm):
    """No norm at all: a branch that reads the residual as it is gets its rows in the activation dtype (rounded once). It
    stands where a wiring names "the norm that reads the residual next", so that whoever completes the residual rows can
    tell that the next reader wants them as they are."""
    launches_through_kernels_only = True

    def __init__(self, spec=None, *, hidden_size: int = 0):
        super().__init__(spec)
        self.hidden_size = hidden_size

    def forward(self, ctx, x, out, rows=None) -> None:
        kernels.cast_rows(x, out, rows)


class LayerNorm(Norm):
    """out_j = (x_j - mean) / sqrt(var + eps) * w_j + b_j over a row, var the mean of the squared deviations; statistics
    and the result in float32, rounded once to the activation dtype. The bias is optional (``spec.bias``)."""
    launches_through_kernels_only = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        self.eps = float(spec.eps)
        self.hidden_size = hidden_size

    def param_specs(self):
        specs = {"weight": ParamSpec((self.hidden_size,), role="gain")}
        if self.spec.bias:
            specs["bias"] = ParamSpec((self.hidden_size,), role="gain", init=(0.0, 0.02))
        return specs

    def as_layernorm(self):
        """(weight, bias or None, eps): what a kernel that forms the row itself needs to apply this norm on the way."""
        return self.params["weight"], self.params.get("bias"), self.eps

    def forward(self, ctx, x, out, rows=None) -> None:
        kernels.streams_step(x, 1, norm=self.as_layernorm(), h=out, rows=rows)


register_part("norm", "none", ResidualItself, replace=True)
register_part("norm", "layernorm", LayerNorm, replace=True)
register_part("norm", "rmsnorm", RmsNorm, replace=True)
register_part("norm", "rmsnorm_unit_offset", UnitOffsetRmsNorm, replace=True)
