"""Two mixers side by side: both read the same input, and the output is left_scale * left + right_scale * right.

Either mixer may be any registered one; their caches share the layer's cache layer (at most one of them may keep pages, any
may keep a state per request: ``combine_cache_specs``). Each writes its output into a float32 buffer of its own (as under
a wiring that norms a branch: ``ctx.overwrite_output``); one small kernel forms the weighted sum and stores it or adds it
into the residual, in float32.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import Mixer, build_part, combine_cache_specs, register_part, sub_view


class ParallelMixer(Mixer):
    can_overwrite_output = True
    launches_through_kernels_only = False      # (clearing the buffer for a part that adds is a torch operation)

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        self.hidden_size = hidden_size
        self.left = build_part("mixer", spec.left, hidden_size=hidden_size)
        self.right = build_part("mixer", spec.right, hidden_size=hidden_size)

    def sub_parts(self):
        return {"left": self.left, "right": self.right}

    def recordable(self, decode_only: bool) -> bool:
        return True

    def cache_spec(self):
        return combine_cache_specs([("left", self.left.cache_spec()), ("right", self.right.cache_spec())])

    def forward(self, ctx, h, residual, cache, writes_cache: bool) -> None:
        n, d = residual.shape
        overwrite = getattr(ctx, "overwrite_output", False)
        outs = []
        for name, part in (("left", self.left), ("right", self.right)):
            y = ctx.scratch("parallel_" + name, (n, d), torch.float32)
            ctx.overwrite_output = bool(part.can_overwrite_output)
            if not ctx.overwrite_output:
                y.zero_()
            try:
                part.forward(ctx, h, y, sub_view(cache, name, part.cache_spec()), writes_cache)
            finally:
                ctx.overwrite_output = overwrite
            outs.append(y)
        kernels.scaled_sum(outs[0], outs[1], self.spec.left_scale, self.spec.right_scale, residual, accumulate=not overwrite)


register_part("mixer", "parallel", ParallelMixer, replace=True)
