"""A layer: a mixer and a feed-forward wired around the float32 residual stream.

"pre_norm" is x += mixer(norm(x)); x += ffn(norm(x)), with no norms after the parts
(crates/glassbox-core/src/model.rs:251-348; a layer may lack the feed-forward). "sandwich_norm" norms each branch on the
way out as well: x += post(mixer(norm(x))); x += post(ffn(norm(x))). "branch_norm" norms them on the way out only: the
branches read the residual itself, x += post(mixer(x)); x += post(ffn(x)). "hyper_connections" keeps the residual as several
streams x_1 .. x_S per token: a branch reads u = sum_s read[s] x_s through its norm, and its output y comes back into all
streams at once, x_t <- sum_s mix[s, t] x_s + write[t] y. The arrangement is looked up by name, so another
wiring (post-norm, parallel branches) is another registered class.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.binding import ParamSpec
from .base import DeferredNorm, Part, StateSpec, build_part, combine_cache_specs, register_part, sub_view
from .norm import ResidualItself


class PreNormBlock(Part):
    launches_through_kernels_only = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        self.hidden_size = hidden_size
        self.mixer_norm = build_part("norm", spec.mixer_norm, hidden_size=hidden_size)
        self.mixer = build_part("mixer", spec.mixer, hidden_size=hidden_size)
        self.ffn = self.ffn_norm = None          # (a layer may be a mixer alone)
        if spec.ffn is not None:
            self.ffn_norm = build_part("norm", spec.ffn_norm, hidden_size=hidden_size)
            self.ffn = build_part("ffn", spec.ffn, hidden_size=hidden_size)

    def sub_parts(self):
        parts = {"mixer_norm": self.mixer_norm, "mixer": self.mixer}
        if self.ffn is not None:
            parts.update({"ffn_norm": self.ffn_norm, "ffn": self.ffn})
        return parts

    def entry_norm(self):
        """The norm that reads the residual first when this layer runs (whoever runs the layer before may tell
        its last product, through ``ctx.next_norm``, to prepare it)."""
        return self.mixer_norm

    def forward(self, ctx, x, cache, writes_cache: bool, after_mixer=None) -> None:
        """``after_mixer`` (optional) is called once the mixer's kernels are launched: the model uses it
        to let the next layer's mixer start its prefetch beside this layer's feed-forward.
        ``ctx.norm_after_layer`` (optional) is the norm that will read ``x`` after this layer."""
        after_layer = getattr(ctx, "norm_after_layer", None)
        h = DeferredNorm(ctx, self.mixer_norm, x)
        # a hint to the product that adds the mixer's output into x
        ctx.next_norm = self.ffn_norm if self.ffn is not None else after_layer
        self.mixer.forward(ctx, h if self.mixer.accepts_deferred_input else h.tensor(), x, cache, writes_cache)
        if after_mixer is not None:
            after_mixer()
        if self.ffn is not None:
            h = DeferredNorm(ctx, self.ffn_norm, x)
            ctx.next_norm = after_layer
            self.ffn.forward(ctx, h if self.ffn.accepts_deferred_input else h.tensor(), x)
        ctx.next_norm = None


class SandwichNormBlock(Part):
    """x += post_norm(mixer(norm(x))), then x += post_norm(ffn(norm(x))) (the second half only if the layer has a
    feed-forward). A branch cannot add into the residual stream itself, because its output is normed first: it is given
    a float32 buffer of the residual's shape instead. Parts that say ``can_overwrite_output`` store their result there
    (``ctx.overwrite_output`` tells them so); for any other part the buffer is cleared and the part adds into it as it
    would into the residual. The post norm then adds the normed branch into x (``Norm.add_normed``)."""
    launches_through_kernels_only = False      # (clearing the buffer for a part that adds is a torch operation)

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        if spec.mixer_post_norm is None or (spec.ffn is not None and spec.ffn_post_norm is None):
            raise ValueError("a sandwich_norm layer needs a norm behind its mixer and behind its feed-forward")
        self.hidden_size = hidden_size
        self.mixer_norm = build_part("norm", spec.mixer_norm, hidden_size=hidden_size)
        self.mixer = build_part("mixer", spec.mixer, hidden_size=hidden_size)
        self.mixer_post_norm = build_part("norm", spec.mixer_post_norm, hidden_size=hidden_size)
        self.ffn = self.ffn_norm = self.ffn_post_norm = None
        if spec.ffn is not None:
            self.ffn_norm = build_part("norm", spec.ffn_norm, hidden_size=hidden_size)
            self.ffn = build_part("ffn", spec.ffn, hidden_size=hidden_size)
            self.ffn_post_norm = build_part("norm", spec.ffn_post_norm, hidden_size=hidden_size)

    def sub_parts(self):
        parts = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "mixer_post_norm": self.mixer_post_norm}
        if self.ffn is not None:
            parts.update({"ffn_norm": self.ffn_norm, "ffn": self.ffn, "ffn_post_norm": self.ffn_post_norm})
        return parts

    def entry_norm(self):
        return self.mixer_norm

    def _branch(self, ctx, part, norm, post, x, run) -> None:
        branch = ctx.scratch("branch", tuple(x.shape), torch.float32)
        ctx.overwrite_output = bool(part.can_overwrite_output)
        if not ctx.overwrite_output:
            branch.zero_()
        h = DeferredNorm(ctx, norm, x)
        try:
            run(h if part.accepts_deferred_input else h.tensor(), branch)
        finally:
            ctx.overwrite_output = False
        post.add_normed(ctx, branch, x)
        ctx.prepared_norm = None         # x has changed behind the back of whatever was prepared from it

    def forward(self, ctx, x, cache, writes_cache: bool, after_mixer=None) -> None:
        ctx.next_norm = None             # no product of this layer completes residual rows: nothing to prepare
        self._branch(ctx, self.mixer, self.mixer_norm, self.mixer_post_norm, x,
                     lambda h, out: self.mixer.forward(ctx, h, out, cache, writes_cache))
        if after_mixer is not None:
            after_mixer()
        if self.ffn is not None:
            self._branch(ctx, self.ffn, self.ffn_norm, self.ffn_post_norm, x, lambda h, out: self.ffn.forward(ctx, h, out))


class BranchNormBlock(Part):
    """x += post_norm(mixer(x)), then x += post_norm(ffn(x)) (the second half only if the layer has a feed-forward): the
    branches read the residual itself, in the activation dtype (a float32 engine hands them the residual where it lies),
    and only their outputs are normed. A branch gets a float32 buffer for its output, as in the sandwich wiring, and may
    leave a bias of its last product to the post norm (``ctx.accepts_output_bias`` / ``ctx.output_bias``). The kernel that
    norms a branch into the residual also writes the new residual rows in the activation dtype when the next reader wants
    them as they are (the feed-forward of this layer; the mixer of the next, if that layer is wired like this one: the
    model says so through ``ctx.norm_after_layer``), so that a branch costs one launch beside its own."""
    launches_through_kernels_only = False      # (clearing the buffer for a part that adds is a torch operation)

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        if spec.mixer_post_norm is None or (spec.ffn is not None and spec.ffn_post_norm is None):
            raise ValueError("a branch_norm layer needs a norm behind its mixer and behind its feed-forward")
        if spec.mixer_norm is not None or spec.ffn_norm is not None:
            raise ValueError("a branch_norm layer has no norm in front of its branches")
        self.hidden_size = hidden_size
        self.entry = ResidualItself(hidden_size=hidden_size)
        self.mixer = build_part("mixer", spec.mixer, hidden_size=hidden_size)
        self.mixer_post_norm = build_part("norm", spec.mixer_post_norm, hidden_size=hidden_size)
        self.ffn = self.ffn_post_norm = None
        if spec.ffn is not None:
            self.ffn = build_part("ffn", spec.ffn, hidden_size=hidden_size)
            self.ffn_post_norm = build_part("norm", spec.ffn_post_norm, hidden_size=hidden_size)

    def sub_parts(self):
        parts = {"mixer": self.mixer, "mixer_post_norm": self.mixer_post_norm}
        if self.ffn is not None:
            parts.update({"ffn": self.ffn, "ffn_post_norm": self.ffn_post_norm})
        return parts

    def entry_norm(self):
        return self.entry

    def _input(self, ctx, x):
        """The residual rows as a branch reads them."""
        ready, ctx.residual_copy = getattr(ctx, "residual_copy", None), None
        if x.dtype == ctx.dtype:
            return x
        if ready is not None and ready[0] == x.data_ptr() and ready[1] == x.shape[0]:
            return ready[2]
        h = ctx.scratch("h", tuple(x.shape))
        self.entry.forward(ctx, x, h)
        return h

    def _branch(self, ctx, part, post, x, run, copy_after: bool) -> None:
        h = self._input(ctx, x)
        branch = ctx.scratch("branch", tuple(x.shape), torch.float32)
        ctx.overwrite_output = bool(part.can_overwrite_output)
        if not ctx.overwrite_output:
            branch.zero_()
        ctx.accepts_output_bias, ctx.output_bias = True, None
        try:
            run(h, branch)
        finally:
            ctx.overwrite_output = ctx.accepts_output_bias = False
        bias, ctx.output_bias = ctx.output_bias, None
        copy = ctx.scratch("h", tuple(x.shape)) if copy_after and x.dtype != ctx.dtype else None
        post.add_normed(ctx, branch, x, bias=bias, copy=copy)
        ctx.prepared_norm = None         # x has changed behind the back of whatever was prepared from it
        if copy is not None:
            ctx.residual_copy = (x.data_ptr(), x.shape[0], copy)

    def forward(self, ctx, x, cache, writes_cache: bool, after_mixer=None) -> None:
        ctx.next_norm = None             # no product of this layer completes residual rows: nothing to prepare
        next_reads_as_is = isinstance(getattr(ctx, "norm_after_layer", None), ResidualItself)
        self._branch(ctx, self.mixer, self.mixer_post_norm, x,
                     lambda h, out: self.mixer.forward(ctx, h, out, cache, writes_cache),
                     copy_after=self.ffn is not None or next_reads_as_is)
        if after_mixer is not None:
            after_mixer()
        if self.ffn is not None:
            self._branch(ctx, self.ffn, self.ffn_post_norm, x, lambda h, out: self.ffn.forward(ctx, h, out),
                         copy_after=next_reads_as_is)


class StreamMixing(Part):
    """The three learned pieces of one branch of a hyper-connection layer over S residual streams: ``read`` [S] (how the
    branch's input is mixed from the streams), ``write`` [S] (how much of the branch's output each stream takes) and
    ``mix`` [S, S], indexed [from, to] (how the streams feed one another meanwhile). Float32."""
    launches_through_kernels_only = True

    def __init__(self, streams: int, learned: bool = True, scale: float = 1.0):
        """``learned`` False: no tensors; the branch reads the plain sum, every stream keeps itself and takes the output
        once. ``scale`` multiplies the branch's output on its way into the streams (it is folded into ``write`` once, in
        float32, when the weights arrive)."""
        super().__init__(None)
        self.streams, self.learned, self.scale = streams, learned, float(scale)

    def param_specs(self):
        if not self.learned:
            return {}
        s = self.streams
        return {"read": ParamSpec((s,), role="gain", init=(1.0 / s, 0.1 / s)), "write": ParamSpec((s,), role="gain", init=(1.0, 0.1)),
                "mix": ParamSpec((s, s), role="gain", init=(1.0 / s, 0.1 / s))}

    def bind(self, params) -> None:
        super().bind(params)
        if self.learned and self.scale != 1.0:
            self.params["write"] = (self.params["write"].float() * self.scale).contiguous()

    def on_device(self, device):
        """(read, mix, write) as the kernel takes them; the constants of an unlearned mixing are made at first use."""
        if not self.learned and "write" not in self.params:
            s = self.streams
            self.params = {"read": torch.ones(s, dtype=torch.float32, device=device),
                           "mix": torch.eye(s, dtype=torch.float32, device=device).contiguous(),
                           "write": torch.full((s,), self.scale, dtype=torch.float32, device=device)}
        return self.params["read"], self.params["mix"], self.params["write"]


class InputConvolution(Part):
    """A causal convolution over time, per channel, added to its own input: h_t <- h_t + sum_j w[:, j] h_(t - taps + 1 + j),
    zeros before a sequence's start; ``weight`` [channels, taps], the last column weighs the current token. The last
    taps - 1 inputs are kept per request (float32) so that a sequence may arrive in portions."""
    launches_through_kernels_only = True

    def __init__(self, channels: int, taps: int):
        super().__init__(None)
        if not 1 <= taps <= 64:
            raise ValueError(f"a convolution of {taps} taps is outside 1..64")
        self.channels, self.taps = channels, taps

    def param_specs(self):
        return {"weight": ParamSpec((self.channels, self.taps), role="gain", init=(0.0, 0.3))}

    def cache_spec(self):
        return StateSpec((max(self.taps - 1, 1) * self.channels,), torch.float32)

    def forward(self, ctx, h, out, state, writes_cache: bool) -> None:
        kernels.residual_conv(h, self.params["weight"], out, state, 0, ctx.row_seq, ctx.positions, ctx.seq_first_row,
                              ctx.seq_start_pos, ctx.seq_slots, writes_cache, ctx.status, single_rows=ctx.decode_only)


class HyperConnectionBlock(Part):
    """A layer over a residual of S streams per token (``xs`` float32 [n, S * d]). For the mixer, then (if the layer has
    one) the feed-forward: u = sum_s read[s] x_s; y = branch(norm(u)); x_t <- sum_s mix[s, t] x_s + write[t] y for all t
    at once. A branch gets a float32 buffer for y, as in the sandwich wiring. The fold of y into the streams is not
    launched here: it is left in ``ctx.pending_fold`` and the kernel that reads the streams next (the next branch's read
    and norm, in this or the next layer, or the sum in front of the final norm: ``collapse_streams``) performs it on
    its way, so that a branch costs one launch beside its own."""
    launches_through_kernels_only = False      # (clearing the buffer for a part that adds is a torch operation)

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        if spec.streams < 1:
            raise ValueError("a hyper_connections layer needs at least one residual stream")
        self.hidden_size, self.streams = hidden_size, spec.streams
        self.mixer_norm = build_part("norm", spec.mixer_norm, hidden_size=hidden_size)
        self.mixer = build_part("mixer", spec.mixer, hidden_size=hidden_size)
        learned, scale = getattr(spec, "learned_streams", True), getattr(spec, "branch_scale", 1.0)
        self.mixer_streams = StreamMixing(spec.streams, learned, scale)
        taps = getattr(spec, "mixer_input_conv", 0)
        self.mixer_conv = InputConvolution(hidden_size, taps) if taps else None
        self.ffn = self.ffn_norm = self.ffn_streams = None
        if spec.ffn is not None:
            self.ffn_norm = build_part("norm", spec.ffn_norm, hidden_size=hidden_size)
            self.ffn = build_part("ffn", spec.ffn, hidden_size=hidden_size)
            self.ffn_streams = StreamMixing(spec.streams, learned, scale)

    def sub_parts(self):
        parts = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "mixer_streams": self.mixer_streams}
        if self.mixer_conv is not None:
            parts["mixer_conv"] = self.mixer_conv
        if self.ffn is not None:
            parts.update({"ffn_norm": self.ffn_norm, "ffn": self.ffn, "ffn_streams": self.ffn_streams})
        return parts

    def cache_spec(self):
        """What this layer's cache layer keeps: the mixer's cache and, with a convolution on the mixer's input, its last
        inputs."""
        if self.mixer_conv is None:
            return self.mixer.cache_spec()
        return combine_cache_specs([("mixer", self.mixer.cache_spec()), ("input_conv", self.mixer_conv.cache_spec())])

    def _branch(self, ctx, part, norm, mixing, xs, run, conv=None) -> None:
        n, d = xs.shape[0], self.hidden_size
        h = ctx.scratch("h", (n, d))
        fold, ctx.pending_fold = getattr(ctx, "pending_fold", None), None
        read, mix, write = mixing.on_device(xs.device)
        as_ln = getattr(norm, "as_layernorm", None)
        if as_ln is not None:
            kernels.streams_step(xs, self.streams, fold=fold, read=read, norm=as_ln(), h=h, positions=ctx.positions)
        else:
            u = ctx.scratch("stream_mix", (n, d), torch.float32)
            kernels.streams_step(xs, self.streams, fold=fold, read=read, u_out=u, positions=ctx.positions)
            norm.forward(ctx, u, h)
        if conv is not None:
            h = conv(h)
        y = ctx.scratch("branch", (n, d), torch.float32)
        ctx.overwrite_output = bool(part.can_overwrite_output)
        if not ctx.overwrite_output:
            y.zero_()
        # a part whose output is a weighted sum of rows may hand over the parts instead (``kernels.WeightedRows`` in
        # ``ctx.weighted_rows``): the kernel that folds the output into the streams forms the sum on its way
        ctx.accepts_weighted_rows, ctx.weighted_rows = True, None
        try:
            run(h, y)
        finally:
            ctx.overwrite_output = ctx.accepts_weighted_rows = False
        out, ctx.weighted_rows = (ctx.weighted_rows if ctx.weighted_rows is not None else y), None
        ctx.pending_fold = (out, mix, write)

    def forward(self, ctx, xs, cache, writes_cache: bool, after_mixer=None) -> None:
        ctx.next_norm = ctx.prepared_norm = None      # no product of this layer completes residual rows
        conv = None
        if self.mixer_conv is not None:
            conv_state = cache.states["input_conv"]
            cache = sub_view(cache, "mixer", self.mixer.cache_spec())

            def conv(h):
                out = ctx.scratch("h_conv", tuple(h.shape))
                self.mixer_conv.forward(ctx, h, out, conv_state, writes_cache)
                return out
        self._branch(ctx, self.mixer, self.mixer_norm, self.mixer_streams, xs,
                     lambda h, out: self.mixer.forward(ctx, h, out, cache, writes_cache), conv=conv)
        if after_mixer is not None:
            after_mixer()
        if self.ffn is not None:
            self._branch(ctx, self.ffn, self.ffn_norm, self.ffn_streams, xs, lambda h, out: self.ffn.forward(ctx, h, out))


def collapse_streams(ctx, xs, streams: int, norm, out, rows=None, total=None) -> None:
    """The end of a residual of several streams: out = norm(sum_s x_s) for the rows ``rows`` (all, if None), after whatever
    fold is still pending. ``total`` (float32, optional) also receives the sum itself."""
    fold, ctx.pending_fold = getattr(ctx, "pending_fold", None), None
    as_ln = getattr(norm, "as_layernorm", None) if norm is not None else None
    if as_ln is not None:
        kernels.streams_step(xs, streams, fold=fold, norm=as_ln(), h=out, u_out=total, rows=rows)
        return
    n_out = rows.shape[0] if rows is not None else xs.shape[0]
    u = total if total is not None else ctx.scratch("stream_sum", (n_out, xs.shape[1] // streams), torch.float32)
    kernels.streams_step(xs, streams, fold=fold, u_out=u, rows=rows)
    if norm is not None:
        norm.forward(ctx, u, out)


register_part("arrangement", "hyper_connections",
              lambda kind, *, layer_spec, hidden_size: HyperConnectionBlock(layer_spec, hidden_size=hidden_size), replace=True)
register_part("arrangement", "branch_norm",
              lambda kind, *, layer_spec, hidden_size: BranchNormBlock(layer_spec, hidden_size=hidden_size), replace=True)
register_part("arrangement", "sandwich_norm",
              lambda kind, *, layer_spec, hidden_size: SandwichNormBlock(layer_spec, hidden_size=hidden_size), replace=True)
register_part("arrangement", "pre_norm", lambda kind, *, layer_spec, hidden_size: PreNormBlock(layer_spec, hidden_size=hidden_size),
              replace=True)


def build_block(layer_spec, *, hidden_size: int):
    """Build the layer that ``layer_spec.arrangement`` names."""
    return build_part("arrangement", layer_spec.arrangement, layer_spec=layer_spec, hidden_size=hidden_size)
