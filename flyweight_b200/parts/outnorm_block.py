"""The output-norm residual arrangement: a norm sits on each sublayer's *output*, and the sublayers
read the residual stream itself,

    x += norm_a(mixer(shift(x)));   x += norm_b(feed_forward(x))

``shift`` (optional) is a mix along the sequence in front of the mixer; the feed-forward and its norm
may be absent.  The norms are of a kind that can add into the stream (``add_normed``), so a sublayer's
norm, its residual sum and the rounding of the new stream for the next matrix product are one kernel.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Arrangement, register_arrangement


@register_arrangement("outnorm_residual")
class OutputNormResidual(Arrangement):
    ROLES = {"shift": ("shift", False), "mixer": ("mixer", True), "mixer_out_norm": ("norm", True),
             "feed_forward": ("feed_forward", False), "ffn_out_norm": ("norm", False)}

    def __init__(self, layer):
        super().__init__(layer)
        if (self.feed_forward is None) != (self.ffn_out_norm is None):
            raise ValueError("arrangement 'outnorm_residual': a feed-forward and its output norm come together")
        for norm in (self.mixer_out_norm, self.ffn_out_norm):
            if norm is not None and not hasattr(norm, "add_normed"):
                raise ValueError(f"arrangement 'outnorm_residual': norm {norm.kind!r} cannot add into the stream")

    def stateful_parts(self):
        return tuple(part for part in (self.mixer, self.shift) if part is not None)

    def plan(self, builder, cache):
        """This layer's operations for the native step plan (the symbolic twin of ``forward``)."""
        from ..engine.plan import NotPlannable
        if self.shift is None or getattr(self.shift, "plan", None) is None:
            raise NotPlannable("the output-norm arrangement has a native form with a stream shift only")
        for part in (self.mixer, self.feed_forward):
            if part is not None and getattr(part, "plan_stream", None) is None:
                raise NotPlannable(f"part {part.kind!r} has no native form behind an unnormed stream")
        for norm in (self.mixer_out_norm, self.ffn_out_norm):
            if norm is not None and getattr(norm, "gain", None) is None:
                raise NotPlannable(f"norm {norm.kind!r} has no native form behind a sublayer")
        act = builder.act_dtype
        h = builder.tokens(builder.hidden, act)
        self.shift.plan(builder, h, cache)
        y = builder.delta                      # a sublayer's output, fp32; the norm behind it adds it into x
        self.mixer.plan_stream(builder, h, cache, y)
        builder.free(h)
        if self.feed_forward is None:
            builder.gain_add(y, self.mixer_out_norm.gain, self.mixer_out_norm.eps, None)
            return
        copy = builder.tokens(builder.hidden, act) if act != torch.float32 else None
        builder.gain_add(y, self.mixer_out_norm.gain, self.mixer_out_norm.eps, copy)
        self.feed_forward.plan_stream(builder, builder.x if copy is None else copy, y)
        builder.free(copy)
        builder.gain_add(y, self.ffn_out_norm.gain, self.ffn_out_norm.eps, None)

    def forward(self, ctx, x, pending, cache):
        if pending is not None:
            ops.add_(x, pending)
        act = ctx.precision.act_dtype
        h = self.shift.forward(ctx, x, cache) if self.shift is not None else ops.cast(x, act)
        y = self.mixer.forward(ctx, h, cache)
        if self.feed_forward is None:
            self.mixer_out_norm.add_normed(ctx, x, y)
            return x, None
        # the feed-forward reads the stream itself: in 16-bit mode the sum's kernel also rounds it
        h = self.mixer_out_norm.add_normed(ctx, x, y, copy_dtype=None if act == torch.float32 else act)
        self.ffn_out_norm.add_normed(ctx, x, self.feed_forward.forward(ctx, x if h is None else h))
        return x, None
