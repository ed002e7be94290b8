"""The sandwich residual arrangement: a weighted RMS norm in front of every sublayer and another on
its output, ahead of the residual sum,

    x += norm_b(mixer(norm_a(x)));   x += norm_d(feed_forward(norm_c(x)))

The feed-forward and its two norms may be absent.  A sublayer's output norm, the residual sum and
the norm in front of the next sublayer of the same layer are one kernel (``ops.rmsnorm_add_``); the
stream stays fp32.
"""
from __future__ import annotations

from ..kernels import ops
from .base import Arrangement, register_arrangement


@register_arrangement("sandwich_residual")
class SandwichResidual(Arrangement):
    ROLES = {"mixer_norm": ("norm", True), "mixer": ("mixer", True), "mixer_out_norm": ("norm", True),
             "ffn_norm": ("norm", False), "feed_forward": ("feed_forward", False),
             "ffn_out_norm": ("norm", False)}

    def __init__(self, layer):
        super().__init__(layer)
        present = [part is not None for part in (self.ffn_norm, self.feed_forward, self.ffn_out_norm)]
        if any(present) and not all(present):
            raise ValueError("arrangement 'sandwich_residual': a feed-forward comes with the norm in front of "
                             "it and the norm behind it")
        for norm in (self.mixer_out_norm, self.ffn_norm, self.ffn_out_norm):
            if norm is not None and getattr(norm, "plan_params", None) is None:
                raise ValueError(f"arrangement 'sandwich_residual': norm {norm.kind!r} is no weighted RMS norm")

    def forward(self, ctx, x, pending, cache):
        act = ctx.precision.act_dtype
        h = self.mixer_norm.forward(ctx, x, delta=pending)
        y = self.mixer.forward(ctx, h, cache)
        w, eps = self.mixer_out_norm.plan_params()
        if self.feed_forward is None:
            ops.rmsnorm_add_(x, y, w, eps)
            return x, None
        w_next, eps_next = self.ffn_norm.plan_params()
        h = ops.rmsnorm_add_(x, y, w, eps, w_next, eps_next, act)
        w, eps = self.ffn_out_norm.plan_params()
        fused = getattr(self.feed_forward, "forward_add_normed", None)
        if fused is not None:
            fused(ctx, h, x, w, eps)           # the part's last kernel norms its output and adds it
        else:
            ops.rmsnorm_add_(x, self.feed_forward.forward(ctx, h), w, eps)
        return x, None
