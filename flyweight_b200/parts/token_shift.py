"""Token shift: the mixer reads ``x_n + (x_{n-1} - x_n) * mu`` instead of ``x_n``, with a weight
``mu`` per channel and zeros in front of a sequence's first token.  ``x_{n-1}`` is the stream as it
entered this layer for the token before, so every live request keeps that one row (fp32) per layer
in a state slot; the kernel reads it at the head of a portion and stores the portion's last row."""
from __future__ import annotations

from ..kernels import latent as latent_kernels
from ..weights.loader import TensorDecl
from .base import FixedState, Precision, StreamShift, register_shift


@register_shift("token_shift")
class TokenShift(StreamShift):
    """params: size.  tensors: weight [size]."""
    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(self.params["size"])
        self.weight = None

    def declare(self):
        return {self.names["weight"]: TensorDecl((self.size,), "bias")}

    def bind(self, get, precision: Precision, device):
        self.weight = precision.vector(get(self.names["weight"]), device)

    def weight_bytes(self):
        return self.size * 4

    def state_spec(self):
        return FixedState((self.size,))

    def plan(self, builder, out, cache):
        """The same operation for the native step plan: the shifted stream into ``out``."""
        builder.token_shift(self.weight, cache.state, out)

    def forward(self, ctx, x, cache):
        return latent_kernels.token_shift(x, self.weight, cache.state, ctx.batch, ctx.precision.act_dtype)
