"""Embedding parts: what enters the first layer for a step's tokens.

``hashed_pairs``: the scaled row of the token table plus one row of a second table that is
indexed by a hash of the token and the one before it, ``(before * mul_prev + token * mul_cur) mod
buckets``; the table's last row (number ``buckets``) serves a sequence's first token.  The token
before the head of a portion was part of an earlier step, so every live request keeps its last
token in a state slot on the device; the kernel reads it and moves it on (nothing passes through the
host, so steps that take their ids from the sampler's output on the device work unchanged).
"""
from __future__ import annotations

import torch

from ..kernels import latent as latent_kernels
from ..weights.loader import TensorDecl
from .base import Embedding, FixedState, Precision, register_embedding


@register_embedding("hashed_pairs")
class HashedPairEmbedding(Embedding):
    """params: hidden_size, scale, buckets, mul_prev, mul_cur.  tensors: pairs [buckets + 1][hidden]."""
    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.scale = float(p.get("scale", 1.0))
        self.buckets = int(p["buckets"])
        self.mul_prev = int(p["mul_prev"])
        self.mul_cur = int(p["mul_cur"])
        if self.buckets <= 0:
            raise ValueError("a hashed pair table needs at least one bucket")
        self.pairs = None

    def declare(self):
        return {self.names["pairs"]: TensorDecl((self.buckets + 1, self.hidden), "embedding")}

    def bind(self, get, precision: Precision, device):
        self.pairs = precision.matrix(get(self.names["pairs"]), device)

    def state_spec(self):
        return FixedState((1,), torch.int32)

    def plan(self, builder, table, vocab, cache):
        """The same operation for the native step plan."""
        from ..engine.plan import NotPlannable
        if cache is None or cache.state is None:
            raise NotPlannable("the hashed pair embedding has no state slot")
        builder.embed_pairs(table, self.pairs, vocab, self.buckets, self.mul_prev, self.mul_cur, self.scale,
                            cache.state)

    def forward(self, ctx, table, cache):
        pairs = self.pairs if self.pairs.dtype == table.dtype else self.pairs.to(table.dtype)
        return latent_kernels.embed_pair_hash(table, pairs, ctx.batch, cache.state, self.buckets,
                                              self.mul_prev, self.mul_cur, ctx.bad_token_flag, self.scale)
