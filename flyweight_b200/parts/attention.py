"""Grouped-query attention mixer with per-head q/k RMSNorm and rotary positions.

Order of operations (native/src/v2_runtime.cpp:28429-28478): q, k, v projections
without bias; RMSNorm over each head of q and of k with a [head_dim] weight shared by
all heads; rotary encoding of q and k; k and v appended to the cache; scores of query
head j against KV head j // (heads / kv_heads), scaled by head_dim^-1/2, causal,
softmax in fp32; output projection without gate.
"""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Mixer, PagedKV, Precision, build_position, register_mixer


@register_mixer("gqa_attention")
class GQAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, qk_norm_eps (None: no
    q/k norm), position (PartSpec of a position encoding), window (0: all keys),
    shares_cache (True: reads the cache of another execution and projects q only).
    tensors: q, k, v, o, q_norm, k_norm.

    Further params, all optional: ``scale`` (head_dim^-1/2 when absent); ``chunk`` (> 0: the sequence
    is cut into runs of that many positions counted from position 0, and a query sees only the keys of
    its own run up to itself); ``qk_unit_rms_eps`` (not None: instead of the weighted norm in front of
    the rotation, every head of q and k is brought to unit root mean square behind it, without a
    weight; no ``q_norm``/``k_norm`` tensors); ``value_dim`` (the size of a value head when it differs
    from ``head_dim``: the pools and kernels then run at the larger of the two, the smaller heads padded
    with zero channels through zero rows and columns of the matrices)."""
    graph_safe = True
    takes_deferred_norm = True
    adds_residual = True

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["num_heads"])
        self.n_kv = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.eps = p.get("qk_norm_eps")
        self.window = int(p.get("window", 0) or 0)
        self.shares_cache = bool(p.get("shares_cache", False))
        self.scale = float(p.get("scale", 1.0 / math.sqrt(self.head_dim)))
        self.position = build_position(p["position"])
        self.chunk = int(p.get("chunk", 0) or 0)
        self.unit_rms_eps = p.get("qk_unit_rms_eps")
        # what the checkpoint's matrices have per head, and what the pools and kernels run at
        self.qk_dim = self.head_dim
        self.value_dim = int(p.get("value_dim", self.head_dim) or self.head_dim)
        if self.n_heads % self.n_kv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.chunk and self.window:
            raise ValueError("an attention mixer has a sliding window or chunks, not both")
        if self.unit_rms_eps is not None and self.eps is not None:
            raise ValueError("an attention mixer norms q and k in front of the rotation or behind it, not both")
        if self.value_dim != self.qk_dim or self.unit_rms_eps is not None or self.chunk:
            self.head_dim = -(-max(self.qk_dim, self.value_dim) // 16) * 16
        if self.head_dim % 16:
            raise ValueError(f"head size {self.head_dim}: the attention kernels take head sizes "
                             "in steps of 16")
        if self.head_dim != self.qk_dim and self.eps is not None:
            raise ValueError("padded heads go with the unweighted q/k norm only")
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    @property
    def _kv_in(self) -> int:
        return 0 if self.shares_cache else self.n_kv

    def declare(self):
        n, hd, H = self.names, self.qk_dim, self.hidden
        out = {n["q"]: TensorDecl((self.n_heads * hd, H)),
               n["o"]: TensorDecl((H, self.n_heads * self.value_dim))}
        if not self.shares_cache:
            out[n["k"]] = TensorDecl((self.n_kv * hd, H))
            out[n["v"]] = TensorDecl((self.n_kv * self.value_dim, H))
        if self.eps is not None:
            out[n["q_norm"]] = TensorDecl((hd,), "norm")
            if not self.shares_cache:
                out[n["k_norm"]] = TensorDecl((hd,), "norm")
        return out

    def bind(self, get, precision: Precision, device):
        n = self.names
        D = self.head_dim

        def rows_padded(matrix, per_head):
            """[heads * per_head][H] -> [heads * D][H]: zero rows behind every head's own."""
            if per_head == D:
                return matrix
            heads = matrix.shape[0] // per_head
            wide = matrix.new_zeros((heads, D, matrix.shape[1]))
            wide[:, :per_head] = matrix.view(heads, per_head, -1)
            return wide.view(heads * D, -1)

        mats = [rows_padded(get(n["q"]), self.qk_dim)]
        if not self.shares_cache:
            mats += [rows_padded(get(n["k"]), self.qk_dim), rows_padded(get(n["v"]), self.value_dim)]
        dtypes = {m.dtype for m in mats}
        if len(dtypes) > 1:
            mats = [m.to(torch.float32) for m in mats]
        # one projection for q|k|v: the rows of the three matrices, one after the other
        self.w_qkv = precision.matrix(torch.cat(mats, dim=0), device)
        w_o = get(n["o"])
        if self.value_dim != D:                   # zero columns where the padded channels of a head arrive
            wide = w_o.new_zeros((w_o.shape[0], self.n_heads, D))
            wide[:, :, :self.value_dim] = w_o.view(w_o.shape[0], self.n_heads, self.value_dim)
            w_o = wide.view(w_o.shape[0], self.n_heads * D)
        self.w_o = precision.matrix(w_o, device)
        if self.eps is not None:
            self.q_norm = precision.vector(get(n["q_norm"]), device)
            if not self.shares_cache:
                self.k_norm = precision.vector(get(n["k_norm"]), device)

    def weight_bytes(self):
        return (self.w_qkv.numel() * self.w_qkv.element_size()
                + self.w_o.numel() * self.w_o.element_size())

    def flops_per_token(self):
        return 2.0 * (self.w_qkv.numel() + self.w_o.numel())

    def context_flops(self, n_tokens):
        # QK^T and PV: 4 operations per (query, visible key, channel); half the pairs are masked
        if self.chunk and n_tokens > self.chunk:
            whole, rest = divmod(n_tokens, self.chunk)
            return 2.0 * (whole * self.chunk * self.chunk + rest * rest) * self.n_heads * self.head_dim
        return 2.0 * n_tokens * n_tokens * self.n_heads * self.head_dim

    @property
    def span(self) -> int:
        """The mask parameter of the attention kernels: a window (> 0), chunks (< 0), or all keys."""
        return -self.chunk if self.chunk else self.window

    def _encode_extra(self) -> dict:
        if self.unit_rms_eps is None:
            return {}
        return {"unit_rms_after": True, "norm_dim": self.qk_dim}

    def state_spec(self):
        return None if self.shares_cache else PagedKV(self.n_kv, self.head_dim, self.window)

    def prepare(self, max_positions, device):
        self.position.prepare(max_positions, device)

    def forward(self, ctx, h, cache, residual=None):
        act = ctx.precision.act_dtype
        # q|k|v in the activation dtype; the head norm and the rotation widen it to fp32
        qkv = ops.linear(h, self.w_qkv, act)
        block_table = ctx.batch.block_tables[cache.group]
        from ..kernels import attention as attention_kernels
        rotation = self.position.rotation() if self.unit_rms_eps is None else None
        if rotation is not None and attention_kernels.decode_fusable(ctx, qkv, cache, block_table, self.n_heads, rotation[1], self.window):
            # a step of single tokens whose position part is a plain rotation: the decode attention
            # kernel norms, turns and stores its own token's heads (one kernel and one pass less)
            table, rotary_dim, pairing = rotation
            out = attention_kernels.fused_decode_attention(
                ctx, qkv, cache, block_table, self.n_heads, self._kv_in, self.window, self.scale,
                self.q_norm, self.k_norm, self.eps, table, rotary_dim, pairing)
            return ops.linear_into_residual(out, self.w_o, residual)
        # positions are the position part's business: it norms, encodes and writes the pages
        q = self.position.encode(ctx, qkv, n_heads=self.n_heads, n_kv_in=self._kv_in,
                                 head_dim=self.head_dim, q_norm=self.q_norm, k_norm=self.k_norm,
                                 eps=self.eps if self.unit_rms_eps is None else self.unit_rms_eps,
                                 cache=cache, block_table=block_table, **self._encode_extra())
        out = attention_kernels.paged_attention(ctx, q, cache, block_table, self.n_heads,
                                                self.span, self.scale, act)
        return ops.linear_into_residual(out, self.w_o, residual)

    def plan(self, builder, norm, cache):
        """The same operations for the native step plan (``engine/plan.py``)."""
        from ..engine.plan import EPI_ACT, NotPlannable
        act = builder.act_dtype
        plan_position = getattr(self.position, "plan", None)
        if self.unit_rms_eps is not None:
            raise NotPlannable("the q/k norm behind the rotation has no native plan form")
        if plan_position is None:
            raise NotPlannable(f"position encoding {self.position.kind!r} has no native form")
        width = self.n_heads * self.head_dim
        qkv = builder.tokens(width + 2 * self._kv_in * self.head_dim, act)
        builder.norm_linear(norm, self.w_qkv, EPI_ACT, qkv, "q|k|v")
        q = builder.tokens(width, act)
        plan_position(builder, qkv, q, n_heads=self.n_heads, n_kv_in=self._kv_in, head_dim=self.head_dim,
                      q_norm=self.q_norm, k_norm=self.k_norm, eps=self.eps, cache=cache)
        builder.free(qkv)
        out = builder.tokens(width, act)
        builder.attention(q, cache, out, self.n_heads, self.span, self.scale)
        builder.free(q)
        builder.linear_residual(out, self.w_o, "attention out_proj")
        builder.free(out)
