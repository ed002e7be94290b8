"""Gated delta rule mixer: a recurrence whose state is one [dim][vdim] matrix per head and request.

Per token, with h the mixer's input:  q, k (kv_heads x dim) and v (heads x vdim) are projections of h
that pass a short causal convolution over time per channel and silu; q and k become unit vectors per
head (q also times dim^-1/2); beta = sigmoid(W_b h) and the decay g = exp(-exp(A_log) softplus(W_a h +
dt_bias)) are one number per head.  Then, per head (query head j reads q/k head j // (heads/kv_heads)),

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

and the output is W_o of  norm_weight * o / rms(o) * silu(W_g h)  with the root mean square over vdim.
S and the convolution's last inputs live in the request's state slot (fp32, zero at admission), so a
sequence may be cut into steps anywhere.  One fused projection q|k|v|gate|b|a leaves its product in
fp32: everything behind it that enters the recurrence is computed in 32-bit in both precisions.
"""
from __future__ import annotations

import torch

from ..kernels import ops, recurrent
from ..weights.loader import TensorDecl
from .base import FixedState, Mixer, Precision, register_mixer


@register_mixer("gated_delta_rule")
class GatedDeltaRule(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, dim, vdim, taps, eps (of the output's norm).
    tensors: q, k, v [rows][H]; q_conv, k_conv, v_conv [channels][taps]; b, a [heads][H]; a_log,
    dt_bias [heads]; gate [heads vdim][H]; norm [vdim]; o [H][heads vdim]."""
    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["num_heads"])
        self.n_kv = int(p["num_kv_heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p["vdim"])
        self.taps_len = int(p["taps"])
        self.eps = float(p["eps"])
        if self.n_heads % self.n_kv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.taps_len < 1:
            raise ValueError("the short convolution needs at least one tap")
        self.w_in = self.w_o = self.taps = self.a_log = self.dt_bias = self.norm = None

    @property
    def _qk(self) -> int:
        return self.n_kv * self.dim

    @property
    def _v(self) -> int:
        return self.n_heads * self.vdim

    def declare(self):
        n, H, L = self.names, self.hidden, self.taps_len
        return {n["q"]: TensorDecl((self._qk, H)), n["k"]: TensorDecl((self._qk, H)),
                n["v"]: TensorDecl((self._v, H)), n["gate"]: TensorDecl((self._v, H)),
                n["b"]: TensorDecl((self.n_heads, H)), n["a"]: TensorDecl((self.n_heads, H)),
                n["q_conv"]: TensorDecl((self._qk, L), "taps"), n["k_conv"]: TensorDecl((self._qk, L), "taps"),
                n["v_conv"]: TensorDecl((self._v, L), "taps"),
                n["a_log"]: TensorDecl((self.n_heads,), "bias"), n["dt_bias"]: TensorDecl((self.n_heads,), "bias"),
                n["norm"]: TensorDecl((self.vdim,), "norm"), n["o"]: TensorDecl((H, self._v))}

    def bind(self, get, precision: Precision, device):
        n = self.names
        mats = [get(n[name]) for name in ("q", "k", "v", "gate", "b", "a")]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.to(torch.float32) for m in mats]
        # one projection: the rows of the six matrices, one after the other
        self.w_in = precision.matrix(torch.cat(mats, dim=0), device)
        self.w_o = precision.matrix(get(n["o"]), device)
        self.taps = precision.vector(torch.cat([get(n["q_conv"]), get(n["k_conv"]), get(n["v_conv"])], dim=0), device)
        self.a_log = precision.vector(get(n["a_log"]), device)
        self.dt_bias = precision.vector(get(n["dt_bias"]), device)
        self.norm = precision.vector(get(n["norm"]), device)

    def weight_bytes(self):
        return (self.w_in.numel() * self.w_in.element_size() + self.w_o.numel() * self.w_o.element_size()
                + self.taps.numel() * 4)

    def flops_per_token(self):
        # the products, and per head three passes over the [dim][vdim] state (decay and read, write, read-out)
        return 2.0 * (self.w_in.numel() + self.w_o.numel()) + 6.0 * self.n_heads * self.dim * self.vdim

    def state_spec(self):
        return FixedState((recurrent.delta_state_size(self.n_heads, self.n_kv, self.dim, self.vdim, self.taps_len),))

    def forward(self, ctx, h, cache):
        p = ops.linear(h, self.w_in, torch.float32)
        o = recurrent.delta_rule(p, self.taps, self.a_log, self.dt_bias, cache.state, ctx.batch, self.n_heads,
                                 self.n_kv, self.dim, self.vdim)
        gate_at = 2 * self._qk + self._v
        z = recurrent.gated_head_norm(o, p[:, gate_at:gate_at + self._v], self.norm, self.eps,
                                      ctx.precision.act_dtype)
        return ops.linear(z, self.w_o, torch.float32)
