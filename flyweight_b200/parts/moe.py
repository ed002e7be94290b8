"""Mixture-of-experts feed-forward with a grouped, bias-corrected softmax router and identity experts.

Router scores s = softmax(W_router h) over all router outputs, in fp32.  The choice is made on s +
correction: the outputs form ``groups`` equal runs of neighbours, only the ``keep_groups`` runs with
the largest choice value stay in the race, and the ``top`` largest survivors are chosen; the weights
are the plain s of the chosen, not renormalised.  The first ``experts`` outputs are small gated
feed-forwards, down(act(gate h) * (up h)); the ``identity`` outputs behind them hand h itself on.  The
result is the weighted sum over the chosen.
"""
from __future__ import annotations

import torch

from ..kernels import experts as expert_kernels
from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import FeedForward, Precision, register_feed_forward


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    """params: hidden_size, ffn_dim (of one expert), experts, identity (0), top, groups (1), keep_groups
    (1), activation ("silu").  tensors: router [experts + identity][H], correction [experts + identity],
    and per expert j ``gate{j}``, ``up{j}`` [F][H], ``down{j}`` [H][F]."""
    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.ffn_dim = int(p["ffn_dim"])
        self.n_experts = int(p["experts"])
        self.n_identity = int(p.get("identity", 0) or 0)
        self.top = int(p["top"])
        self.groups = int(p.get("groups", 1) or 1)
        self.keep_groups = int(p.get("keep_groups", self.groups) or self.groups)
        self.activation = str(p.get("activation", "silu"))
        outputs = self.n_experts + self.n_identity
        if self.activation not in ops.GATE_ACTIVATIONS:
            raise ValueError(f"unknown gate activation {self.activation!r}")
        if self.n_experts < 0 or self.n_identity < 0 or outputs <= 0:
            raise ValueError("a router needs at least one output")
        if outputs % self.groups or not 0 < self.keep_groups <= self.groups:
            raise ValueError(f"{outputs} router outputs do not form {self.groups} equal groups of which "
                             f"{self.keep_groups} are kept")
        if not 0 < self.top <= self.keep_groups * (outputs // self.groups):
            raise ValueError(f"top {self.top} does not fit the {self.keep_groups} kept groups")
        self.router = self.correction = self.w_gate_up = self.w_down = None

    @property
    def n_outputs(self) -> int:
        return self.n_experts + self.n_identity

    def declare(self):
        n, H, F = self.names, self.hidden, self.ffn_dim
        out = {n["router"]: TensorDecl((self.n_outputs, H)), n["correction"]: TensorDecl((self.n_outputs,), "bias")}
        for j in range(self.n_experts):
            out[n[f"gate{j}"]] = TensorDecl((F, H))
            out[n[f"up{j}"]] = TensorDecl((F, H))
            out[n[f"down{j}"]] = TensorDecl((H, F))
        return out

    def bind(self, get, precision: Precision, device):
        n = self.names
        # the router runs in fp32 whatever the precision (a bfloat16 matrix widens exactly)
        self.router = precision.vector(get(n["router"]), device)
        self.correction = precision.vector(get(n["correction"]), device)
        mats = [get(n[f"{role}{j}"]) for j in range(self.n_experts) for role in ("gate", "up", "down")]
        dtype = torch.float32 if (precision.name == "float32" or len({m.dtype for m in mats}) > 1) \
            else (mats[0].dtype if mats else precision.act_dtype)
        H, F, E = self.hidden, self.ffn_dim, self.n_experts
        if E:
            # [E][gate rows | up rows][H] and [E][H][F]: one stacked tensor per product
            gate_up = torch.stack([torch.cat([get(n[f"gate{j}"]).to(dtype), get(n[f"up{j}"]).to(dtype)], dim=0)
                                   for j in range(E)])
            down = torch.stack([get(n[f"down{j}"]).to(dtype) for j in range(E)])
        else:
            gate_up, down = torch.empty((0, 2 * F, H), dtype=dtype), torch.empty((0, H, F), dtype=dtype)
        self.w_gate_up = gate_up.to(device).contiguous()
        self.w_down = down.to(device).contiguous()

    def weight_bytes(self):
        # what a step reads at most: the router, and the experts its tokens choose (all of them, from
        # enough tokens on)
        return (self.router.numel() * 4 + self.w_gate_up.numel() * self.w_gate_up.element_size()
                + self.w_down.numel() * self.w_down.element_size())

    def active_weight_bytes(self, n_tokens):
        chosen = min(self.n_experts, n_tokens * self.top)
        per_expert = 3 * self.ffn_dim * self.hidden * self.w_gate_up.element_size()
        return self.router.numel() * 4 + chosen * per_expert

    def flops_per_token(self):
        return 2.0 * self.router.numel() + 2.0 * self.top * 3 * self.ffn_dim * self.hidden

    def forward(self, ctx, h, add_normed_into=None):
        ids, weights = expert_kernels.route(h, self.router, self.correction, self.groups, self.keep_groups, self.top)
        if h.dtype != self.w_gate_up.dtype:
            h = ops.cast(h, self.w_gate_up.dtype)
        return expert_kernels.experts_forward(h, ids, weights, self.w_gate_up, self.w_down, self.activation,
                                              add_normed_into)

    def forward_add_normed(self, ctx, h, x, norm_weight, eps):
        """``x += norm_weight * unit(ff(h))`` with the weighted sum, the output norm and the residual sum in
        one kernel (an arrangement with a norm on the sublayer's output asks for it)."""
        self.forward(ctx, h, add_normed_into=(x, norm_weight, eps))
