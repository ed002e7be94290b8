"""Python faces of the gated-delta-rule kernels (``csrc/delta_rule.cu``): the recurrence over a
step's ragged segments with the per-request state in a slot, and the gated per-head norm behind it."""
from __future__ import annotations

import torch

from . import lib
from .lib import KernelError, c_float, c_longlong, check_tensor, is_bf16, ptr, stream
from .ops import _i32


def delta_state_size(heads: int, kv_heads: int, dim: int, vdim: int, taps: int) -> int:
    """fp32 entries of one request's slot: the [heads][vdim][dim] state, then the convolution's last
    ``taps - 1`` inputs of every channel of q, k and v (rounded up to a multiple of 4)."""
    size = heads * dim * vdim + (2 * kv_heads * dim + heads * vdim) * (taps - 1)
    return -(-size // 4) * 4            # slots start on 16-byte borders


def delta_rule(p: torch.Tensor, taps: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
               state: torch.Tensor, batch, heads: int, kv_heads: int, dim: int, vdim: int) -> torch.Tensor:
    """The gated delta rule over the step's tokens.  ``p``: fp32 [T][q | k | v | gate | b | a], the fused
    projection; ``taps``: fp32 [2 kv_heads dim + heads vdim][L]; ``state``: fp32 [slots][delta_state_size],
    read at the head of every segment and advanced.  Returns o, fp32 [T][heads][vdim]."""
    check_tensor("delta projection", p, torch.float32)
    T = p.shape[0]
    channels = 2 * kv_heads * dim + heads * vdim
    if p.shape[1] != channels + heads * vdim + 2 * heads:
        raise KernelError(f"the delta projection has {p.shape[1]} columns, expected "
                          f"{channels + heads * vdim + 2 * heads}")
    if taps.dim() != 2:
        raise KernelError("conv taps must be [channels][taps]")
    L = taps.shape[1]
    check_tensor("conv taps", taps, torch.float32, (channels, L))
    check_tensor("A_log", a_log, torch.float32, (heads,))
    check_tensor("dt_bias", dt_bias, torch.float32, (heads,))
    size = delta_state_size(heads, kv_heads, dim, vdim, L)
    if (not state.is_cuda or state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] != size
            or state.stride(1) != 1):
        raise KernelError(f"the delta state must be CUDA fp32 [slots][{size}], got {tuple(state.shape)}")
    stride = state.stride(0) if state.shape[0] > 1 else size
    S = batch.n_segments
    _i32("seg_start", batch.seg_start, S + 1)
    _i32("seg_slot", batch.seg_slot, S)
    _i32("tok_seg", batch.tok_seg, T)
    r = torch.empty((T, -(-(channels + 2 * heads + kv_heads) // 4) * 4), dtype=torch.float32, device=p.device)
    o = torch.empty((T, heads, vdim), dtype=torch.float32, device=p.device)
    lib.call("fwb_delta_rule", ptr(p), ptr(taps), ptr(a_log), ptr(dt_bias), ptr(state), c_longlong(stride),
             ptr(batch.seg_start), ptr(batch.seg_slot), ptr(batch.tok_seg), ptr(r), ptr(o), T, S, heads, kv_heads,
             dim, vdim, L, stream(), launches=2)
    return o


def gated_head_norm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float,
                    out_dtype: torch.dtype) -> torch.Tensor:
    """``weight * o / sqrt(mean(o^2) + eps) * silu(gate)`` per (token, head).  o: fp32 [T][H][e];
    ``gate``: fp32 [T][H e], possibly a view of columns of a wider row-major tensor; weight: fp32 [e]."""
    check_tensor("recurrence output", o, torch.float32)
    T, H, e = o.shape
    if (not gate.is_cuda or gate.dtype != torch.float32 or tuple(gate.shape) != (T, H * e)
            or gate.stride(1) != 1):
        raise KernelError(f"the gate must be CUDA fp32 [{T}][{H * e}] with contiguous rows")
    check_tensor("head norm weight", weight, torch.float32, (e,))
    out = torch.empty((T, H * e), dtype=out_dtype, device=o.device)
    lib.call("fwb_gated_head_norm", ptr(o), ptr(gate), c_longlong(gate.stride(0)), ptr(weight), c_float(eps),
             ptr(out), is_bf16(out), T, H, e, stream())
    return out
