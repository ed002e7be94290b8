"""Python faces of the kernels behind the latent-attention mixer, the token shift, the hashed
pair embedding and the gain-only output norm (``csrc/latent_attention.cu``,
``csrc/head_linear_mma.cu``, ``csrc/stream_mix.cu``).  The bfloat16 attention itself runs on the
engine's paged attention kernels (``kernels/attention.py``): the cached row is key and value at once."""
from __future__ import annotations

from typing import Optional

import torch

from . import lib
from .lib import KernelError, c_float, c_longlong, check_tensor, is_bf16, ptr, stream
from .ops import ROPE_PAIRINGS, _i32


def _slot_stride(name: str, state: torch.Tensor, row: int) -> int:
    """Distance between two slots of a per-request state whose rows hold ``row`` contiguous entries."""
    if not state.is_cuda or state.dim() != 2 or state.shape[1] != row or (row > 1 and state.stride(1) != 1):
        raise KernelError(f"{name} must be a CUDA tensor [slots][{row}] with contiguous rows, got "
                          f"{tuple(state.shape)}")
    return state.stride(0) if state.shape[0] > 1 else max(row, 1)


def embed_pair_hash(table: torch.Tensor, pairs: torch.Tensor, batch, last_token: torch.Tensor, buckets: int,
                    mul_prev: int, mul_cur: int, bad_flag: Optional[torch.Tensor], scale: float) -> torch.Tensor:
    """``scale * table[id] + pairs[(id_before * mul_prev + id * mul_cur) mod buckets]`` (row ``buckets``
    at position 0) for the step's tokens, fp32 [T][W].  ``last_token``: int32 [slots][1], the last id
    of every live request; read at the head of a portion and advanced by this launch."""
    check_tensor("embedding table", table)
    check_tensor("pair table", pairs, table.dtype, (buckets + 1, table.shape[1]))
    if last_token.dtype != torch.int32:
        raise KernelError("the last-token state must be int32")
    stride = _slot_stride("last-token state", last_token, 1)
    V, W = table.shape
    T = batch.token_ids.numel()
    out = torch.empty((T, W), dtype=torch.float32, device=table.device)
    lib.call("fwb_embed_pair_hash", ptr(table), ptr(pairs), is_bf16(table), ptr(batch.token_ids),
             ptr(batch.positions), ptr(batch.tok_seg), ptr(batch.seg_start), ptr(batch.seg_slot),
             ptr(last_token), c_longlong(stride), ptr(out), T, W, V, int(buckets), c_longlong(mul_prev),
             c_longlong(mul_cur), ptr(bad_flag), c_float(scale), stream())
    return out


def token_shift(x: torch.Tensor, mu: torch.Tensor, last_row: torch.Tensor, batch,
                out_dtype: torch.dtype) -> torch.Tensor:
    """``x[t] + (x[t-1] - x[t]) * mu`` along every request's tokens (zeros in front of position 0);
    ``last_row``: fp32 [slots][W], every live request's last row of x, read and advanced here."""
    check_tensor("residual", x, torch.float32)
    T, W = x.shape
    check_tensor("shift weights", mu, torch.float32, (W,))
    if last_row.dtype != torch.float32:
        raise KernelError("the shift state must be fp32")
    stride = _slot_stride("shift state", last_row, W)
    out = torch.empty((T, W), dtype=out_dtype, device=x.device)
    lib.call("fwb_token_shift", ptr(x), ptr(mu), ptr(last_row), c_longlong(stride), ptr(batch.positions),
             ptr(batch.tok_seg), ptr(batch.seg_start), ptr(batch.seg_slot), ptr(out), is_bf16(out), T, W,
             stream())
    return out


def unit_rms_gain_add_(x: torch.Tensor, y: torch.Tensor, gain: torch.Tensor, eps: float,
                       copy_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """``x += gain * y / sqrt(mean(y^2) + eps)`` row by row, in place and in fp32; returns the new x
    in ``copy_dtype`` as well when one is asked for (written by the same launch)."""
    check_tensor("residual", x, torch.float32)
    check_tensor("sublayer output", y, torch.float32, x.shape)
    check_tensor("gain", gain, torch.float32)
    T, W = x.shape
    copy = torch.empty((T, W), dtype=copy_dtype, device=x.device) if copy_dtype is not None else None
    lib.call("fwb_unit_rms_gain_add", ptr(x), ptr(y), ptr(gain), ptr(copy),
             is_bf16(copy) if copy is not None else 0, T, W, c_float(eps), stream())
    return copy


def latent_prepare(proj: torch.Tensor, kv_col: int, norm_w: Optional[torch.Tensor], table: torch.Tensor,
                   batch, block_table: Optional[torch.Tensor], pool: Optional[torch.Tensor], heads: int,
                   dim: int, rot: int, rot_dims: int, pairing: str, rank: int, row: int,
                   eps: float) -> torch.Tensor:
    """Turn the rotated part of every query head and (with ``pool``) write the token's cache row:
    the RMS-normed latent, the turned shared key part, zero padding.  Returns qa [T][heads][row] whose
    columns [rank, row) are set; the per-head product fills [0, rank)."""
    check_tensor("projection", proj)
    check_tensor("rope table", table, torch.float32)
    T, ld = proj.shape
    page_size = max_pages = 0
    if pool is not None:
        check_tensor("latent pool", pool)
        check_tensor("latent norm weight", norm_w, torch.float32, (rank,))
        _i32("block table", block_table)
        if pool.dim() != 4 or pool.shape[1] != 1 or pool.shape[3] != row:
            raise KernelError(f"the latent pool must be [pages][1][page_size][{row}], got {tuple(pool.shape)}")
        page_size, max_pages = pool.shape[2], block_table.shape[1]
    if table.dim() != 3 or table.shape[1] != max(1, rot_dims // 2) or table.shape[2] != 2:
        raise KernelError("rope table must be [positions][rot_dims/2][2]")
    qa = torch.empty((T, heads, row), dtype=proj.dtype, device=proj.device)
    lib.call("fwb_latent_prepare", ptr(proj), is_bf16(proj), ld, int(kv_col), ptr(norm_w), ptr(table),
             ptr(batch.positions), ptr(batch.tok_seg), ptr(block_table), max_pages, page_size, ptr(qa),
             ptr(pool), is_bf16(pool) if pool is not None else 0, T, heads, dim, rot, rot_dims,
             ROPE_PAIRINGS[pairing], rank, row, c_float(eps), stream())
    return qa


_mma_enabled = True


def set_tensor_cores(flag: bool) -> None:
    """Test switch: the bfloat16 tensor-core forms of the per-head products and of the attention
    (on by default) or the fp32-FMA kernels for everything."""
    global _mma_enabled
    _mma_enabled = bool(flag)
    lib.set_option("latent_tensorcore", _mma_enabled)


def tensor_cores() -> bool:
    from . import attention
    return _mma_enabled and attention.mma_enabled()


def head_linear(x: torch.Tensor, x_col: int, x_head: int, in_features: int, w: torch.Tensor,
                y: torch.Tensor, y_col: int, y_head: int) -> None:
    """``y[t][y_col + h*y_head + n] = sum_k w[h][n][k] * x[t][x_col + h*x_head + k]`` for every head h.
    x, y: 2-D row-major (any row length); w: [heads][N][K] contiguous, K = ``in_features``."""
    check_tensor("per-head input", x)
    check_tensor("per-head weight", w, x.dtype)
    check_tensor("per-head output", y, x.dtype)
    heads, N, K = w.shape
    if K != in_features or x.shape[0] != y.shape[0]:
        raise KernelError("per-head product: sizes do not fit")
    if x_col + (heads - 1) * x_head + K > x.shape[1] or y_col + (heads - 1) * y_head + N > y.shape[1]:
        raise KernelError("per-head product: a head lies outside its row")
    size = x.element_size()
    x_ptr, y_ptr = x.data_ptr() + x_col * size, y.data_ptr() + y_col * size
    if (_mma_enabled and x.dtype == torch.bfloat16
            and all(v % 2 == 0 for v in (N, K, x.shape[1], x_col, x_head, y.shape[1], y_col, y_head))):
        lib.call("fwb_head_linear_mma", x_ptr, ptr(w), y_ptr, x.shape[0], N, K, heads, c_longlong(x.shape[1]),
                 c_longlong(x_head), c_longlong(y.shape[1]), c_longlong(y_head), stream())
        return
    lib.call("fwb_head_linear", x_ptr, ptr(w), y_ptr, is_bf16(x), x.shape[0], N, K, heads,
             c_longlong(x.shape[1]), c_longlong(x_head), c_longlong(y.shape[1]), c_longlong(y_head), stream())


def latent_attention(qa: torch.Tensor, pool: torch.Tensor, sink: Optional[torch.Tensor], batch,
                     block_table: torch.Tensor, rank: int, used: int, scale: float) -> torch.Tensor:
    """Causal attention of every query row of qa [T][heads][row] over its request's cached latent
    rows (pool [pages][1][page_size][row]): scores over the first ``used`` columns, values the first
    ``rank``; ``sink`` (fp32 [heads]) joins every softmax denominator.  Returns [T][heads*rank]."""
    check_tensor("latent queries", qa)
    check_tensor("latent pool", pool, qa.dtype)
    T, heads, row = qa.shape
    if pool.dim() != 4 or pool.shape[1] != 1 or pool.shape[3] != row:
        raise KernelError(f"the latent pool must be [pages][1][page_size][{row}], got {tuple(pool.shape)}")
    if sink is not None:
        check_tensor("sink", sink, torch.float32, (heads,))
    _i32("block table", block_table)
    out = torch.empty((T, heads * rank), dtype=qa.dtype, device=qa.device)
    lib.call("fwb_latent_attention_simt", ptr(qa), ptr(pool), is_bf16(qa), ptr(sink), ptr(batch.positions),
             ptr(batch.tok_seg), ptr(block_table), block_table.shape[1], pool.shape[2], ptr(out), T, heads,
             rank, used, row, c_float(scale), stream())
    return out
