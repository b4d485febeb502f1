"""Grouped expert GEMM on the tcgen05 kernel (MoE experts).

Rows of ``x`` are sorted by expert and every expert's segment is padded to a multiple of
128 rows, so an M tile never straddles two experts: ``tile_group[m_tile]`` names the expert
(or -1 for an unused tile) and selects the expert's weight block by a row offset in the
stacked weight.  Forward ``y = x W_e^T``; backward ``dx = dy W_e`` (weights read MN-major)
and ``dW_e += dy_e^T x_e`` with each expert's token range as its K range, accumulated with
fp32 atomics into ``w.main_grad``.  No host synchronisation anywhere.
Reference: at::_grouped_mm over sorted tokens with a transposed weight copy per call
(src/model/qwen3_5_text.cc:971-976).
"""
from __future__ import annotations

import torch

from .. import _native as nv
from .gemm import gemm_raw, use_native, _alloc_out

TILE_M = 128


def grouped_linear_ref(x, w, tile_group):
    """x [M_pad, K], w [E, N, K], tile_group [M_pad/128] -> [M_pad, N] (zeros on unused tiles)."""
    M = x.shape[0]
    E, N, K = w.shape
    rows_group = tile_group.long().repeat_interleave(TILE_M)[:M]
    y = x.new_zeros((M, N))
    for e in range(E):
        sel = (rows_group == e).nonzero().squeeze(-1)
        if sel.numel():
            y[sel] = (x[sel].float() @ w[e].float().t()).to(x.dtype)
    return y


class _GroupedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, tile_group, group_offsets):
        M, K = x.shape
        E, N, _ = w.shape
        w2 = w.view(E * N, K)
        y = torch.zeros((M, N), dtype=x.dtype, device=x.device)   # unused tiles stay zero
        gemm_raw(x, w2, y, M, N, K, a_mn=False, b_mn=False, epi=nv.EPI_STORE_BF16, block_n=256 if N >= 256 else 128,
                 tile_group=tile_group, b_group_rows=N, b_total_rows=E * N)
        ctx.save_for_backward(x, w, tile_group, group_offsets)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, tile_group, group_offsets = ctx.saved_tensors
        M, K = x.shape
        E, N, _ = w.shape
        dy = dy.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.zeros((M, K), dtype=x.dtype, device=x.device)
            # dx = dy @ W_e : GEMM K = N (out features), B = W_e [N, K] read MN-major, row offset e*N
            gemm_raw(dy, w.view(E * N, K), dx, M, K, N, a_mn=False, b_mn=True, epi=nv.EPI_STORE_BF16,
                     block_n=256 if K >= 256 else 128, tile_group=tile_group, b_group_rows=N, b_total_rows=E * N)
        dw = None
        if ctx.needs_input_grad[1]:
            main_grad = getattr(w, "main_grad", None)
            acc = main_grad if main_grad is not None else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
            # dW_e[N, K] += dy_e^T x_e : both operands MN-major, K range = expert e's rows
            gemm_raw(dy, x, acc.view(E * N, K), N, K, M, a_mn=True, b_mn=True, epi=nv.EPI_ATOMIC_F32,
                     block_n=256 if K >= 256 else 128, k_group_offsets=group_offsets, num_groups=E,
                     c_group_stride=N * K)
            if main_grad is None:
                dw = acc.to(w.dtype)
        return dx, dw, None, None


def grouped_linear(x: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor,
                   group_offsets: torch.Tensor) -> torch.Tensor:
    """``y[r] = x[r] @ w[expert(r)].T`` for expert-sorted, 128-row padded ``x``.

    ``tile_group`` int32 [M_pad/128]; ``group_offsets`` int32 [E+1] padded row offsets.
    """
    if use_native(x) and x.shape[0] % TILE_M == 0 and x.shape[1] % 8 == 0 and w.shape[1] % 8 == 0:
        return _GroupedLinear.apply(x.contiguous(), w, tile_group.to(torch.int32), group_offsets.to(torch.int32))
    return _grouped_linear_autograd_ref(x, w, tile_group)


def _grouped_linear_autograd_ref(x, w, tile_group):
    M = x.shape[0]
    E = w.shape[0]
    rows_group = tile_group.long().repeat_interleave(TILE_M)[:M]
    onehot = torch.nn.functional.one_hot(rows_group.clamp_min(0), E).to(x.dtype) * (rows_group >= 0).unsqueeze(-1)
    # y = sum_e mask_e * (x @ w_e^T): differentiable and free of data-dependent shapes
    y = torch.einsum("mk,enk->men", x.float(), w.float())
    return (y * onehot.float().unsqueeze(-1)).sum(1).to(x.dtype)
