"""Tensor-parallel linear layers whose all-reduce is fused into the GEMM.

Row-parallel forward (``o_proj``, ``out_proj``, ``down_proj``) and column-parallel backward (the input
gradient of ``qkv``, ``in_proj``, ``gate_up``) each end in an all-reduce of a ``[tokens, hidden]`` partial
product over the TP group.  Here the tcgen05 GEMM's epilogue stores every finished tile both into this
rank's slot of a peer-mapped buffer and, over NVLink, into the same slot of every peer's copy (mirror
stores, tile by tile while the tensor cores work on the next tile); after one flag barrier each rank sums
the slots of its local copy.  No library collective runs on this path.

Two buffers alternate, so a rank can never overwrite a slot that a peer is still summing: a peer reaches
the barrier of use ``k+1`` only after its sum of use ``k``, and the buffer of use ``k`` is next written in
use ``k+2``.  All members of the group must issue the same sequence of fused linears (they do: same model).

The reference does GEMM then ``ncclAllReduce`` (src/distributed/parallel_ops.cc:28-58,
src/model/qwen3_5_text.cc:195-205).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as nv
from ..ops import gemm as G
from .symm import SymmBarrier, SymmetricHeap


class TpSymm:
    def __init__(self, group, device, max_rows: int, max_cols: int):
        self.heap = SymmetricHeap(group, device)
        self.world, self.rank = self.heap.world, self.heap.index
        self.slot_elems = (max_rows * max_cols + 7) // 8 * 8
        self.max_rows, self.max_cols = max_rows, max_cols
        self.bufs = [self.heap.alloc(self.world * self.slot_elems * 2) for _ in range(2)]
        self.barrier = SymmBarrier(self.heap)
        self.cur = 0
        self.device = torch.device(device)

    def fits(self, rows: int, cols: int) -> bool:
        return rows * cols <= self.slot_elems and cols % 64 == 0

    def _reduce_gemm(self, a: torch.Tensor, b: torch.Tensor, rows: int, cols: int, K: int, b_mn: bool) -> torch.Tensor:
        """all_reduce_sum over the group of ``a @ b^T`` (``b_mn`` False) or ``a @ b`` (``b_mn`` True)."""
        buf = self.bufs[self.cur]
        self.cur ^= 1
        off = self.rank * self.slot_elems * 2
        mine = buf.tensor(rows * cols, torch.bfloat16, off).view(rows, cols)
        mirrors = [p + off for i, p in enumerate(buf.peer_ptrs) if i != self.rank]
        a, b = G._row_major_2d(a), G._row_major_2d(b)
        G.gemm_raw(a, b, mine, rows, cols, K, a_mn=False, b_mn=b_mn, epi=nv.EPI_STORE_BF16,
                   block_n=G._pick_block_n(rows, cols), mirrors=mirrors)
        self.barrier()
        out = torch.empty((rows, cols), dtype=torch.bfloat16, device=self.device)
        nv.check(nv.cuda().cvb_sum_parts(buf.block.ptr, self.slot_elems, self.world, out.data_ptr(), rows * cols,
                                         nv.stream()), "cvb_sum_parts")
        G.count_launch()
        return out

    def reduce_gemm_nt(self, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        return self._reduce_gemm(a, w, a.shape[0], w.shape[0], a.shape[1], False)

    def reduce_gemm_nn(self, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        return self._reduce_gemm(a, w, a.shape[0], w.shape[1], a.shape[1], True)


def _acc_dw(ctx, dy2, x2, w):
    main_grad = getattr(w, "main_grad", None)
    if main_grad is not None:
        G.gemm_tn_acc(dy2, x2, main_grad)
        return None
    acc = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
    G.gemm_tn_acc(dy2, x2, acc)
    return acc.to(w.dtype)


class _RowParallelLinear(torch.autograd.Function):
    """y = all_reduce(x_shard @ w_shard^T); the backward is local."""

    @staticmethod
    def forward(ctx, x, w, tps: TpSymm):
        ctx.save_for_backward(x, w)
        x2 = x.reshape(-1, x.shape[-1])
        return tps.reduce_gemm_nt(x2, w).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2, x2 = dy.reshape(-1, dy.shape[-1]), x.reshape(-1, x.shape[-1])
        dx = G.gemm_nn(dy2, w).reshape(x.shape) if ctx.needs_input_grad[0] else None
        dw = _acc_dw(ctx, dy2, x2, w) if ctx.needs_input_grad[1] else None
        return dx, dw, None


class _ColumnParallelLinear(torch.autograd.Function):
    """y_shard = x @ w_shard^T with x replicated; dx = all_reduce(dy_shard @ w_shard)."""

    @staticmethod
    def forward(ctx, x, w, tps: TpSymm):
        ctx.save_for_backward(x, w)
        ctx.tps = tps
        x2 = x.reshape(-1, x.shape[-1])
        return G.gemm_nt(x2, w).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2, x2 = dy.reshape(-1, dy.shape[-1]), x.reshape(-1, x.shape[-1])
        dx = ctx.tps.reduce_gemm_nn(dy2, w).reshape(x.shape) if ctx.needs_input_grad[0] else None
        dw = _acc_dw(ctx, dy2, x2, w) if ctx.needs_input_grad[1] else None
        return dx, dw, None


def usable(tps: Optional[TpSymm], x: torch.Tensor, rows: int, cols: int) -> bool:
    return tps is not None and G.use_native(x) and tps.fits(rows, cols)


def row_parallel_linear(x: torch.Tensor, w: torch.Tensor, tps: TpSymm) -> torch.Tensor:
    return _RowParallelLinear.apply(x, w, tps)


def column_parallel_linear(x: torch.Tensor, w: torch.Tensor, tps: TpSymm) -> torch.Tensor:
    return _ColumnParallelLinear.apply(x, w, tps)
