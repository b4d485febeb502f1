"""bf16 GEMM on the tcgen05 kernel, and the autograd ``linear`` built on it.

``gemm_nt/nn/tn`` launch ``cuda/gemm_tcgen05.cu`` for CUDA bf16 operands and
fall back to a plain fp32 ``torch.matmul`` on CPU (the oracle of the tests).
``linear(x, w)`` is ``x @ w.T`` with

* dx = dy @ w            (B operand read MN-major, no transpose copy)
* dW += dy.T @ x         (both operands MN-major; accumulated with fp32 atomics
                          straight into ``w.main_grad`` when the parameter has
                          one, which fuses micro-batch gradient accumulation)

The reference runs these as library GEMMs (src/model/qwen3_5_text.cc:86-89).
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from .. import _native as nv

_FORCE_LIBRARY = os.environ.get("CVERL_B200_GEMM", "native") == "cublas"

launch_counter = {"n": 0}


def count_launch(k: int = 1) -> None:
    launch_counter["n"] += k


def use_native(t: torch.Tensor) -> bool:
    if t.is_cuda and t.dtype != torch.bfloat16 and not _FORCE_LIBRARY:
        from ..utils import fallbacks
        fallbacks.note("gemm", f"dtype {t.dtype}: the tcgen05 GEMM takes bf16 operands")
    return t.is_cuda and t.dtype == torch.bfloat16 and not _FORCE_LIBRARY


def _lib_mm(a: torch.Tensor, b: torch.Tensor, alpha: float) -> torch.Tensor:
    """Library matmul: fp32 on CPU (test oracle), model dtype on CUDA (labelled baseline mode)."""
    if a.is_cuda:
        r = a @ b
    else:
        r = a.float() @ b.float()
    return r if alpha == 1.0 else r * alpha


def _row_major_2d(t: torch.Tensor) -> torch.Tensor:
    """2-D view with unit inner stride, 16-byte aligned base and row stride (what TMA needs)."""
    if t.dim() != 2:
        t = t.reshape(-1, t.shape[-1])
    per16 = 16 // t.element_size()
    if t.stride(1) == 1 and t.stride(0) % per16 == 0 and t.data_ptr() % 16 == 0:
        return t
    cols = t.shape[1]
    if cols % per16 == 0:
        t = t.contiguous()
        if t.data_ptr() % 16 == 0:
            return t
        return t.clone()
    # odd width: copy into a buffer whose rows are padded to 16 bytes and hand back the narrow view
    buf = torch.zeros((t.shape[0], (cols + per16 - 1) // per16 * per16), dtype=t.dtype, device=t.device)
    buf[:, :cols].copy_(t)
    return buf[:, :cols]


def _alloc_out(M: int, N: int, dtype, device) -> torch.Tensor:
    """[M, N] output whose row stride is a multiple of 16 bytes (vector stores in the epilogue)."""
    per16 = 16 // torch.empty((), dtype=dtype).element_size()
    Np = (N + per16 - 1) // per16 * per16
    buf = torch.empty((M, Np), dtype=dtype, device=device)
    return buf if Np == N else buf[:, :N]


def gemm_raw(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, M: int, N: int, K: int, *, a_mn: bool,
             b_mn: bool, epi: int, alpha: float = 1.0, split_k: int = 0, block_n: int = 0,
             tile_group=None, b_group_rows: int = 0, b_total_rows: int = 0, k_group_offsets=None,
             num_groups: int = 0, c_group_stride: int = 0, targets=None, part_max=None, part_sum=None,
             tgt_logit=None, lse=None, gscale=None, max_ctas: int = 0, mirrors=(), scatter=None,
             ldc: int = 0, row_addr=None) -> None:
    """One launch of the tcgen05 GEMM. Operands are 2-D bf16 tensors with unit inner stride.

    ``scatter=(bases, rows_per_owner)``: reduce-scatter epilogue - row block ``row // rows_per_owner`` of the
    bf16 result is stored only at raw address ``bases[block] + (row * ldc + col) * 2`` (``out`` is None and ``ldc``
    is given).  ``row_addr`` (int64 [M], device): output row r is stored only at byte address ``row_addr[r]``
    (0 drops it); ``out`` is None."""
    lib = nv.cuda()
    args = nv.GemmArgs()
    args.A, args.B, args.C = a.data_ptr(), b.data_ptr(), out.data_ptr() if out is not None else None
    args.lda, args.ldb = a.stride(0), b.stride(0)
    args.ldc = out.stride(0) if out is not None else ldc
    args.M, args.N, args.K = M, N, K
    args.a_mn, args.b_mn = int(a_mn), int(b_mn)
    args.epi, args.alpha = epi, alpha
    args.split_k, args.block_n, args.group_m, args.max_ctas = split_k, block_n, 0, max_ctas
    args.tile_group = nv.ptr(tile_group)
    args.b_group_rows, args.b_total_rows = b_group_rows, b_total_rows
    args.k_group_offsets = nv.ptr(k_group_offsets)
    args.num_groups, args.c_group_stride = num_groups, c_group_stride
    args.targets, args.part_max, args.part_sum = nv.ptr(targets), nv.ptr(part_max), nv.ptr(part_sum)
    args.tgt_logit, args.lse, args.gscale = nv.ptr(tgt_logit), nv.ptr(lse), nv.ptr(gscale)
    args.status = nv.status_word(a.device).data_ptr()
    args.n_mirror = len(mirrors)
    for i, m in enumerate(mirrors):   # raw addresses of peers' copies of ``out``
        args.mirror[i] = m
    if scatter is not None:
        bases, rows_per_owner = scatter
        args.scatter_rows = rows_per_owner
        for i, base in enumerate(bases):
            args.scatter_base[i] = base
    args.row_addr = nv.ptr(row_addr)
    rc = lib.cvb_gemm_bf16(C.byref(args), nv.stream())
    nv.check(rc, "cvb_gemm_bf16")
    count_launch()


def _pick_block_n(M: int, N: int) -> int:
    # 128 x 256 tiles unless that leaves most SMs idle and 128 x 128 fills more of them
    tiles256 = ((M + 127) // 128) * ((N + 255) // 256)
    if N <= 128 or (tiles256 < 148 and N % 256 != 0 and N % 128 == 0):
        return 128
    if tiles256 < 100:
        return 128
    return 256


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, *, out_dtype=None,
            alpha: float = 1.0) -> torch.Tensor:
    """``a [M,K] @ b[N,K].T -> [M,N]``"""
    M, K = a.shape
    N = b.shape[0]
    if not use_native(a):
        r = _lib_mm(a, b.t(), alpha).to(out_dtype or a.dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    a, b = _row_major_2d(a), _row_major_2d(b)
    dt = out_dtype or torch.bfloat16
    if out is None:
        out = _alloc_out(M, N, dt, a.device)
    epi = nv.EPI_STORE_BF16 if out.dtype == torch.bfloat16 else nv.EPI_STORE_F32
    gemm_raw(a, b, out, M, N, K, a_mn=False, b_mn=False, epi=epi, alpha=alpha, block_n=_pick_block_n(M, N))
    return out


def gemm_nn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, *, out_dtype=None,
            alpha: float = 1.0) -> torch.Tensor:
    """``a [M,K] @ b[K,N] -> [M,N]`` (b read MN-major)."""
    M, K = a.shape
    N = b.shape[1]
    if not use_native(a):
        r = _lib_mm(a, b, alpha).to(out_dtype or a.dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    a, b = _row_major_2d(a), _row_major_2d(b)
    dt = out_dtype or torch.bfloat16
    if out is None:
        out = _alloc_out(M, N, dt, a.device)
    epi = nv.EPI_STORE_BF16 if out.dtype == torch.bfloat16 else nv.EPI_STORE_F32
    gemm_raw(a, b, out, M, N, K, a_mn=False, b_mn=True, epi=epi, alpha=alpha, block_n=_pick_block_n(M, N))
    return out


def gemm_tn_acc(a: torch.Tensor, b: torch.Tensor, acc: torch.Tensor, *, alpha: float = 1.0) -> torch.Tensor:
    """``acc[M,N] (fp32) += a[K,M].T @ b[K,N]`` (both MN-major, split-K with fp32 atomics)."""
    K, M = a.shape
    N = b.shape[1]
    if not use_native(a):
        acc.add_(_lib_mm(a.t(), b, alpha).float())
        return acc
    a, b = _row_major_2d(a), _row_major_2d(b)
    assert acc.dtype == torch.float32 and acc.stride(1) == 1
    gemm_raw(a, b, acc, M, N, K, a_mn=True, b_mn=True, epi=nv.EPI_ATOMIC_F32, alpha=alpha,
             block_n=256 if N >= 256 else 128)
    return acc


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm_nt(x2, w)
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm_nn(dy2, w).reshape(x.shape)
        dw = None
        if ctx.needs_input_grad[1]:
            main_grad = getattr(w, "main_grad", None)
            if main_grad is not None:
                gemm_tn_acc(dy2, x2, main_grad)
            else:
                acc = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
                gemm_tn_acc(dy2, x2, acc)
                dw = acc.to(w.dtype)
        return dx, dw


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` with the tcgen05 GEMM in forward and backward."""
    return _Linear.apply(x, w)
