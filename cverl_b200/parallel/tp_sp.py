"""Tensor parallelism with a token-sharded residual stream: GEMM -> reduce-scatter and all-gather -> GEMM
without a library collective.

Megatron-style tensor parallelism all-reduces a ``[tokens, hidden]`` partial product after every
row-parallel linear (the reference: src/model/qwen3_5_text.cc:195-205,1023,1225,1449), and every rank then
repeats the residual add and the RMSNorm on ALL tokens.  Here the residual stream lives sharded by token
rows (rank ``r`` of a group of ``n`` owns rows ``[r*T/n, (r+1)*T/n)``), and each all-reduce is split into
its two halves, each fused into the kernel next to it:

* **GEMM -> reduce-scatter.**  The row-parallel GEMM's epilogue stores every finished 128-row slab of its
  partial product ONLY to the rank that owns those rows - into slot ``me`` of that rank's ``parts`` buffer,
  its own memory or a peer's over NVLink (``scatter`` mode of ``cuda/gemm_tcgen05.cu``) - tile by tile while
  the tensor cores run the next tile.  Nothing else is sent: ``(n-1)/n`` of the tile bytes cross the link.
* **norm -> all-gather -> GEMM.**  After one flag barrier, ``sp_add_rmsnorm_fwd`` (``cuda/norm_ops.cu``) sums
  the ``n`` slots of its own rows with the residual, normalises ``T/n`` rows instead of ``T`` and writes them
  into its row range of the gathered activation.  The rows then travel to the peers' copies over NVLink on a
  side stream (copy engines, no SM) while the column-parallel GEMM already runs on the rows this rank
  produced; a second barrier on that side stream tells each rank that its peers' rows have landed, and the
  GEMM's remaining row blocks follow.  Each remote row crosses the link once and is read from local memory;
  no TMA load ever targets peer memory.  (``overlap=False`` makes the norm kernel store to every rank
  directly and the GEMM wait for all rows: one launch more exposed to the link, fewer launches.)

The backward pass is the mirror image: the column-parallel linear's input-gradient GEMM scatters its partial
product the same way, ``sp_add_rmsnorm_bwd`` sums the slots, runs the norm backward on ``T/n`` rows and
stores the result into the gathered output-gradient of the row-parallel linear on every rank.

Gathered forward activations are kept for the weight-gradient GEMMs, so they live in an arena of
peer-mapped slots, one per norm of the forward pass; ``begin_pass()`` rewinds it (one forward / backward in
flight at a time: no pipeline parallelism on this path).  All waits are the bounded flag barrier of
``parallel/symm.py``.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional

import torch

from .. import _native as nv
from ..ops import gemm as G
from ..ops.gemm import count_launch
from .symm import SymmBarrier, SymmetricHeap
from .tp_symm import _acc_dw


class TpSp:
    def __init__(self, group, device, max_rows: int, hidden: int, arena_slots: int, overlap: bool = True):
        """``max_rows``: tokens of one micro-batch over the whole group (a multiple of ``128 * world``)."""
        self.heap = SymmetricHeap(group, device)
        self.world, self.rank = self.heap.world, self.heap.index
        self.device = torch.device(device)
        if max_rows % (128 * self.world):
            raise ValueError("TpSp needs the token count to be a multiple of 128 * tensor-parallel size")
        self.max_rows, self.hidden = max_rows, hidden
        self.slot_bytes = max_rows * hidden * 2
        # parts[j]: [world][rows_local, hidden] - slot s = the partial product of rank s for this rank's rows
        self.parts = [self.heap.alloc(self.slot_bytes) for _ in range(2)]
        self.gath = [self.heap.alloc(self.slot_bytes) for _ in range(2)]      # gathered output gradients
        self.arena = self.heap.alloc(self.slot_bytes * arena_slots)           # gathered forward activations
        self.arena_slots = arena_slots
        self.barrier = SymmBarrier(self.heap)
        # the gather travels on a side stream with a barrier of its own (flag epochs are per barrier object:
        # two streams must not share one)
        self.overlap = overlap = overlap and os.environ.get("CVERL_B200_TP_SP_OVERLAP", "1") != "0"
        self.side = torch.cuda.Stream(device=self.device) if overlap else None
        self.side_barrier = SymmBarrier(self.heap) if overlap else None
        self.pending = None            # (event, first row, end row) of a gather still in flight
        self._views = {}               # (buffer id, byte offset, rows) -> cached tensor view
        self.cur_parts = 0
        self.cur_gath = 0
        self.slot = 0
        self.active = False

    # ------------------------------------------------------------------------------------------------
    def view(self, buf, rows: int, offset_bytes: int = 0) -> torch.Tensor:
        """``[rows, hidden]`` bf16 view of a symmetric buffer; the views are cached (building one from a raw pointer
        costs tens of microseconds of host time, and there are four per norm)."""
        key = (id(buf), offset_bytes, rows)
        t = self._views.get(key)
        if t is None:
            t = buf.tensor(rows * self.hidden, torch.bfloat16, offset_bytes).view(rows, self.hidden)
            self._views[key] = t
        return t

    def fits(self, rows: int, hidden: int) -> bool:
        return (hidden == self.hidden and rows <= self.max_rows and rows % (128 * self.world) == 0
                and hidden % 64 == 0)

    def begin_pass(self) -> None:
        """Start of a forward pass: the arena's slots are free again once every rank has finished the previous
        backward, whose last GEMMs still read them - hence the barrier."""
        self.slot = 0
        self.barrier()

    def _next_parts(self):
        self.cur_parts ^= 1
        return self.parts[self.cur_parts]

    def scatter_gemm(self, a: torch.Tensor, b: torch.Tensor, rows: int, K: int, b_mn: bool) -> torch.Tensor:
        """``a @ b^T`` (or ``a @ b`` with ``b_mn``) -> [rows, hidden] partial product, reduce-scattered: row block
        ``o`` is stored into slot ``rank`` of rank ``o``'s parts buffer.  Returns this rank's parts buffer viewed
        as [rows, hidden] (slot-major); its contents are complete only after the next barrier."""
        buf = self._next_parts()
        rl = rows // self.world
        ldc = self.hidden
        bases = []
        for owner in range(self.world):
            # address of (slot = my rank, row 0) on the owner, minus the owner's first global row
            bases.append(buf.peer_ptrs[owner] + (self.rank * rl - owner * rl) * ldc * 2)
        a, b = G._row_major_2d(a), G._row_major_2d(b)
        G.gemm_raw(a, b, None, rows, self.hidden, K, a_mn=False, b_mn=b_mn, epi=nv.EPI_STORE_BF16,
                   block_n=G._pick_block_n(rows, self.hidden), scatter=(bases, rl), ldc=ldc)
        return self.view(buf, rows)

    def push_rows(self, buf, offset_bytes: int, rl: int) -> None:
        """This rank's ``rl`` rows at ``offset_bytes`` of ``buf`` were just written locally (on the current
        stream): send them to the same place in every peer's copy on the side stream, then barrier there.  Leaves
        ``pending`` for the consumer, which may use rows ``[rank*rl, (rank+1)*rl)`` at once and the others after
        waiting for the event."""
        wrote = torch.cuda.Event()
        wrote.record(torch.cuda.current_stream(self.device))
        nbytes = rl * self.hidden * 2
        off = offset_bytes + self.rank * nbytes
        side = self.side.cuda_stream
        self.side.wait_event(wrote)
        copy = nv.cuda().cvb_device_memcpy_async
        for j in range(self.world):
            if j != self.rank:
                nv.check(copy(buf.peer_ptrs[j] + off, buf.peer_ptrs[self.rank] + off, nbytes, side),
                         "cudaMemcpyAsync(peer)")
        self.side_barrier(side)
        landed = torch.cuda.Event()
        landed.record(self.side)
        self.pending = (landed, self.rank * rl, (self.rank + 1) * rl)

    def take_pending(self):
        p, self.pending = self.pending, None
        return p

    def wait_pending(self) -> None:
        p = self.take_pending()
        if p is not None:
            torch.cuda.current_stream(self.device).wait_event(p[0])

    def parts_view(self, rows: int) -> torch.Tensor:
        return self.view(self.parts[self.cur_parts], rows)


def _ptr_array(ptrs: List[int]):
    return (C.c_void_p * len(ptrs))(*ptrs)


class _SpRowLinear(torch.autograd.Function):
    """Row-parallel linear whose output is left reduce-scattered: returns the parts buffer ``[T, H]`` (slot-major
    handle, consumed by ``_SpNormGather``); its gradient is the gathered ``[T, H]`` output gradient."""

    @staticmethod
    def forward(ctx, x, w, sp: TpSp):
        ctx.save_for_backward(x, w)
        ctx.sp = sp
        x2 = x.reshape(-1, x.shape[-1])
        return sp.scatter_gemm(x2, w, x2.shape[0], x2.shape[1], False)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        sp = ctx.sp
        x2 = x.reshape(-1, x.shape[-1])
        pend = sp.take_pending()
        if pend is None or getattr(w, "main_grad", None) is None:
            if pend is not None:
                torch.cuda.current_stream(sp.device).wait_event(pend[0])
            dx = G.gemm_nn(dy, w).reshape(x.shape) if ctx.needs_input_grad[0] else None
            dw = _acc_dw(ctx, dy, x2, w) if ctx.needs_input_grad[1] else None
            return dx, dw, None
        # the rows this rank produced are here already: start on them while the peers' rows arrive
        landed, r0, r1 = pend
        T = dy.shape[0]
        dx2 = torch.empty((T, w.shape[1]), dtype=torch.bfloat16, device=dy.device) if ctx.needs_input_grad[0] else None
        blocks = [(r0, r1)] + [b for b in ((0, r0), (r1, T)) if b[1] > b[0]]
        for k, (a, b) in enumerate(blocks):
            if k == 1:
                torch.cuda.current_stream(sp.device).wait_event(landed)
            if dx2 is not None:
                G.gemm_nn(dy[a:b], w, out=dx2[a:b])
            if ctx.needs_input_grad[1]:
                G.gemm_tn_acc(dy[a:b], x2[a:b], w.main_grad)
        return (dx2.reshape(x.shape) if dx2 is not None else None), None, None


class _SpColLinear(torch.autograd.Function):
    """Column-parallel linear on the gathered activation; its input gradient leaves reduce-scattered in the parts
    buffers (the returned tensor is only a handle of the right shape)."""

    @staticmethod
    def forward(ctx, x, w, sp: TpSp):
        ctx.save_for_backward(x, w)
        ctx.sp = sp
        pend = sp.take_pending()
        if pend is None:
            return G.gemm_nt(x, w)
        # the rows this rank normalised are here already: start on them while the peers' rows arrive
        landed, r0, r1 = pend
        T = x.shape[0]
        y = G._alloc_out(T, w.shape[0], torch.bfloat16, x.device)
        G.gemm_nt(x[r0:r1], w, out=y[r0:r1])
        torch.cuda.current_stream(sp.device).wait_event(landed)
        if r0 > 0:
            G.gemm_nt(x[:r0], w, out=y[:r0])
        if r1 < T:
            G.gemm_nt(x[r1:], w, out=y[r1:])
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        sp = ctx.sp
        dy2 = dy.reshape(-1, dy.shape[-1])
        handle = sp.scatter_gemm(dy2, w, dy2.shape[0], dy2.shape[1], True)
        # the weight gradient does not depend on the scatter: it runs while those stores drain over NVLink
        dw = _acc_dw(ctx, dy2, x, w) if ctx.needs_input_grad[1] else None
        return handle, dw, None


class _SpNormGather(torch.autograd.Function):
    """``(parts | local delta, resid) -> (gathered rmsnorm(delta + resid) [T, H], delta + resid [T/n, H])``."""

    @staticmethod
    def forward(ctx, delta, resid, w, eps, w_offset, sp: TpSp, from_parts: bool, grad_in_tensor: bool):
        H = sp.hidden
        if from_parts:
            rows = delta.shape[0]
            rl = rows // sp.world
            src, stride, nparts = delta, rl * H, sp.world
        else:
            rl = delta.shape[0]
            rows = rl * sp.world
            src, stride, nparts = delta.contiguous(), 0, 1
        if sp.slot >= sp.arena_slots:
            raise RuntimeError("TpSp arena exhausted: more norms in one pass than slots")
        slot_off = sp.slot * sp.slot_bytes
        sp.slot += 1
        resid_out = torch.empty((rl, H), dtype=torch.bfloat16, device=sp.device)
        rstd = torch.empty(rl, dtype=torch.float32, device=sp.device)
        r2 = resid.contiguous() if resid is not None else None
        if from_parts:
            sp.barrier()                     # every rank's scatter stores into my parts buffer have landed
        if sp.overlap:
            dst, ndst = _ptr_array([sp.arena.peer_ptrs[sp.rank] + slot_off]), 1
        else:
            dst, ndst = _ptr_array([p + slot_off for p in sp.arena.peer_ptrs]), sp.world
        nv.check(nv.cuda().cvb_sp_add_rmsnorm_fwd(src.data_ptr(), stride, nparts, nv.ptr(r2), w.data_ptr(), dst,
                                                  ndst, sp.rank * rl, resid_out.data_ptr(), rstd.data_ptr(),
                                                  rl, H, eps, w_offset, nv.stream()), "cvb_sp_add_rmsnorm_fwd")
        count_launch()
        if sp.overlap:
            sp.push_rows(sp.arena, slot_off, rl)
            if grad_in_tensor:               # the consumer is not one of this module's GEMMs: wait here
                sp.wait_pending()
        else:
            sp.barrier()                     # every rank's rows of the gathered activation are in place
        ctx.save_for_backward(resid_out, w, rstd)
        ctx.sp, ctx.w_offset, ctx.rl = sp, w_offset, rl
        ctx.from_parts, ctx.has_resid, ctx.grad_in_tensor = from_parts, resid is not None, grad_in_tensor
        return sp.view(sp.arena, rows, slot_off), resid_out

    @staticmethod
    def backward(ctx, d_full, d_resid_out):
        from ..ops.norm import _wgrad_buffer
        h, w, rstd = ctx.saved_tensors
        sp, rl = ctx.sp, ctx.rl
        H = sp.hidden
        rows = rl * sp.world
        if ctx.grad_in_tensor:
            # the consumer's gradient is already summed over the group (LM head): read this rank's rows of it
            g = d_full.contiguous()
            src, stride, nparts = g[sp.rank * rl:(sp.rank + 1) * rl], 0, 1
        else:
            sp.barrier()                     # the input-gradient partials of all ranks have landed in my parts
            src, stride, nparts = sp.parts_view(rows), rl * H, sp.world
        dres = d_resid_out.contiguous() if d_resid_out is not None else None
        dx = torch.empty((rl, H), dtype=torch.bfloat16, device=sp.device)
        dwbuf, is_main = _wgrad_buffer(w)
        if ctx.from_parts:
            sp.cur_gath ^= 1
            gbuf = sp.gath[sp.cur_gath]
            if sp.overlap:
                dst, ndst = _ptr_array([gbuf.peer_ptrs[sp.rank]]), 1
            else:
                dst, ndst = _ptr_array(list(gbuf.peer_ptrs)), sp.world
        else:
            dst, ndst = None, 0
        nv.check(nv.cuda().cvb_sp_add_rmsnorm_bwd(src.data_ptr(), stride, nparts, h.data_ptr(), w.data_ptr(),
                                                  rstd.data_ptr(), nv.ptr(dres), dx.data_ptr(), dst, ndst,
                                                  sp.rank * rl, dwbuf.data_ptr(), rl, H, ctx.w_offset, nv.stream()),
                 "cvb_sp_add_rmsnorm_bwd")
        count_launch()
        dw = None if is_main else dwbuf.to(w.dtype)
        if ctx.from_parts:
            if sp.overlap:
                sp.push_rows(gbuf, 0, rl)    # consumed by the row-parallel linear's backward, own rows first
            else:
                sp.barrier()                 # the gathered output gradient is complete on every rank
            d_delta = sp.view(gbuf, rows)
        else:
            d_delta = dx
        return d_delta, (dx if ctx.has_resid else None), dw, None, None, None, None, None


def row_linear(x: torch.Tensor, w: torch.Tensor, sp: TpSp) -> torch.Tensor:
    return _SpRowLinear.apply(x, w, sp)


def col_linear(x: torch.Tensor, w: torch.Tensor, sp: TpSp) -> torch.Tensor:
    return _SpColLinear.apply(x, w, sp)


def norm_gather(delta: torch.Tensor, resid: Optional[torch.Tensor], w: torch.Tensor, eps: float, w_offset: float,
                sp: TpSp, from_parts: bool, grad_in_tensor: bool = False):
    """See ``_SpNormGather``.  ``from_parts``: ``delta`` is the handle a ``row_linear`` returned (else a local
    ``[T/n, H]`` tensor, e.g. the embedding rows).  ``grad_in_tensor``: the gathered output's gradient arrives as a
    full tensor already summed over the group (final norm before the LM head) instead of through the parts."""
    return _SpNormGather.apply(delta, resid, w, eps, w_offset, sp, from_parts, grad_in_tensor)
