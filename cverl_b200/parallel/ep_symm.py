"""Expert-parallel dispatch / combine over peer-mapped memory, without a host read.

Every (token, slot) row routed to an expert on another rank is stored straight into that rank's receive
buffer over NVLink by ``cvb_p2p_scatter_rows`` (one warp per row); expert outputs are pulled back with
``cvb_p2p_gather_rows``.  The destination row of every routed entry is computed on the device from a
table of per-(source, destination) counts that the ranks push to each other first, so the layer never
synchronises with the host (the all-to-all path reads the split sizes on the host).  The backward of a
dispatch is a gather, the backward of a combine is a scatter.

The combine can also ride on the experts' down projection (``fused_down_combine``, the default): the grouped GEMM's
epilogue stores every output row straight into the return buffer of the rank the token came from, addressed
through a per-row table that ``plan`` builds from the (source rank, source entry) pair each dispatched row carries.

Buffers have a fixed capacity (``capacity_rows`` per rank); rows beyond the received count are marked with
the expert id ``num_local_experts`` and skipped by the grouped GEMM.  Overflow sets a device flag that
``check()`` turns into an exception.

The reference exchanges rows with four NCCL all-to-alls per layer (src/distributed/expert_parallel.cc:43-167).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as nv
from ..ops.gemm import count_launch
from .symm import SymmBarrier, SymmetricHeap


def plan_rows(table: torch.Tensor, rank: int, dst_rank: torch.Tensor, capacity_rows: int):
    """Destination row of every routed entry, from the count table ``table[src, dst]`` (int64) that the ranks
    exchanged: entries for one destination land after the rows of all lower source ranks, in their original
    order.  Returns ``(peer_rank int32 [n], peer_row int64 [n], overflow int32 [1])``.  A destination that would
    receive more than ``capacity_rows`` rows sets ``overflow``, and the entries that do not fit get rank -1,
    which the row kernels leave out - nothing is ever written past a buffer.  Pure tensor arithmetic: runs on
    any device."""
    world = table.shape[0]
    n = dst_rank.numel()
    dev = dst_rank.device
    base = table[:rank].sum(0)
    if dst_rank.is_cuda and n > 0:
        # stable position of every entry inside its destination's group from the layout kernels (no sort)
        from ..models.moe import expert_layout
        pos, _, starts32, _ = expert_layout(dst_rank, world, tile_m=1)
        peer_row = pos - starts32.to(torch.int64)[dst_rank] + base[dst_rank]
    else:
        counts = torch.bincount(dst_rank, minlength=world)[:world].to(torch.int64)
        order = torch.argsort(dst_rank, stable=True)
        starts = torch.zeros(world + 1, dtype=torch.int64, device=dev)
        starts[1:] = counts.cumsum(0)
        sorted_dst = dst_rank[order]
        idx_in_seg = torch.arange(n, device=dev) - starts[sorted_dst]
        peer_row = torch.empty(n, dtype=torch.int64, device=dev)
        peer_row[order] = base[sorted_dst] + idx_in_seg
    fits = peer_row < capacity_rows
    peer_rank = torch.where(fits, dst_rank.to(torch.int32), torch.full_like(dst_rank, -1, dtype=torch.int32))
    peer_row = torch.where(fits, peer_row, torch.zeros_like(peer_row))
    overflow = (table.sum(0).max() > capacity_rows).to(torch.int32).reshape(1)
    return peer_rank, peer_row, overflow


class EpSymm:
    def __init__(self, group, device, capacity_rows: int, hidden: int):
        self.heap = SymmetricHeap(group, device)
        self.world, self.rank = self.heap.world, self.heap.index
        self.device = torch.device(device)
        self.cap, self.hidden = capacity_rows, hidden
        row = hidden * 2
        self.row_bytes = row
        self.b_rows = self.heap.alloc(capacity_rows * row)      # dispatched activations (forward)
        self.b_out = self.heap.alloc(capacity_rows * row)       # expert outputs to be pulled (forward)
        self.b_gout = self.heap.alloc(capacity_rows * row)      # gradient of the expert outputs (backward)
        self.b_grow = self.heap.alloc(capacity_rows * row)      # gradient of the dispatched rows (backward)
        self.b_ids = self.heap.alloc(capacity_rows * 16)        # per received row: local expert, source entry, source rank
        self.b_ret = self.heap.alloc(capacity_rows * row)       # expert outputs stored back by the down-projection GEMM
        self.b_cnt = self.heap.alloc(self.world * 32)           # count table [src][8] int32
        self.rows = self.b_rows.tensor(capacity_rows * hidden, torch.bfloat16).view(capacity_rows, hidden)
        self.out = self.b_out.tensor(capacity_rows * hidden, torch.bfloat16).view(capacity_rows, hidden)
        self.gout = self.b_gout.tensor(capacity_rows * hidden, torch.bfloat16).view(capacity_rows, hidden)
        self.grow = self.b_grow.tensor(capacity_rows * hidden, torch.bfloat16).view(capacity_rows, hidden)
        self.ids = self.b_ids.tensor(capacity_rows * 4, torch.int32).view(capacity_rows, 4)
        self.ret = self.b_ret.tensor(capacity_rows * hidden, torch.bfloat16).view(capacity_rows, hidden)
        self.ret_bases = torch.tensor(self.b_ret.peer_ptrs, dtype=torch.int64, device=self.device)
        self.return_addr: Optional[torch.Tensor] = None         # set by ``plan``: see ``fused_down_combine``
        self.cnt = self.b_cnt.tensor(self.world * 8, torch.int32).view(self.world, 8)
        self.barrier = SymmBarrier(self.heap)
        self.overflow = torch.zeros(1, dtype=torch.int32, device=self.device)
        # down projection + combine in one GEMM (``fused_down_combine``); CVERL_B200_EP_FUSE_COMBINE=0 keeps them apart
        import os
        self.fuse_combine = os.environ.get("CVERL_B200_EP_FUSE_COMBINE", "1") != "0"
        self.fused_combines = 0                                  # layers that took the fused path (for tests)
        if self.world > 8:
            raise ValueError("EpSymm supports up to 8 ranks per expert-parallel group")

    # -- raw row movement ------------------------------------------------------------------------------
    def _move(self, gather: bool, local: torch.Tensor, buf, peer_rank: torch.Tensor, peer_row: torch.Tensor,
              row_bytes: int, capacity_rows: Optional[int] = None) -> None:
        """One warp per row between ``local`` and the peers' copies of ``buf``.  The kernel skips (and reports in
        the device status word) any entry whose rank or row lies outside the group / the buffer."""
        fn = nv.cuda().cvb_p2p_gather_rows if gather else nv.cuda().cvb_p2p_scatter_rows
        nv.check(fn(local.data_ptr(), buf.ptr_array(), self.world, peer_rank.data_ptr(), peer_row.data_ptr(),
                    peer_rank.numel(), row_bytes, self.cap if capacity_rows is None else capacity_rows,
                    nv.status_word(self.device).data_ptr(), nv.stream()), "cvb_p2p_rows")
        count_launch()

    def plan(self, dst_rank: torch.Tensor, local_expert: torch.Tensor, num_local: int):
        """Exchanges counts and returns ``(peer_rank int32 [n], peer_row int64 [n], recv_expert int64 [cap])``:
        where each routed entry lands, and the local expert of every row this rank receives (``num_local``
        marks unused capacity)."""
        n = dst_rank.numel()
        dev = self.device
        # Expert ids come from data (a router fed non-finite activations yields ids outside the table): such an
        # entry is routed nowhere and reported through the overflow flag (bit 1) - no index below may leave its table
        bad = (dst_rank < 0) | (dst_rank >= self.world) | (local_expert < 0) | (local_expert >= num_local)
        self.overflow.copy_(self.overflow | (bad.any().to(torch.int32) * 2))
        dst_rank = torch.where(bad, torch.zeros_like(dst_rank), dst_rank)
        local_expert = torch.where(bad, torch.zeros_like(local_expert), local_expert)
        counts = torch.bincount(dst_rank, minlength=self.world)[:self.world].to(torch.int32)
        mine = torch.zeros(8, dtype=torch.int32, device=dev)
        mine[:self.world] = counts
        self.barrier()                                           # previous users of the table are done
        src = mine.unsqueeze(0).expand(self.world, 8).contiguous()
        peers = torch.arange(self.world, dtype=torch.int32, device=dev)
        slot = torch.full((self.world,), self.rank, dtype=torch.int64, device=dev)
        self._move(False, src, self.b_cnt, peers, slot, 32, capacity_rows=self.world)
        self.barrier()
        table = self.cnt[:, :self.world].to(torch.int64)         # [src, dst]
        received = table[:, self.rank].sum().clamp(max=self.cap)
        peer_rank, peer_row, over = plan_rows(table, self.rank, dst_rank, self.cap)
        peer_rank = torch.where(bad, torch.full_like(peer_rank, -1), peer_rank)     # the row kernels skip rank -1
        self.overflow.copy_(self.overflow | over)
        # expert ids travel as 16-byte rows
        idrow = torch.zeros((n, 4), dtype=torch.int32, device=dev)
        idrow[:, 0] = local_expert.to(torch.int32)
        idrow[:, 1] = torch.arange(n, dtype=torch.int32, device=dev)     # where the expert's output goes back to
        idrow[:, 2] = self.rank
        self._move(False, idrow, self.b_ids, peer_rank, peer_row, 16)
        self.barrier()
        valid = torch.arange(self.cap, device=dev) < received
        recv_expert = torch.where(valid, self.ids[:, 0].to(torch.int64),
                                  torch.full((self.cap,), num_local, dtype=torch.int64, device=dev))
        # byte address, in the SOURCE rank's return buffer, of the row each received entry's output belongs to
        # (0 for unused capacity, and for a source rank / entry outside the tables: such a row is dropped)
        src_rank, src_row = self.ids[:, 2].to(torch.int64), self.ids[:, 1].to(torch.int64)
        ok = valid & (src_rank >= 0) & (src_rank < self.world) & (src_row >= 0) & (src_row < self.cap)
        addr = self.ret_bases[src_rank.clamp(0, self.world - 1)] + src_row.clamp(0, self.cap - 1) * self.row_bytes
        self.return_addr = torch.where(ok, addr, torch.zeros_like(addr))
        return peer_rank, peer_row, recv_expert

    def check(self) -> None:
        code = int(self.overflow.item())
        if code != 0:
            self.overflow.zero_()
            what = []
            if code & 1:
                what.append("a rank received more rows than its buffer capacity")
            if code & 2:
                what.append("the router produced expert ids outside the table (non-finite activations?)")
            raise RuntimeError("EpSymm: " + "; ".join(what))


class _Dispatch(torch.autograd.Function):
    """rows [n, H] -> this rank's receive buffer [cap, H] (a view of symmetric memory)."""

    @staticmethod
    def forward(ctx, rows, peer_rank, peer_row, eps: EpSymm):
        ctx.eps, ctx.n = eps, rows.shape[0]
        ctx.save_for_backward(peer_rank, peer_row)
        eps.barrier()                                            # receivers finished with the previous contents
        eps._move(False, rows.contiguous(), eps.b_rows, peer_rank, peer_row, eps.row_bytes)
        eps.barrier()
        return eps.rows.clone()

    @staticmethod
    def backward(ctx, g):
        eps = ctx.eps
        peer_rank, peer_row = ctx.saved_tensors
        eps.barrier()
        eps.grow.copy_(g)
        eps.barrier()                                            # every rank's gradient rows are in place
        # zeros, not empty: the gather leaves out the entries that did not fit a receive buffer (rank -1), and
        # their rows must be a defined value (an uninitialised row here becomes a non-finite weight gradient)
        out = torch.zeros((ctx.n, eps.hidden), dtype=torch.bfloat16, device=g.device)
        eps._move(True, out, eps.b_grow, peer_rank, peer_row, eps.row_bytes)
        return out, None, None, None


class _Combine(torch.autograd.Function):
    """expert outputs [cap, H] on the expert ranks -> rows [n, H] back at their source."""

    @staticmethod
    def forward(ctx, y, peer_rank, peer_row, eps: EpSymm):
        ctx.eps = eps
        ctx.save_for_backward(peer_rank, peer_row)
        eps.barrier()
        eps.out.copy_(y)
        eps.barrier()
        out = torch.zeros((peer_rank.numel(), eps.hidden), dtype=torch.bfloat16, device=y.device)   # see _Dispatch
        eps._move(True, out, eps.b_out, peer_rank, peer_row, eps.row_bytes)
        return out

    @staticmethod
    def backward(ctx, g):
        eps = ctx.eps
        peer_rank, peer_row = ctx.saved_tensors
        eps.barrier()
        eps.gout.zero_()
        eps.barrier()                                            # cleared everywhere before anyone writes
        eps._move(False, g.contiguous(), eps.b_gout, peer_rank, peer_row, eps.row_bytes)
        eps.barrier()
        return eps.gout.clone(), None, None, None


def dispatch(rows: torch.Tensor, peer_rank, peer_row, eps: EpSymm) -> torch.Tensor:
    return _Dispatch.apply(rows, peer_rank, peer_row, eps)


def combine(y: torch.Tensor, peer_rank, peer_row, eps: EpSymm) -> torch.Tensor:
    return _Combine.apply(y, peer_rank, peer_row, eps)


class _DownCombine(torch.autograd.Function):
    """The experts' down projection with the combine in its epilogue: every output row of the grouped GEMM is
    stored straight into the return buffer of the rank its token came from (``row_addr``), so the expert ranks
    neither materialise their outputs nor have them gathered.  ``act`` [m_pad, I] is expert-sorted and padded,
    ``row`` [cap] the padded row of every received entry; returns the ``n`` rows this rank routed, in entry order.
    Backward: the gradient rows travel to the expert ranks like any combine's (peer stores), then the grouped
    input- and weight-gradient GEMMs run on them."""

    @staticmethod
    def forward(ctx, act, w, tile_group, group_offsets, row_addr, row, peer_rank, peer_row, eps: EpSymm):
        from ..ops.gemm import gemm_raw
        M, K = act.shape
        E, N, _ = w.shape
        n = peer_rank.numel()
        eps.barrier()                                            # everyone has taken the previous layer's rows
        gemm_raw(act, w.view(E * N, K), None, M, N, K, a_mn=False, b_mn=False, epi=nv.EPI_STORE_BF16,
                 block_n=256 if N >= 256 else 128, tile_group=tile_group, b_group_rows=N, b_total_rows=E * N,
                 row_addr=row_addr, ldc=N)
        eps.barrier()                                            # every expert rank's stores have landed
        out = eps.ret[:n].clone()
        out.masked_fill_((peer_rank < 0).unsqueeze(-1), 0)       # entries that did not fit a receive buffer
        ctx.eps = eps
        ctx.save_for_backward(act, w, tile_group, group_offsets, row, peer_rank, peer_row)
        return out

    @staticmethod
    def backward(ctx, g):
        from ..ops.gemm import gemm_raw
        eps = ctx.eps
        act, w, tile_group, group_offsets, row, peer_rank, peer_row = ctx.saved_tensors
        M, K = act.shape
        E, N, _ = w.shape
        eps.barrier()
        eps.gout.zero_()
        eps.barrier()                                            # cleared everywhere before anyone writes
        eps._move(False, g.contiguous(), eps.b_gout, peer_rank, peer_row, eps.row_bytes)
        eps.barrier()
        dy = torch.zeros((M, N), dtype=torch.bfloat16, device=g.device).index_copy(0, row, eps.gout)
        dact = None
        if ctx.needs_input_grad[0]:
            dact = torch.zeros((M, K), dtype=act.dtype, device=act.device)
            gemm_raw(dy, w.view(E * N, K), dact, M, K, N, a_mn=False, b_mn=True, epi=nv.EPI_STORE_BF16,
                     block_n=256 if K >= 256 else 128, tile_group=tile_group, b_group_rows=N, b_total_rows=E * N)
        dw = None
        if ctx.needs_input_grad[1]:
            main_grad = getattr(w, "main_grad", None)
            acc = main_grad if main_grad is not None else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
            gemm_raw(dy, act, acc.view(E * N, K), N, K, M, a_mn=True, b_mn=True, epi=nv.EPI_ATOMIC_F32,
                     block_n=256 if K >= 256 else 128, k_group_offsets=group_offsets, num_groups=E,
                     c_group_stride=N * K)
            if main_grad is None:
                dw = acc.to(w.dtype)
        return dact, dw, None, None, None, None, None, None, None


def fused_down_combine(act, w, tile_group, group_offsets, row, peer_rank, peer_row, eps: EpSymm) -> torch.Tensor:
    """Down projection of the local experts whose epilogue IS the combine (see ``_DownCombine``).  ``row`` maps the
    ``cap`` received entries to padded rows; ``eps.return_addr`` (from ``plan``) names each entry's home."""
    m_pad = act.shape[0]
    eps.fused_combines += 1
    row_addr = torch.zeros(m_pad, dtype=torch.int64, device=act.device).index_copy(0, row, eps.return_addr)
    return _DownCombine.apply(act.contiguous(), w, tile_group.to(torch.int32), group_offsets.to(torch.int32), row_addr,
                              row, peer_rank, peer_row, eps)
