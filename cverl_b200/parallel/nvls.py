"""NVSwitch multicast (NVLS) buffers and the collectives written on them.

``NvlsBuffer`` is a same-sized allocation on every rank of a group that is additionally bound to an NVSwitch
multicast object, so that there is one more address - the multicast address - at which a store reaches every
rank's copy and a reducing load returns the sum of all copies (``multimem.st`` / ``multimem.ld_reduce``,
``cuda/nvls_ops.cu``).  The allocation and the binding come from PyTorch's symmetric-memory allocator
(``torch.distributed._symmetric_memory``: ``cuMemCreate`` + ``cuMulticast*`` behind one call); rank
synchronisation uses this package's own flag barrier with bounded waits (``SymmBarrier``), not the allocator's.

* ``NvlsBroadcaster``     trainer -> rollout weight push: the sender stores each 16 bytes once, the switch
                          delivers them to every rank of the group (reference: ncclBroadcast per tensor,
                          src/distributed/weight_sync.cc:140-189).
* ``NvlsReduceScatter``   ZeRO gradient reduce-scatter with the sum formed in the switch: each rank receives
                          only its shard (reference: ncclReduceScatter, src/distributed/optimizer_sharding.cc:463-585).
* ``NvlsAllReduce``       one-shot all-reduce of a bf16 buffer: every rank reduces and re-broadcasts its slice.

Multicast objects are for ranks that live and die together: a process that exits while its memory is still bound
takes the other ranks' mappings down with it.  The failure-detection tests and every path exercised by them
therefore stay on plain peer loads and stores (``parallel/symm.py``); these classes are opt-in.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as nv
from ..ops.gemm import count_launch
from .symm import SymmBarrier, SymmetricHeap


def available() -> bool:
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
    except Exception:
        return False
    return torch.cuda.is_available()


class NvlsBuffer:
    """``nbytes`` on every rank of ``group`` plus the multicast address of the set (collective constructor)."""

    def __init__(self, group, device, nbytes: int):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.device = torch.device(device)
        self.group = group if group is not None else dist.group.WORLD
        self.nbytes = (nbytes + 255) // 256 * 256
        self.local = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        self.local.zero_()
        self.handle = symm_mem.rendezvous(self.local, self.group)
        self.rank, self.world = self.handle.rank, self.handle.world_size
        self.multicast_ptr = int(self.handle.multicast_ptr)
        if self.multicast_ptr == 0:
            raise RuntimeError("this system gives no NVSwitch multicast address (NVLS unavailable)")
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]

    def tensor(self, numel: int, dtype: torch.dtype, offset_bytes: int = 0) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        return self.local[offset_bytes: offset_bytes + numel * esz].view(dtype)


class _WithBarrier:
    def __init__(self, group, device):
        self.heap = SymmetricHeap(group, device)
        self.barrier = SymmBarrier(self.heap)

    def close(self) -> None:
        self.heap.close()


class NvlsBroadcaster(_WithBarrier):
    """Weight push through the multicast address: ``push`` on the sender(s), ``sync`` on everyone."""

    def __init__(self, group, device, nbytes: int):
        super().__init__(group, device)
        self.buf = NvlsBuffer(group, device, nbytes)

    def tensor(self, numel: int, dtype: torch.dtype, offset_bytes: int = 0) -> torch.Tensor:
        return self.buf.tensor(numel, dtype, offset_bytes)

    def push(self, src: torch.Tensor, offset_bytes: int = 0, max_blocks: int = 0) -> None:
        """Stores ``src`` at ``offset_bytes`` of EVERY rank's buffer (the sender's own included)."""
        nbytes = src.numel() * src.element_size()
        if offset_bytes % 16 or offset_bytes + nbytes > self.buf.nbytes:
            raise ValueError("NvlsBroadcaster.push: offset must be a multiple of 16 bytes and the piece must fit")
        nv.check(nv.cuda().cvb_multimem_broadcast_store(src.data_ptr(), self.buf.multicast_ptr + offset_bytes, nbytes,
                                                        max_blocks, nv.stream()), "cvb_multimem_broadcast_store")
        count_launch()

    def sync(self) -> None:
        """Flag barrier on the current stream: after it every push issued before it has landed everywhere."""
        self.barrier()


class NvlsReduceScatter(_WithBarrier):
    """fp32 gradient buffer in multicast memory; ``reduce`` returns this rank's shard of the mean."""

    def __init__(self, group, device, numel: int):
        super().__init__(group, device)
        self.buf = NvlsBuffer(group, device, numel * 4)
        self.grad = self.buf.tensor(numel, torch.float32)
        self.sq = torch.zeros(1, dtype=torch.float32, device=self.buf.device)

    def reduce(self, out_shard: torch.Tensor, begin: int, accumulate: bool = False, max_blocks: int = 0) -> torch.Tensor:
        """``out_shard (+)= mean over ranks of grad[begin : begin + len]``; returns the 1-float squared norm of the
        result.  Brackets the kernel with barriers: all gradients written before, all reads done after."""
        self.barrier()
        self.sq.zero_()
        nv.check(nv.cuda().cvb_multimem_reduce_scatter(self.buf.multicast_ptr, begin, out_shard.numel(),
                                                       1.0 / self.buf.world, out_shard.data_ptr(), int(accumulate),
                                                       self.sq.data_ptr(), max_blocks, nv.stream()),
                 "cvb_multimem_reduce_scatter")
        count_launch()
        self.barrier()
        return self.sq


def allreduce_slice(n: int, world: int, rank: int):
    """``(begin, length)`` of the slice of an ``n``-element bf16 buffer that ``rank`` reduces and re-broadcasts: equal
    parts rounded up to 8 elements (16 bytes), the last rank taking what is left; the slices tile ``[0, n)``."""
    per = (n // world + 7) // 8 * 8
    lo = min(rank * per, n)
    hi = min(lo + per, n) if rank < world - 1 else n
    return lo, max(hi - lo, 0)


class NvlsAllReduce(_WithBarrier):
    """bf16 buffer in multicast memory; ``all_reduce`` sums it over the ranks in place on every rank."""

    def __init__(self, group, device, numel: int):
        super().__init__(group, device)
        self.buf = NvlsBuffer(group, device, numel * 2)
        self.data = self.buf.tensor(numel, torch.bfloat16)
        self.numel = numel

    def all_reduce(self, numel: Optional[int] = None, max_blocks: int = 0) -> torch.Tensor:
        n = self.numel if numel is None else numel
        lo, length = allreduce_slice(n, self.buf.world, self.buf.rank)
        hi = lo + length
        if length % 8:
            raise ValueError("NvlsAllReduce: element count must be a multiple of 8")
        self.barrier()                   # every rank's partial result is in its buffer
        nv.check(nv.cuda().cvb_multimem_allreduce_bf16(self.buf.multicast_ptr, lo, hi - lo, max_blocks, nv.stream()),
                 "cvb_multimem_allreduce_bf16")
        count_launch()
        self.barrier()                   # every slice has been reduced and re-broadcast
        return self.data[:n]
