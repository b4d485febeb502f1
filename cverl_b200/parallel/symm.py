"""Symmetric (peer-mapped) device memory and the collectives written on top of it.

``SymmetricHeap`` gives every rank of a process group a same-sized device allocation and a table
of pointers to all peers' copies (``cudaMalloc`` + CUDA IPC handles exchanged through the group).
Kernels in ``cuda/symm_ops.cu`` then move data with plain loads and stores over NVLink:

* ``SymmBarrier``     - flag exchange with bounded waits; a timeout surfaces as a kernel status code,
                        never as a hang;
* ``FusedZeroComm``   - ZeRO step without a library collective: reduce-scatter + mean + squared norm in
                        one kernel pulling from peers' gradient buffers, and FlatAdamW whose bf16 result
                        is stored into every peer's parameter buffer (the parameter all-gather);
* ``P2pBroadcaster``  - trainer -> rollout weight push with one read and one store per destination.

The reference reaches peers only through NCCL (src/distributed/nccl_collectives.cc).  TMA loads
with cluster multicast are never used on peer memory anywhere in this package.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from .. import _native as nv
from ..ops.gemm import count_launch


class _DeviceBlock:
    """A cudaMalloc'd block exposed to torch through the CUDA array interface."""

    def __init__(self, nbytes: int, device: torch.device):
        self.nbytes, self.device = nbytes, device
        p = C.c_void_p()
        with torch.cuda.device(device):
            nv.check(nv.cuda().cvb_device_malloc(C.addressof(p), nbytes), "cudaMalloc")
            nv.check(nv.cuda().cvb_device_memset(p.value, 0, nbytes, nv.stream()), "cudaMemset")
            torch.cuda.synchronize(device)  # zeroed before any peer can learn the address
        self.ptr = p.value

    def tensor(self, offset: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        typestr = {torch.float32: "<f4", torch.bfloat16: "<u2", torch.int32: "<i4", torch.uint8: "|u1",
                   torch.float16: "<f2", torch.int64: "<i8"}[dtype]

        class _View:
            pass
        v = _View()
        v.__cuda_array_interface__ = {"shape": (numel,), "typestr": typestr, "data": (self.ptr + offset, False),
                                      "version": 3, "strides": None}
        t = torch.as_tensor(v, device=self.device)
        if dtype == torch.bfloat16:
            t = t.view(torch.bfloat16)
        t._cverl_block = self
        assert t.numel() * esz <= self.nbytes - offset
        return t

    def free(self):
        if self.ptr:
            nv.cuda().cvb_device_free(self.ptr)
            self.ptr = None


class SymmBuffer:
    """One symmetric allocation: the local tensor view plus every group member's base pointer."""

    def __init__(self, block: _DeviceBlock, peer_ptrs: List[int], my_index: int, mapped: List[int]):
        self.block, self.peer_ptrs, self.my_index, self._mapped = block, peer_ptrs, my_index, mapped

    def tensor(self, numel: int, dtype: torch.dtype, offset_bytes: int = 0) -> torch.Tensor:
        return self.block.tensor(offset_bytes, numel, dtype)

    def ptr_array(self, offset_bytes: int = 0):
        return (C.c_void_p * len(self.peer_ptrs))(*[p + offset_bytes for p in self.peer_ptrs])


class SymmetricHeap:
    def __init__(self, group, device):
        import torch.distributed as dist
        self.group, self.device = group, torch.device(device)
        self.world = dist.get_world_size(group)
        self.index = dist.get_rank(group)
        self._buffers: List[SymmBuffer] = []

    def alloc(self, nbytes: int) -> SymmBuffer:
        """Collective over the group: everyone allocates ``nbytes`` and maps everyone else's block."""
        import torch.distributed as dist
        nbytes = (nbytes + 255) // 256 * 256
        block = _DeviceBlock(nbytes, self.device)
        raw = (C.c_ubyte * 64)()
        off = C.c_longlong()
        with torch.cuda.device(self.device):
            nv.check(nv.cuda().cvb_ipc_get_handle(block.ptr, C.addressof(raw), C.addressof(off)), "cudaIpcGetMemHandle")
        handles: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(handles, bytes(raw), group=self.group)
        ptrs, mapped = [], []
        for i, h in enumerate(handles):
            if i == self.index:
                ptrs.append(block.ptr)
                continue
            buf = (C.c_ubyte * 64).from_buffer_copy(h)
            base = C.c_void_p()
            with torch.cuda.device(self.device):
                nv.check(nv.cuda().cvb_ipc_open_handle(C.addressof(buf), C.addressof(base)), "cudaIpcOpenMemHandle")
            ptrs.append(base.value)
            mapped.append(base.value)
        sb = SymmBuffer(block, ptrs, self.index, mapped)
        self._buffers.append(sb)
        return sb

    def close(self) -> None:
        """Unmaps peers and frees local blocks; call with no kernel in flight and after a group barrier."""
        for sb in self._buffers:
            for p in sb._mapped:
                nv.cuda().cvb_ipc_close_handle(p)
            sb._mapped = []
        for sb in self._buffers:
            sb.block.free()
        self._buffers = []


class SymmBarrier:
    """Device-side barrier of the group on the current stream (monotonic epochs)."""

    def __init__(self, heap: SymmetricHeap):
        self.heap = heap
        self.flags = heap.alloc(256)
        self.epoch = 0

        self._ptrs = self.flags.ptr_array()
        self._status = nv.status_word(heap.device).data_ptr()

    def __call__(self, stream: Optional[int] = None) -> None:
        """Enqueues the barrier on the current stream, or on the raw ``cudaStream_t`` handle given."""
        self.epoch += 1
        nv.check(nv.cuda().cvb_symm_barrier(self._ptrs, self.heap.index, self.heap.world, self.epoch, self._status,
                                            nv.stream() if stream is None else stream), "cvb_symm_barrier")
        count_launch()


class FusedZeroComm:
    """Symmetric-memory ZeRO communication for ``FlatZeroOptimizer``.

    ``param_flat`` / ``grad_flat`` are this rank's tensors that live in symmetric buffers
    (``allocator`` creates them for ``FlatParams``); peers are addressed through the pointer tables.
    """

    def __init__(self, heap: SymmetricHeap):
        self.heap = heap
        self.n = 0
        self.params = self.grads = None
        self.param_flat = self.grad_flat = None
        self.barrier = SymmBarrier(heap)
        self.sq = torch.zeros(1, dtype=torch.float32, device=heap.device)

    def allocator(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """Hook for ``FlatParams`` (collective over the group): the bf16 parameter buffer on the first
        call, the fp32 gradient buffer on the second."""
        if self.params is None:
            if dtype != torch.bfloat16:
                raise TypeError("the fused ZeRO path keeps model parameters in bf16")
            self.n = numel
            self.params = self.heap.alloc(numel * 2)
            self.param_flat = self.params.tensor(numel, torch.bfloat16)
            return self.param_flat
        if self.grads is None and dtype == torch.float32 and numel == self.n:
            self.grads = self.heap.alloc(numel * 4)
            self.grad_flat = self.grads.tensor(numel, torch.float32)
            return self.grad_flat
        raise ValueError("FusedZeroComm.allocator: unexpected request")

    def reduce_scatter_mean_sumsq(self, out_shard: torch.Tensor, begin: int) -> torch.Tensor:
        """out_shard = mean over ranks of grad[begin : begin+len]; returns the shard's squared norm (1 float)."""
        self.barrier()                      # every rank's backward has finished writing its gradients
        self.sq.zero_()
        n = out_shard.numel()
        nv.check(nv.cuda().cvb_reduce_scatter_sumsq(self.grads.ptr_array(), self.heap.world, self.heap.index, begin, n,
                                                    1.0 / self.heap.world, out_shard.data_ptr(), self.sq.data_ptr(),
                                                    nv.stream()), "cvb_reduce_scatter_sumsq")
        count_launch()
        self.barrier()                      # every peer has finished reading this rank's gradients
        self.grad_flat.zero_()
        return self.sq

    def adamw_allgather(self, adam, grad_shard: torch.Tensor, clip: Optional[torch.Tensor], begin: int) -> None:
        o = adam.options
        adam.step_count += 1
        nv.check(nv.cuda().cvb_flat_adamw_allgather(grad_shard.data_ptr(), nv.ptr(adam.master), adam.exp_avg.data_ptr(),
                                                    adam.exp_avg_sq.data_ptr(), nv.ptr(clip), self.params.ptr_array(),
                                                    self.heap.world, self.heap.index, begin, grad_shard.numel(), o.lr,
                                                    o.beta1, o.beta2, o.eps, o.weight_decay, adam.step_count,
                                                    nv.stream()), "cvb_flat_adamw_allgather")
        count_launch()
        self.barrier()                      # all shards have landed everywhere before the next forward


class P2pBroadcaster:
    """Pushes a contiguous tensor from one rank into the same symmetric buffer on a set of peers."""

    def __init__(self, heap: SymmetricHeap, nbytes: int):
        self.heap = heap
        self.buf = heap.alloc(nbytes)
        self.barrier = SymmBarrier(heap)

    def tensor(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        return self.buf.tensor(numel, dtype)

    def push(self, src: torch.Tensor, dst_indices: Sequence[int]) -> None:
        """Called on the sending rank: stores ``src`` into every destination's buffer."""
        nbytes = src.numel() * src.element_size()
        ptrs = (C.c_void_p * len(dst_indices))(*[self.buf.peer_ptrs[i] for i in dst_indices])
        nv.check(nv.cuda().cvb_broadcast_store(src.data_ptr(), ptrs, len(dst_indices), nbytes, nv.stream()),
                 "cvb_broadcast_store")
        count_launch()

    def sync(self) -> None:
        """Group barrier on the stream: after it the pushed bytes are visible on the receivers."""
        self.barrier()
