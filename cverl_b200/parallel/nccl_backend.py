"""``NcclCollectives``: the framework's own NCCL backend behind the ``Collectives`` interface.

One native communicator (``nccl/nccl_backend.cc``) per instance, with a dedicated non-blocking CUDA
stream (taken from torch's stream pool and lent to the native layer); rendezvous through a file that holds the NCCL unique id, so that processes started by
any launcher - or by none - can form a communicator (the reference:
src/distributed/nccl_collectives.cc:156-196).  Two completion modes, as in the reference
(:278-312): ``sync_after_op=True`` waits on the host after every operation; the default async mode
makes the caller's current stream wait for the operation through an event and returns at once.
In async mode the tensors must outlive the operation on the communicator's stream; instead of the
reference's keep-alive list they are registered with the caching allocator
(``Tensor.record_stream``), which then will not hand their memory out again before that stream has
passed them.

Sub-groups are ``ncclCommSplit`` children created on first use of a rank list (collective over the
parent, like ``TorchDistCollectives.pg``) and cached.  Mean is a sum followed by a division,
gather / scatter / all-to-all work on dim 0, ``send_recv`` is one grouped send + receive.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Optional, Sequence, Tuple

import torch

from .collectives import Collectives, ReduceOp

_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.int32: 3, torch.int64: 4, torch.uint8: 5}
_OPS = {ReduceOp.SUM: 0, ReduceOp.MEAN: 0, ReduceOp.MAX: 1, ReduceOp.MIN: 2}
_lib = None


def library():
    """The native communicator library (needs ``libnccl.so.2`` and a CUDA runtime at load time)."""
    global _lib
    if _lib is None:
        from .. import _build
        path = _build.NCCL_LIB
        if not path.exists():
            _build.build_nccl()
        if not path.exists():
            raise RuntimeError("libcverl_nccl.so is not built: nccl.h / libnccl.so.2 were not found")
        lib = C.CDLL(str(path))
        lib.cvn_last_error.restype = C.c_char_p
        lib.cvn_comm_create.restype = C.c_void_p
        lib.cvn_comm_create.argtypes = [C.c_int, C.c_int, C.c_int, C.c_char_p, C.c_int, C.c_void_p]
        lib.cvn_comm_split.restype = C.c_void_p
        lib.cvn_comm_split.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        lib.cvn_comm_destroy.argtypes = [C.c_void_p]
        lib.cvn_comm_stream.restype = C.c_void_p
        lib.cvn_comm_stream.argtypes = [C.c_void_p]
        lib.cvn_unique_id_create.argtypes = [C.c_char_p]
        lib.cvn_unique_id_write_file.argtypes = [C.c_char_p, C.c_char_p]
        lib.cvn_unique_id_read_file.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.c_int]
        p, ll, i = C.c_void_p, C.c_longlong, C.c_int
        lib.cvn_all_reduce.argtypes = [p, p, p, ll, i, i, p]
        lib.cvn_broadcast.argtypes = [p, p, p, ll, i, i, p]
        lib.cvn_all_gather.argtypes = [p, p, p, ll, i, p]
        lib.cvn_reduce_scatter.argtypes = [p, p, p, ll, i, i, p]
        lib.cvn_all_to_all.argtypes = [p, p, p, ll, i, p]
        lib.cvn_send.argtypes = [p, p, ll, i, i, p]
        lib.cvn_recv.argtypes = [p, p, ll, i, i, p]
        lib.cvn_send_recv.argtypes = [p, p, ll, i, p, ll, i, i, p]
        lib.cvn_barrier.argtypes = [p, p, p]
        _lib = lib
    return _lib


def create_unique_id() -> bytes:
    lib = library()
    buf = C.create_string_buffer(lib.cvn_unique_id_bytes())
    if lib.cvn_unique_id_create(buf) != 0:
        raise RuntimeError(lib.cvn_last_error().decode())
    return buf.raw


def write_unique_id_file(path: str, unique_id: bytes) -> None:
    lib = library()
    if lib.cvn_unique_id_write_file(os.fsencode(path), unique_id) != 0:
        raise RuntimeError(lib.cvn_last_error().decode())


def read_unique_id_file(path: str, timeout_s: float = 5.0, poll_ms: int = 25) -> bytes:
    lib = library()
    buf = C.create_string_buffer(lib.cvn_unique_id_bytes())
    polls = max(1, int(timeout_s * 1000 / poll_ms))
    if lib.cvn_unique_id_read_file(os.fsencode(path), buf, polls, poll_ms) != 0:
        raise TimeoutError(lib.cvn_last_error().decode())
    return buf.raw


class NcclCollectives(Collectives):
    def __init__(self, rank: int, world_size: int, device, unique_id: Optional[bytes] = None,
                 id_file: Optional[str] = None, sync_after_op: bool = False, id_timeout_s: float = 5.0,
                 _handle=None, _global_ranks: Optional[Sequence[int]] = None, _stream=None):
        """``unique_id`` (bytes from ``create_unique_id`` of rank 0) or ``id_file``: rank 0 creates the id and
        writes the file, the others poll for it."""
        self._lib = library()
        self.device = torch.device(device)
        self._rank, self._world = rank, world_size
        self._root_world = world_size          # a split child reports its parent's world through the interface
        self._sync = sync_after_op
        self._global_ranks = list(_global_ranks) if _global_ranks is not None else list(range(world_size))
        self._children: Dict[Tuple[int, ...], Optional["NcclCollectives"]] = {}
        # The communicator's stream comes from torch's pool and is lent to the native layer: the caching
        # allocator records events on it when a tensor registered by ``record_stream`` is freed, which may be
        # after ``close()``, so the stream must never be destroyed.
        self._stream = _stream if _stream is not None else torch.cuda.Stream(device=self.device)
        if _handle is not None:
            self._h = _handle
        else:
            if unique_id is None:
                if id_file is None:
                    raise ValueError("NcclCollectives needs a unique id or an id file")
                if rank == 0:
                    unique_id = create_unique_id()
                    write_unique_id_file(id_file, unique_id)
                else:
                    unique_id = read_unique_id_file(id_file, id_timeout_s)
            idx = self.device.index if self.device.index is not None else torch.cuda.current_device()
            self._h = self._lib.cvn_comm_create(rank, world_size, idx, unique_id, int(sync_after_op),
                                                self._stream.cuda_stream)
            if not self._h:
                raise RuntimeError("NCCL communicator: " + self._lib.cvn_last_error().decode())
        self._scratch = torch.zeros(1, dtype=torch.float32, device=self.device)

    # ---- interface ----------------------------------------------------------------------------------------
    def rank(self) -> int:
        return self._global_ranks[self._rank]

    def world_size(self) -> int:
        return self._root_world

    def close(self) -> None:
        for child in self._children.values():
            if child is not None:
                child.close()
        self._children = {}
        if self._h:
            self._lib.cvn_comm_destroy(self._h)
            self._h = None

    # ---- helpers ------------------------------------------------------------------------------------------
    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise RuntimeError(f"{what}: {self._lib.cvn_last_error().decode()}")

    def _caller(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _keep(self, *tensors: torch.Tensor) -> None:
        if not self._sync:
            for t in tensors:
                t.record_stream(self._stream)

    @staticmethod
    def _contig(t: torch.Tensor) -> torch.Tensor:
        if not t.is_contiguous():
            raise ValueError("collectives require contiguous tensors")
        if t.dtype not in _DTYPES:
            raise TypeError(f"NcclCollectives does not move {t.dtype}")
        return t

    def _comm_for(self, group: Optional[Sequence[int]]) -> "NcclCollectives":
        """The communicator of a list of GLOBAL ranks: this one, or a cached ``ncclCommSplit`` child.  Creating a
        child is collective over this communicator: every rank must ask for the same groups in the same order
        (ranks outside the group take part in the split and get no child)."""
        if group is None:
            return self
        ranks = tuple(int(r) for r in group)
        if ranks == tuple(self._global_ranks):
            return self
        if ranks in self._children:
            child = self._children[ranks]
        else:
            me = self._global_ranks[self._rank]
            color, key = -1, 0
            if me in ranks:
                h = 2166136261                        # FNV-1a over the rank list: members agree on the colour
                for r in ranks:
                    h = ((h ^ (r & 0xFFFFFFFF)) * 16777619) & 0x7FFFFFFF
                color, key = h, ranks.index(me)
            stream = torch.cuda.Stream(device=self.device) if color >= 0 else None
            handle = self._lib.cvn_comm_split(self._h, color, key, len(ranks),
                                              stream.cuda_stream if stream is not None else None)
            child = None
            if color >= 0:
                if not handle:
                    raise RuntimeError("ncclCommSplit: " + self._lib.cvn_last_error().decode())
                child = NcclCollectives(key, len(ranks), self.device, sync_after_op=self._sync, _handle=handle,
                                        _global_ranks=ranks, _stream=stream)
                child._root_world = self.world_size()
            self._children[ranks] = child
        if child is None:
            raise ValueError(f"rank {self.rank()} is not a member of group {list(ranks)}")
        return child

    def ensure_group(self, group: Sequence[int]) -> None:
        """Take part in the creation of ``group``'s communicator (members and non-members alike)."""
        try:
            self._comm_for(group)
        except ValueError:
            pass

    # ---- collectives ----------------------------------------------------------------------------------------
    def barrier(self, group=None) -> None:
        c = self._comm_for(group)
        c._check(c._lib.cvn_barrier(c._h, c._scratch.data_ptr(), c._caller()), "barrier")

    def broadcast(self, tensor, root, group=None):
        c = self._comm_for(group)
        t = self._contig(tensor)
        out = torch.empty_like(t)
        idx = c._global_ranks.index(root) if root in c._global_ranks else -1
        if idx < 0:
            raise ValueError(f"broadcast root {root} is not in the group")
        c._check(c._lib.cvn_broadcast(c._h, t.data_ptr(), out.data_ptr(), t.numel(), _DTYPES[t.dtype], idx,
                                      c._caller()), "broadcast")
        c._keep(t, out)
        return out

    def all_reduce(self, tensor, op=ReduceOp.SUM, group=None):
        c = self._comm_for(group)
        t = self._contig(tensor)
        out = torch.empty_like(t)
        c._check(c._lib.cvn_all_reduce(c._h, t.data_ptr(), out.data_ptr(), t.numel(), _DTYPES[t.dtype], _OPS[op],
                                       c._caller()), "all_reduce")
        c._keep(t, out)
        if op == ReduceOp.MEAN:
            out.div_(c._world)
        return out

    def all_gather(self, tensor, group=None):
        c = self._comm_for(group)
        t = self._contig(tensor)
        out = t.new_empty((c._world * t.shape[0],) + tuple(t.shape[1:]))
        c._check(c._lib.cvn_all_gather(c._h, t.data_ptr(), out.data_ptr(), t.numel(), _DTYPES[t.dtype], c._caller()),
                 "all_gather")
        c._keep(t, out)
        return out

    def reduce_scatter(self, tensor, op=ReduceOp.SUM, group=None):
        c = self._comm_for(group)
        t = self._contig(tensor)
        if t.shape[0] % c._world:
            raise ValueError("reduce_scatter needs dim 0 divisible by the group size")
        out = t.new_empty((t.shape[0] // c._world,) + tuple(t.shape[1:]))
        c._check(c._lib.cvn_reduce_scatter(c._h, t.data_ptr(), out.data_ptr(), out.numel(), _DTYPES[t.dtype], _OPS[op],
                                           c._caller()), "reduce_scatter")
        c._keep(t, out)
        if op == ReduceOp.MEAN:
            out.div_(c._world)
        return out

    def all_to_all(self, tensor, group=None):
        c = self._comm_for(group)
        t = self._contig(tensor)
        if t.shape[0] % c._world:
            raise ValueError("all_to_all needs dim 0 divisible by the group size")
        out = torch.empty_like(t)
        c._check(c._lib.cvn_all_to_all(c._h, t.data_ptr(), out.data_ptr(), t.numel() // c._world, _DTYPES[t.dtype],
                                       c._caller()), "all_to_all")
        c._keep(t, out)
        return out

    def _peer(self, global_rank: int) -> int:
        if global_rank not in self._global_ranks:
            raise ValueError(f"rank {global_rank} is not in this communicator")
        return self._global_ranks.index(global_rank)

    def send(self, tensor, dst) -> None:
        t = self._contig(tensor)
        self._check(self._lib.cvn_send(self._h, t.data_ptr(), t.numel(), _DTYPES[t.dtype], self._peer(dst),
                                       self._caller()), "send")
        self._keep(t)

    def recv_like(self, like, src):
        out = torch.empty_like(like, device=self.device)
        self._contig(out)
        self._check(self._lib.cvn_recv(self._h, out.data_ptr(), out.numel(), _DTYPES[out.dtype], self._peer(src),
                                       self._caller()), "recv")
        self._keep(out)
        return out

    def send_recv(self, send_tensor, dst, recv_like, src):
        t = self._contig(send_tensor)
        out = torch.empty_like(recv_like, device=self.device)
        if t.dtype != out.dtype:
            raise TypeError("send_recv moves one dtype per call")
        self._check(self._lib.cvn_send_recv(self._h, t.data_ptr(), t.numel(), self._peer(dst), out.data_ptr(),
                                            out.numel(), self._peer(src), _DTYPES[t.dtype], self._caller()),
                    "send_recv")
        self._keep(t, out)
        return out
