"""Communication backends behind one tensor-in / tensor-out interface.

``Collectives`` mirrors the reference's abstract class
(include/cverl/distributed/collectives.h:10-31): a group is a list of GLOBAL
ranks, every call returns a fresh tensor, gather/scatter work on dim 0.

* ``SingleProcessCollectives`` - world of one, identity semantics, for CPU tests
  (src/distributed/collectives.cc:24-85).
* ``TorchDistCollectives`` - ``torch.distributed`` process groups (NCCL on GPUs,
  gloo on CPU); sub-groups are created once per rank list and cached, Mean is a
  sum followed by a division, all-to-all is dim-0 equal split
  (src/distributed/nccl_collectives.cc:252-276,355-357,405-441).
* the in-kernel NVLink paths live in ``cverl_b200.parallel.symm`` and are used
  by the fused ops directly; they are not generic collectives.
"""
from __future__ import annotations

import abc
import enum
from typing import Dict, List, Optional, Sequence, Tuple

import torch


class ReduceOp(enum.Enum):
    SUM = "sum"
    MEAN = "mean"
    MAX = "max"
    MIN = "min"


class Collectives(abc.ABC):
    @abc.abstractmethod
    def rank(self) -> int: ...

    @abc.abstractmethod
    def world_size(self) -> int: ...

    @abc.abstractmethod
    def barrier(self, group: Optional[Sequence[int]] = None) -> None: ...

    @abc.abstractmethod
    def broadcast(self, tensor: torch.Tensor, root: int, group: Optional[Sequence[int]] = None) -> torch.Tensor: ...

    @abc.abstractmethod
    def all_reduce(self, tensor: torch.Tensor, op: ReduceOp = ReduceOp.SUM,
                   group: Optional[Sequence[int]] = None) -> torch.Tensor: ...

    @abc.abstractmethod
    def all_gather(self, tensor: torch.Tensor, group: Optional[Sequence[int]] = None) -> torch.Tensor: ...

    @abc.abstractmethod
    def reduce_scatter(self, tensor: torch.Tensor, op: ReduceOp = ReduceOp.SUM,
                       group: Optional[Sequence[int]] = None) -> torch.Tensor: ...

    @abc.abstractmethod
    def all_to_all(self, tensor: torch.Tensor, group: Optional[Sequence[int]] = None) -> torch.Tensor: ...

    @abc.abstractmethod
    def send(self, tensor: torch.Tensor, dst: int) -> None: ...

    @abc.abstractmethod
    def recv_like(self, like: torch.Tensor, src: int) -> torch.Tensor: ...

    def send_recv(self, send_tensor: torch.Tensor, dst: int, recv_like: torch.Tensor, src: int) -> torch.Tensor:
        """Default: send, then receive (backends may group the pair)."""
        self.send(send_tensor, dst)
        return self.recv_like(recv_like, src)

    # helpers -------------------------------------------------------------
    def _group(self, group: Optional[Sequence[int]]) -> List[int]:
        return list(range(self.world_size())) if group is None else [int(g) for g in group]

    @staticmethod
    def rank_index_in_group(rank: int, group: Sequence[int], what: str = "group") -> int:
        try:
            return list(group).index(rank)
        except ValueError as exc:
            raise ValueError(f"rank {rank} is not a member of {what} {list(group)}") from exc


class SingleProcessCollectives(Collectives):
    """World of one: every collective is the identity on a copy."""

    def rank(self) -> int:
        return 0

    def world_size(self) -> int:
        return 1

    def _check(self, group):
        g = self._group(group)
        if g != [0]:
            raise ValueError("SingleProcessCollectives only supports the group [0]")

    def barrier(self, group=None) -> None:
        self._check(group)

    def broadcast(self, tensor, root, group=None):
        self._check(group)
        if root != 0:
            raise ValueError("broadcast root must be 0 in a single-process world")
        return tensor.clone()

    def all_reduce(self, tensor, op=ReduceOp.SUM, group=None):
        self._check(group)
        return tensor.clone()

    def all_gather(self, tensor, group=None):
        self._check(group)
        return tensor.clone()

    def reduce_scatter(self, tensor, op=ReduceOp.SUM, group=None):
        self._check(group)
        return tensor.clone()

    def all_to_all(self, tensor, group=None):
        self._check(group)
        return tensor.clone()

    def send(self, tensor, dst) -> None:
        raise RuntimeError("send is undefined in a single-process world")

    def recv_like(self, like, src):
        raise RuntimeError("recv is undefined in a single-process world")


class TorchDistCollectives(Collectives):
    """``torch.distributed`` backend: NCCL over NVLink on GPUs, gloo on CPU."""

    def __init__(self, timeout_s: Optional[float] = None):
        import torch.distributed as dist
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self._dist = dist
        self._groups: Dict[Tuple[int, ...], object] = {}
        self._timeout_s = timeout_s

    def rank(self) -> int:
        return self._dist.get_rank()

    def world_size(self) -> int:
        return self._dist.get_world_size()

    def pg(self, group: Optional[Sequence[int]]):
        """Process group of a rank list (created collectively on first use, then cached).

        Like ``ncclCommSplit`` in the reference, creation is collective over the
        WORLD: every rank must request the same groups in the same order.
        """
        ranks = tuple(self._group(group))
        if ranks == tuple(range(self.world_size())):
            return None
        pg = self._groups.get(ranks)
        if pg is None:
            kw = {}
            if self._timeout_s is not None:
                import datetime
                kw["timeout"] = datetime.timedelta(seconds=self._timeout_s)
            pg = self._dist.new_group(list(ranks), **kw)
            self._groups[ranks] = pg
        return pg

    def _member_pg(self, group: Optional[Sequence[int]]):
        """The group's process group for a collective CALL: a rank outside the group is refused (creation through
        ``pg`` stays open to every rank, because it is collective over the world)."""
        if group is not None:
            self.rank_index_in_group(self.rank(), self._group(group), "collective group")
        return self.pg(group)

    def register_group(self, ranks: Sequence[int], pg) -> None:
        self._groups[tuple(int(r) for r in ranks)] = pg

    def barrier(self, group=None) -> None:
        t = torch.zeros(1, device=self._device())
        self._dist.all_reduce(t, group=self._member_pg(group))
        if t.is_cuda:
            torch.cuda.current_stream().synchronize()

    def _device(self):
        if self._dist.get_backend() == "nccl":
            return torch.device("cuda", torch.cuda.current_device())
        return torch.device("cpu")

    @staticmethod
    def _contig(t: torch.Tensor) -> torch.Tensor:
        if not t.is_contiguous():
            raise ValueError("collectives require contiguous tensors")
        return t

    def _op(self, op: ReduceOp):
        d = self._dist
        return {ReduceOp.SUM: d.ReduceOp.SUM, ReduceOp.MEAN: d.ReduceOp.SUM, ReduceOp.MAX: d.ReduceOp.MAX,
                ReduceOp.MIN: d.ReduceOp.MIN}[op]

    def broadcast(self, tensor, root, group=None):
        g = self._group(group)
        self.rank_index_in_group(root, g, "broadcast group")
        out = self._contig(tensor).clone()
        self._dist.broadcast(out, src=root, group=self._member_pg(group))
        return out

    def all_reduce(self, tensor, op=ReduceOp.SUM, group=None):
        out = self._contig(tensor).clone()
        self._dist.all_reduce(out, op=self._op(op), group=self._member_pg(group))
        if op == ReduceOp.MEAN:
            out.div_(len(self._group(group)))
        return out

    def all_gather(self, tensor, group=None):
        n = len(self._group(group))
        t = self._contig(tensor)
        out = t.new_empty((n * t.shape[0],) + tuple(t.shape[1:]))
        self._dist.all_gather_into_tensor(out, t, group=self._member_pg(group))
        return out

    def reduce_scatter(self, tensor, op=ReduceOp.SUM, group=None):
        n = len(self._group(group))
        t = self._contig(tensor)
        if t.shape[0] % n:
            raise ValueError("reduce_scatter: dim 0 must divide by the group size")
        out = t.new_empty((t.shape[0] // n,) + tuple(t.shape[1:]))
        if t.is_cuda:
            self._dist.reduce_scatter_tensor(out, t, op=self._op(op), group=self._member_pg(group))
        else:  # gloo has no reduce_scatter: all-reduce and slice
            full = t.clone()
            self._dist.all_reduce(full, op=self._op(op), group=self._member_pg(group))
            idx = self.rank_index_in_group(self.rank(), self._group(group))
            out.copy_(full.narrow(0, idx * out.shape[0], out.shape[0]))
        if op == ReduceOp.MEAN:
            out.div_(n)
        return out

    def all_to_all(self, tensor, group=None):
        n = len(self._group(group))
        t = self._contig(tensor)
        if t.shape[0] % n:
            raise ValueError("all_to_all: dim 0 must divide by the group size")
        out = torch.empty_like(t)
        if t.is_cuda:
            self._dist.all_to_all_single(out, t, group=self._member_pg(group))
        else:
            # gloo has no all-to-all: every rank gathers every rank's tensor and keeps the chunk addressed to it
            g = self._group(group)
            me = self.rank_index_in_group(self.rank(), g, "all_to_all group")
            parts = [torch.empty_like(t) for _ in range(n)]
            self._dist.all_gather(parts, t, group=self._member_pg(group))
            torch.cat([p.chunk(n, 0)[me] for p in parts], 0, out=out)
        return out

    def send(self, tensor, dst) -> None:
        self._dist.send(self._contig(tensor), dst=dst)

    def recv_like(self, like, src):
        out = torch.empty_like(like)
        self._dist.recv(out, src=src)
        return out

    def send_recv(self, send_tensor, dst, recv_like, src):
        out = torch.empty_like(recv_like)
        ops = [self._dist.P2POp(self._dist.isend, self._contig(send_tensor), dst),
               self._dist.P2POp(self._dist.irecv, out, src)]
        for req in self._dist.batch_isend_irecv(ops):
            req.wait()
        return out
