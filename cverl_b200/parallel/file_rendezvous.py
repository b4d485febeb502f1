"""An independent communicator whose members meet through a file, not through the launcher.

The reference opens every communicator from an id file: one rank writes the NCCL unique id
atomically, the others poll for it (src/distributed/nccl_collectives.cc:156-196), which lets
processes that were started separately - a rollout source and the trainer ranks - form a world
of their own beside the trainer's (tools/model/qwen3_5_pp_tp_ppo_trainer.cc:2064-2080).

``FileRendezvousCollectives`` is that: a ``Collectives`` backend over a process group built
directly on a ``torch.distributed.FileStore`` at ``path`` (NCCL on CUDA devices, gloo on the
CPU).  It needs no default process group, so a process may hold it next to the ``torchrun``
world, and ranks may be numbered with an offset.  Groups are always the whole communicator.
"""
from __future__ import annotations

import datetime
from typing import Optional, Sequence

import torch

from .collectives import Collectives, ReduceOp


class FileRendezvousCollectives(Collectives):
    def __init__(self, path: str, rank: int, world_size: int, device="cpu", timeout_s: float = 60.0):
        import torch.distributed as dist
        if not (0 <= rank < world_size):
            raise ValueError("rank out of range for the file-rendezvous communicator")
        self._dist = dist
        self._rank, self._world = rank, world_size
        self.device = torch.device(device)
        self._store = dist.FileStore(path, world_size)
        timeout = datetime.timedelta(seconds=timeout_s)
        if self.device.type == "cuda":
            opts = dist.ProcessGroupNCCL.Options()
            opts._timeout = timeout
            torch.cuda.set_device(self.device)
            self._pg = dist.ProcessGroupNCCL(self._store, rank, world_size, opts)
        else:
            self._pg = dist.ProcessGroupGloo(self._store, rank, world_size, timeout)

    def rank(self) -> int:
        return self._rank

    def world_size(self) -> int:
        return self._world

    def _whole(self, group: Optional[Sequence[int]]) -> None:
        if group is not None and list(group) != list(range(self._world)):
            raise ValueError("a file-rendezvous communicator has no sub-groups")

    def _wait(self, work) -> None:
        work.wait()

    def barrier(self, group=None) -> None:
        self._whole(group)
        t = torch.zeros(1, device=self.device)
        self._wait(self._pg.allreduce([t]))
        if t.is_cuda:
            torch.cuda.current_stream().synchronize()

    def broadcast(self, tensor, root, group=None):
        self._whole(group)
        out = tensor.contiguous().clone()
        opts = self._dist.BroadcastOptions()
        opts.rootRank = root
        self._wait(self._pg.broadcast([out], opts))
        return out

    def all_reduce(self, tensor, op=ReduceOp.SUM, group=None):
        self._whole(group)
        out = tensor.contiguous().clone()
        opts = self._dist.AllreduceOptions()
        d = self._dist.ReduceOp
        opts.reduceOp = {ReduceOp.SUM: d.SUM, ReduceOp.MEAN: d.SUM, ReduceOp.MAX: d.MAX, ReduceOp.MIN: d.MIN}[op]
        self._wait(self._pg.allreduce([out], opts))
        if op == ReduceOp.MEAN:
            out.div_(self._world)
        return out

    def all_gather(self, tensor, group=None):
        self._whole(group)
        t = tensor.contiguous()
        parts = [torch.empty_like(t) for _ in range(self._world)]
        self._wait(self._pg.allgather([parts], [t]))
        return torch.cat(parts, 0)

    def reduce_scatter(self, tensor, op=ReduceOp.SUM, group=None):
        self._whole(group)
        if tensor.shape[0] % self._world:
            raise ValueError("reduce_scatter needs dim 0 divisible by the world size")
        full = self.all_reduce(tensor, op, None)
        n = tensor.shape[0] // self._world
        return full[self._rank * n:(self._rank + 1) * n].clone()

    def all_to_all(self, tensor, group=None):
        self._whole(group)
        if tensor.shape[0] % self._world:
            raise ValueError("all_to_all needs dim 0 divisible by the world size")
        chunks = list(tensor.contiguous().chunk(self._world, 0))
        out = [torch.empty_like(c) for c in chunks]
        out[self._rank].copy_(chunks[self._rank])
        for peer in range(self._world):
            if peer == self._rank:
                continue
            if self._rank < peer:
                self.send(chunks[peer], peer)
                out[peer] = self.recv_like(out[peer], peer)
            else:
                out[peer] = self.recv_like(out[peer], peer)
                self.send(chunks[peer], peer)
        return torch.cat(out, 0)

    def send(self, tensor, dst) -> None:
        self._wait(self._pg.send([tensor.contiguous()], dst, 0))

    def recv_like(self, like, src):
        out = torch.empty_like(like)
        self._wait(self._pg.recv([out], src, 0))
        return out

    def close(self) -> None:
        self._pg = None
        self._store = None
