"""Trainer -> rollout weight synchronisation.

``broadcast_parameters_from_root`` copies a list of ``ParameterView{name, tensor}`` from a
root rank to every rank of a group, in place, in buckets (25 MB by default) that never mix
dtypes or devices; a bucket of one tensor is sent without the flatten copy; one optional
barrier closes the sync.  ``send_parameter_shards`` / ``recv_parameter_shards`` move the
same buckets point to point.  Semantics follow the reference
(src/distributed/weight_sync.cc:56-272).  On a single NVSwitch node the fast path is
``cverl_b200.parallel.symm.P2pBroadcaster`` (one kernel whose stores land in every receiver's
peer-mapped copy, one pass over the weights); this module is the portable path over any
``Collectives`` backend.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .collectives import Collectives

DEFAULT_BUCKET_BYTES = 25 * 1024 * 1024


@dataclass
class ParameterView:
    name: str
    tensor: torch.Tensor


@dataclass
class WeightSyncStats:
    buckets: int = 0
    tensors: int = 0
    bytes: int = 0
    barriers: int = 0


def module_parameter_views(module: torch.nn.Module) -> List[ParameterView]:
    return [ParameterView(n, p.data) for n, p in module.named_parameters()]


def _buckets(params: Sequence[ParameterView], bucket_bytes: int) -> List[List[ParameterView]]:
    out: List[List[ParameterView]] = []
    cur: List[ParameterView] = []
    cur_bytes = 0
    for pv in params:
        t = pv.tensor
        nbytes = t.numel() * t.element_size()
        split = cur and (t.dtype != cur[0].tensor.dtype or t.device != cur[0].tensor.device
                         or cur_bytes + nbytes > bucket_bytes)
        if split:
            out.append(cur)
            cur, cur_bytes = [], 0
        cur.append(pv)
        cur_bytes += nbytes
    if cur:
        out.append(cur)
    return out


def _flatten(bucket: List[ParameterView]) -> torch.Tensor:
    if len(bucket) == 1 and bucket[0].tensor.is_contiguous():
        return bucket[0].tensor.view(-1)
    return torch.cat([pv.tensor.reshape(-1) for pv in bucket])


def _scatter_back(bucket: List[ParameterView], flat: torch.Tensor) -> None:
    off = 0
    with torch.no_grad():
        for pv in bucket:
            n = pv.tensor.numel()
            pv.tensor.copy_(flat[off:off + n].view_as(pv.tensor))
            off += n


def broadcast_parameters_from_root(params: Sequence[ParameterView], comm: Collectives, root: int,
                                   group: Optional[Sequence[int]] = None,
                                   bucket_bytes: int = DEFAULT_BUCKET_BYTES, barrier: bool = True) -> WeightSyncStats:
    g = list(range(comm.world_size())) if group is None else list(group)
    if root not in g:
        raise ValueError("broadcast root must be a member of the group")
    stats = WeightSyncStats()
    if len(g) == 1:
        Collectives.rank_index_in_group(comm.rank(), g, "weight-sync group")
        return stats
    if bucket_bytes <= 0:
        raise ValueError("bucket_bytes must be positive")
    for bucket in _buckets(params, bucket_bytes):
        flat = _flatten(bucket)
        out = comm.broadcast(flat, root, g)
        if comm.rank() != root:
            _scatter_back(bucket, out)
        stats.buckets += 1
        stats.tensors += len(bucket)
        stats.bytes += flat.numel() * flat.element_size()
    if barrier:
        comm.barrier(g)
        stats.barriers += 1
    return stats


def send_parameter_shards(params: Sequence[ParameterView], comm: Collectives, dst: int,
                          bucket_bytes: int = DEFAULT_BUCKET_BYTES) -> WeightSyncStats:
    stats = WeightSyncStats()
    for bucket in _buckets(params, bucket_bytes):
        flat = _flatten(bucket).contiguous()
        comm.send(flat, dst)
        stats.buckets += 1
        stats.tensors += len(bucket)
        stats.bytes += flat.numel() * flat.element_size()
    return stats


def recv_parameter_shards(params: Sequence[ParameterView], comm: Collectives, src: int,
                          bucket_bytes: int = DEFAULT_BUCKET_BYTES) -> WeightSyncStats:
    stats = WeightSyncStats()
    for bucket in _buckets(params, bucket_bytes):
        like = _flatten(bucket)
        got = comm.recv_like(like, src)
        _scatter_back(bucket, got)
        stats.buckets += 1
        stats.tensors += len(bucket)
        stats.bytes += like.numel() * like.element_size()
    return stats


class PeerMemoryWeightPush:
    """Trainer -> rollout weight push by this package's own kernels instead of library send / recv.

    ``mode="symm"``: every trainer stores the flattened parameters into the peer-mapped receive buffer of each
    rollout rank it serves (``cvb_broadcast_store``: one read, one store per destination, plain NVLink stores).
    ``mode="nvls"``: the trainers hold identical weights after their gradient all-reduce, so trainer t multicasts
    slice t of the flat buffer through the NVSwitch multicast address (``multimem.st``) and every rank's buffer
    ends up with all of it, each sender's links carrying 1 / T of the weights once.
    Both end with a flag barrier over all ranks; the rollout ranks then copy the buffer into their parameters.
    All parameters must share one dtype.  Collective constructor over the default group.
    (Reference: ncclBroadcast / send-recv per bucket, src/distributed/weight_sync.cc:86-189.)"""

    def __init__(self, params: Sequence[ParameterView], device, trainers: int, world: int, mode: str = "symm"):
        import torch.distributed as dist
        self.params = list(params)
        dt = {pv.tensor.dtype for pv in self.params}
        if len(dt) != 1:
            raise ValueError("PeerMemoryWeightPush needs parameters of one dtype")
        self.dtype = dt.pop()
        self.numel = sum(pv.tensor.numel() for pv in self.params)
        esz = torch.empty((), dtype=self.dtype).element_size()
        self.nbytes = (self.numel * esz + 255) // 256 * 256
        self.trainers, self.world, self.mode = trainers, world, mode
        if mode == "symm":
            from .symm import P2pBroadcaster, SymmetricHeap
            self.bc = P2pBroadcaster(SymmetricHeap(dist.group.WORLD, device), self.nbytes)
        elif mode == "nvls":
            from .nvls import NvlsBroadcaster
            self.bc = NvlsBroadcaster(dist.group.WORLD, device, self.nbytes)
        else:
            raise ValueError("mode must be symm or nvls")
        self.recv = self.bc.tensor(self.numel, self.dtype)

    def push(self, rank: int, my_rollouts: Sequence[int]) -> None:
        """Called by every rank once per weight version (trainers send, everyone synchronises, rollout ranks load)."""
        if rank < self.trainers:
            flat = _flatten(self.params)
            padded = (self.numel + 7) // 8 * 8               # whole 16-byte pieces for every dtype of 2+ bytes
            if padded != self.numel:
                flat = torch.nn.functional.pad(flat, (0, padded - self.numel))
            if self.mode == "symm":
                if my_rollouts:
                    self.bc.push(flat, list(my_rollouts))
            else:
                per = (padded // self.trainers + 7) // 8 * 8
                lo = min(rank * per, padded)
                hi = padded if rank == self.trainers - 1 else min(lo + per, padded)
                if hi > lo:
                    self.bc.push(flat[lo:hi], lo * flat.element_size())
        self.bc.sync()
        if rank >= self.trainers:
            _scatter_back(self.params, self.recv)
