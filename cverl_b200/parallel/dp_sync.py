"""Data-parallel gradient synchronisation in buckets, and the per-tensor optimizer modes built on it.

Reference behaviour:
* ``data_parallel_sync_gradients`` (src/distributed/parallel_ops.cc:226-272): walk the parameters
  in order, collect gradients into buckets of at most ``bucket_bytes`` (25 MB by default) that never
  mix dtypes or devices, all-reduce each bucket (mean or sum, optionally cast to a communication
  dtype), copy the result back; a data group of one returns at once.
* ``data_parallel_reduce_scatter_gradients`` (:274-321): the same bucketing, each bucket padded to a
  multiple of the group size and reduce-scattered; the caller gets one
  ``GradientReduceScatterBucket`` per bucket.
* ZeRO-1 with per-parameter owners (src/distributed/optimizer_sharding.cc:389-434 and
  tools/model/qwen3_5_pp_tp_ppo_trainer.cc:220-240,2132-2141,2529-2536): gradients are all-reduced in
  full, every parameter has ONE owner rank (largest-first bin packing) that holds its AdamW state
  and updates it, and each owner then broadcasts its parameters in buckets.

What differs here: the framework keeps every gradient in ONE fp32 flat buffer
(``FlatParams.main_grad``), so a bucket is a contiguous slice of that buffer cut at parameter
boundaries and is reduced IN PLACE - there is no flatten copy and no copy back unless a narrower
communication dtype is asked for.  The generic functions below keep the reference's tensor-list
interface over any ``Collectives`` backend (so scripted fakes can play several ranks on a CPU);
``TensorwiseOptimizer`` is the production path over ``FlatParams`` and ``torch.distributed`` groups.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from ..optim.adamw import AdamWOptions, Fp32MasterAdamW
from ..ops import optim as optim_ops
from .collectives import Collectives, ReduceOp
from .zero import greedy_parameter_owners

DEFAULT_BUCKET_BYTES = 25 * 1024 * 1024


def _grad_of(p: torch.Tensor) -> Optional[torch.Tensor]:
    g = getattr(p, "main_grad", None)
    return g if g is not None else p.grad


def _buckets(grads: Sequence[Optional[torch.Tensor]], bucket_bytes: int,
             comm_dtype: Optional[torch.dtype]) -> List[List[int]]:
    """Indices of ``grads`` grouped into buckets: a bucket closes when the next gradient would overflow
    ``bucket_bytes`` or has another (effective) dtype or device."""
    if bucket_bytes <= 0:
        raise ValueError("bucket_bytes must be positive")
    out: List[List[int]] = []
    cur: List[int] = []
    cur_bytes, cur_key = 0, None
    for i, g in enumerate(grads):
        if g is None:
            continue
        eff = comm_dtype or g.dtype
        nbytes = g.numel() * torch.empty((), dtype=eff).element_size()
        key = (eff, g.device)
        if cur and (key != cur_key or cur_bytes + nbytes > bucket_bytes):
            out.append(cur)
            cur, cur_bytes = [], 0
        if not cur:
            cur_key = key
        cur.append(i)
        cur_bytes += nbytes
    if cur:
        out.append(cur)
    return out


def data_parallel_sync_gradients(parameters: Sequence[torch.Tensor], comm: Collectives, data_group: Sequence[int],
                                 average: bool = True, bucket_bytes: int = DEFAULT_BUCKET_BYTES,
                                 comm_dtype: Optional[torch.dtype] = None) -> int:
    """All-reduces the gradients of ``parameters`` (``.main_grad`` if present, else ``.grad``) over
    ``data_group`` in buckets, in place.  Returns the number of all-reduce calls issued."""
    Collectives.rank_index_in_group(comm.rank(), data_group, "data group")
    if bucket_bytes <= 0:
        raise ValueError("data_parallel_sync_gradients bucket_bytes must be positive")
    if len(data_group) == 1:
        return 0
    grads = [_grad_of(p) for p in parameters]
    op = ReduceOp.MEAN if average else ReduceOp.SUM
    calls = 0
    for bucket in _buckets(grads, bucket_bytes, comm_dtype):
        if len(bucket) == 1:                       # a bucket of one travels without the flatten copy
            g = grads[bucket[0]]
            flat = g.contiguous().view(-1)
            flat = flat.to(comm_dtype) if comm_dtype is not None else flat
            g.copy_(comm.all_reduce(flat, op, data_group).view_as(g))
        else:
            dt = comm_dtype or grads[bucket[0]].dtype
            flat = torch.cat([grads[i].reshape(-1).to(dt) for i in bucket])
            red = comm.all_reduce(flat, op, data_group)
            off = 0
            for i in bucket:
                n = grads[i].numel()
                grads[i].copy_(red[off:off + n].view_as(grads[i]))
                off += n
        calls += 1
    return calls


@dataclass
class GradientReduceScatterBucket:
    shard: torch.Tensor
    original_numel: int
    padded_numel: int
    parameter_indices: List[int] = field(default_factory=list)
    parameter_numels: List[int] = field(default_factory=list)


def data_parallel_reduce_scatter_gradients(parameters: Sequence[torch.Tensor], comm: Collectives,
                                           data_group: Sequence[int], average: bool = True,
                                           bucket_bytes: int = DEFAULT_BUCKET_BYTES,
                                           comm_dtype: Optional[torch.dtype] = None
                                           ) -> List[GradientReduceScatterBucket]:
    """Bucketed reduce-scatter: every bucket is zero-padded to a multiple of the group size and each rank
    keeps its slice of it."""
    Collectives.rank_index_in_group(comm.rank(), data_group, "data group")
    grads = [_grad_of(p) for p in parameters]
    op = ReduceOp.MEAN if average else ReduceOp.SUM
    n_ranks = len(data_group)
    out = []
    for bucket in _buckets(grads, bucket_bytes, comm_dtype):
        dt = comm_dtype or grads[bucket[0]].dtype
        numels = [grads[i].numel() for i in bucket]
        total = sum(numels)
        flat = torch.cat([grads[i].reshape(-1).to(dt) for i in bucket]) if len(bucket) > 1 \
            else grads[bucket[0]].reshape(-1).to(dt)
        if n_ranks == 1:
            out.append(GradientReduceScatterBucket(flat.contiguous(), total, total, list(bucket), numels))
            continue
        pad = (-total) % n_ranks
        if pad:
            flat = torch.cat([flat, flat.new_zeros(pad)])
        shard = comm.reduce_scatter(flat.contiguous(), op, data_group)
        out.append(GradientReduceScatterBucket(shard, total, total + pad, list(bucket), numels))
    return out


def broadcast_owner_parameters(parameters: Sequence[torch.Tensor], owners: Sequence[int], comm: Collectives,
                               data_group: Sequence[int], bucket_bytes: int = DEFAULT_BUCKET_BYTES) -> int:
    """After a ZeRO-1 owner step: every owner (an index into ``data_group``) broadcasts the parameters
    it updated, in buckets, in place on every rank.  Returns the number of broadcast calls."""
    if len(owners) != len(parameters):
        raise ValueError("one owner per parameter is required")
    if len(data_group) == 1:
        return 0
    calls = 0
    for owner in range(len(data_group)):
        mine = [p if owners[i] == owner else None for i, p in enumerate(parameters)]
        for bucket in _buckets(mine, bucket_bytes, None):
            root = data_group[owner]
            if len(bucket) == 1:
                p = parameters[bucket[0]]
                with torch.no_grad():
                    p.copy_(comm.broadcast(p.detach().contiguous().view(-1), root, data_group).view_as(p))
            else:
                flat = torch.cat([parameters[i].detach().reshape(-1) for i in bucket])
                got = comm.broadcast(flat, root, data_group)
                off = 0
                with torch.no_grad():
                    for i in bucket:
                        n = parameters[i].numel()
                        parameters[i].copy_(got[off:off + n].view_as(parameters[i]))
                        off += n
            calls += 1
    return calls


def flat_bucket_ranges(numels: Sequence[int], offsets: Sequence[int], bucket_bytes: int,
                       elem_bytes: int) -> List[Tuple[int, int]]:
    """Contiguous ``[begin, end)`` element ranges of a flat buffer, cut at parameter boundaries so that a
    range holds at most ``bucket_bytes`` (one oversized parameter gets a range of its own)."""
    ranges: List[Tuple[int, int]] = []
    begin, cur = None, 0
    for n, off in zip(numels, offsets):
        nbytes = n * elem_bytes
        if begin is not None and cur + nbytes > bucket_bytes:
            ranges.append((begin, prev_end))
            begin, cur = None, 0
        if begin is None:
            begin = off
        cur += nbytes
        prev_end = off + n
    if begin is not None:
        ranges.append((begin, prev_end))
    return ranges


class TensorwiseOptimizer:
    """The trainer's two non-flat optimizer modes over a ``FlatParams`` buffer.

    ``mode="dense"``  every rank all-reduces (mean) the gradients over the data-parallel group in buckets
                      and runs per-tensor ``Fp32MasterAdamW`` on all parameters.
    ``mode="zero1"``  the same all-reduce, but each parameter has one owner rank that keeps its optimizer
                      state and updates it; owners then broadcast their parameters in buckets.

    Buckets are slices of the flat fp32 gradient buffer reduced in place (see the module text); with a
    narrower ``comm_dtype`` a slice is cast, reduced and copied back.  The global gradient norm is summed
    over ``norm_group`` - the ranks of one model replica - as the reference does for these modes
    (trainer.cc:2483-2494), the clip scale is ``max/(norm+1e-6)`` for a finite norm above the bound, and all
    scalars stay on the device in ``last_metrics = [local_sq, global_sq, clip_scale]``.
    """

    def __init__(self, flat_params, options: AdamWOptions, *, mode: str = "dense", dp_group=None, dp_rank: int = 0,
                 dp_size: int = 1, norm_group=None, norm_world: int = 1, max_grad_norm: float = 1.0,
                 comm_dtype: Optional[torch.dtype] = None, bucket_bytes: int = DEFAULT_BUCKET_BYTES):
        if mode not in ("dense", "zero1"):
            raise ValueError("mode must be 'dense' or 'zero1'")
        self.fp, self.mode = flat_params, mode
        self.dp_group, self.dp_rank, self.dp_size = dp_group, dp_rank, dp_size
        self.norm_group, self.norm_world = norm_group, norm_world
        self.max_grad_norm, self.comm_dtype, self.bucket_bytes = max_grad_norm, comm_dtype, bucket_bytes
        self.names = [n for n, _ in flat_params.named_tensors()]
        self.tensors = [t for _, t in flat_params.named_tensors()]
        self.grads = [flat_params.params[n].main_grad for n in self.names]
        numels = [t.numel() for t in self.tensors]
        if mode == "zero1" and dp_size > 1:
            self.owners = greedy_parameter_owners(numels, dp_size)
        else:
            self.owners = [dp_rank] * len(numels)
        self.optimizer_param_indices = [i for i, o in enumerate(self.owners) if o == dp_rank]
        self.adam = Fp32MasterAdamW([self.tensors[i] for i in self.optimizer_param_indices], options,
                                    main_grads=[self.grads[i] for i in self.optimizer_param_indices])
        offsets = [flat_params.offsets[n][0] for n in self.names]
        esize = 4 if comm_dtype is None else torch.empty((), dtype=comm_dtype).element_size()
        self.ranges = flat_bucket_ranges(numels, offsets, bucket_bytes, esize)
        # parameters by owner, as flat ranges, for the owner broadcast
        self.owner_ranges: List[List[Tuple[int, int]]] = []
        for r in range(dp_size):
            idx = [i for i, o in enumerate(self.owners) if o == r]
            psize = flat_params.flat.element_size()
            # ranges may only join parameters that are adjacent in the flat buffer
            runs: List[Tuple[int, int]] = []
            for i in idx:
                b, e = offsets[i], offsets[i] + numels[i]
                if runs and runs[-1][1] == b and (e - runs[-1][0]) * psize <= bucket_bytes:
                    runs[-1] = (runs[-1][0], e)
                else:
                    runs.append((b, e))
            self.owner_ranges.append(runs)
        self.last_metrics = torch.zeros(3, dtype=torch.float32, device=flat_params.flat.device)
        self.collective_calls = 0

    @property
    def step_count(self) -> int:
        return self.adam.step_count

    @torch.no_grad()
    def step(self) -> None:
        import torch.distributed as dist
        fp = self.fp
        if self.dp_size > 1:
            for b, e in self.ranges:
                sl = fp.main_grad[b:e]
                if self.comm_dtype is not None and self.comm_dtype != torch.float32:
                    tmp = sl.to(self.comm_dtype)
                    dist.all_reduce(tmp, group=self.dp_group)
                    sl.copy_(tmp)
                else:
                    dist.all_reduce(sl, group=self.dp_group)
                self.collective_calls += 1
            fp.main_grad.div_(self.dp_size)
        local_sq = optim_ops.sumsq(fp.main_grad)
        global_sq = local_sq
        if self.norm_world > 1:
            global_sq = local_sq.clone()
            dist.all_reduce(global_sq, group=self.norm_group)
        clip = optim_ops.clip_scale(global_sq, self.max_grad_norm)
        self.adam.has_main_grad = True          # the backward kernels filled the adopted accumulators
        if self.max_grad_norm > 0:
            self.adam.scale_gradients(clip[0])
        self.adam.step()
        fp.main_grad.zero_()
        self.last_metrics = torch.cat([local_sq.reshape(1), global_sq.reshape(1), clip[:1]])
        if self.mode == "zero1" and self.dp_size > 1:
            for r, runs in enumerate(self.owner_ranges):
                src = dist.get_global_rank(self.dp_group, r) if self.dp_group is not None else r
                for b, e in runs:
                    dist.broadcast(fp.flat[b:e], src=src, group=self.dp_group)
                    self.collective_calls += 1
