"""ZeRO optimizer sharding: per-parameter owners and the flat-buffer shard.

Reference behaviour (src/distributed/optimizer_sharding.cc):
* ``greedy_parameter_owners`` - largest-first bin packing of whole parameters
  to data-parallel ranks (:389-434);
* the flat shard: parameters concatenated, zero-padded to a multiple of the DP
  size, rank r owns ``[r*S, (r+1)*S)`` (:18-89); gradients reduce-scattered
  (:463-585), global grad-norm all-reduced over a (possibly larger) norm group,
  clip ``max/(norm+1e-6)`` only for a finite norm above the bound, FlatAdamW on
  the shard, parameters all-gathered back (:587-733).

The generic functions take a ``Collectives`` object and plain tensors, so a
multi-rank run can be simulated rank by rank with scripted fakes.
``FlatZeroOptimizer`` is the production path over ``FlatParams``: gradients are
already accumulated in one fp32 flat buffer by the backward kernels, so the step
is reduce-scatter -> squared-norm kernel -> 1-float all-reduce -> clip kernel ->
fused AdamW kernel (zeroing the gradient) -> all-gather, with no host sync.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from ..ops import optim as optim_ops
from ..optim.adamw import AdamWOptions, FlatAdamW
from .collectives import Collectives, ReduceOp


def greedy_parameter_owners(numels: Sequence[int], dp_size: int) -> List[int]:
    """Owner rank of every parameter: largest first onto the least-loaded rank."""
    if dp_size <= 0:
        raise ValueError("dp_size must be positive")
    order = sorted(range(len(numels)), key=lambda i: (-numels[i], i))
    load = [0] * dp_size
    owners = [0] * len(numels)
    for i in order:
        r = min(range(dp_size), key=lambda k: (load[k], k))
        owners[i] = r
        load[r] += numels[i]
    return owners


@dataclass
class FlatParameterShard:
    original_numel: int
    padded_numel: int
    shard_begin: int
    shard_end: int
    shard: torch.Tensor

    @property
    def numel(self) -> int:
        return self.shard_end - self.shard_begin


def _padded(n: int, dp: int) -> int:
    return (n + dp - 1) // dp * dp


def flatten_parameter_shard(parameters: Sequence[torch.Tensor], dp_rank: int, dp_size: int,
                            dtype: Optional[torch.dtype] = None) -> FlatParameterShard:
    """This rank's slice of the conceptual flat concat of ``parameters`` (zero padded)."""
    total = sum(p.numel() for p in parameters)
    padded = _padded(max(total, 1), dp_size)
    size = padded // dp_size
    begin, end = dp_rank * size, (dp_rank + 1) * size
    dt = dtype or (parameters[0].dtype if parameters else torch.float32)
    dev = parameters[0].device if parameters else "cpu"
    shard = torch.zeros(size, dtype=dt, device=dev)
    off = 0
    for p in parameters:
        n = p.numel()
        lo, hi = max(off, begin), min(off + n, end)
        if lo < hi:
            shard[lo - begin:hi - begin].copy_(p.detach().reshape(-1)[lo - off:hi - off].to(dt))
        off += n
    return FlatParameterShard(total, padded, begin, end, shard)


def _flat_gradient(parameters: Sequence[torch.Tensor], padded: int, dtype, require_grad: bool) -> torch.Tensor:
    dev = parameters[0].device if parameters else "cpu"
    flat = torch.zeros(padded, dtype=dtype, device=dev)
    off = 0
    for p in parameters:
        n = p.numel()
        g = getattr(p, "main_grad", None)
        if g is None:
            g = p.grad
        if g is None:
            if require_grad:
                raise RuntimeError("parameter without a gradient in flat reduce-scatter")
        else:
            flat[off:off + n].copy_(g.detach().reshape(-1).to(dtype))
        off += n
    return flat


def reduce_scatter_flat_gradient_shard(parameters, comm: Collectives, group: Sequence[int],
                                       average: bool = True, require_grad: bool = True,
                                       comm_dtype: Optional[torch.dtype] = None,
                                       bucket_numel: int = 0) -> FlatParameterShard:
    """Reduce-scatter of the flat gradient; optionally in buckets of ``bucket_numel`` elements."""
    dp = len(group)
    idx = Collectives.rank_index_in_group(comm.rank(), group, "data group")
    total = sum(p.numel() for p in parameters)
    padded = _padded(max(total, 1), dp)
    size = padded // dp
    dtype = comm_dtype or torch.float32
    flat = _flat_gradient(parameters, padded, dtype, require_grad)
    op = ReduceOp.MEAN if average else ReduceOp.SUM
    if dp == 1:
        shard = flat
    elif bucket_numel and bucket_numel > 0:
        # each bucket carries one contiguous chunk of every rank's shard, interleaved as [dp, chunk]
        chunk = max(1, bucket_numel // dp)
        view = flat.view(dp, size)
        parts = []
        for c0 in range(0, size, chunk):
            c1 = min(size, c0 + chunk)
            parts.append(comm.reduce_scatter(view[:, c0:c1].contiguous().view(-1), op, group))
        shard = torch.cat(parts) if len(parts) > 1 else parts[0]
    else:
        shard = comm.reduce_scatter(flat, op, group)
    return FlatParameterShard(total, padded, idx * size, (idx + 1) * size, shard.float() if comm_dtype is None else shard)


def all_gather_apply_flat_parameter_shard(shard: FlatParameterShard, comm: Collectives, group: Sequence[int],
                                          parameters: Sequence[torch.Tensor], bucket_numel: int = 0) -> None:
    """All-gather every rank's shard and scatter the flat result back into ``parameters``."""
    dp = len(group)
    if dp == 1:
        full = shard.shard
    elif bucket_numel and bucket_numel > 0:
        size = shard.numel
        chunk = max(1, bucket_numel // dp)
        full = shard.shard.new_empty(dp, size)
        for c0 in range(0, size, chunk):
            c1 = min(size, c0 + chunk)
            g = comm.all_gather(shard.shard[c0:c1].contiguous(), group)
            full[:, c0:c1].copy_(g.view(dp, c1 - c0))
        full = full.view(-1)
    else:
        full = comm.all_gather(shard.shard.contiguous(), group)
    off = 0
    with torch.no_grad():
        for p in parameters:
            n = p.numel()
            p.copy_(full[off:off + n].view_as(p).to(p.dtype))
            off += n


@dataclass
class FlatAdamWStepResult:
    gradient_shard: Optional[FlatParameterShard] = None
    local_grad_norm_sq: float = 0.0
    global_grad_norm: float = 0.0
    grad_clip_scale: float = 1.0
    local_grad_norm: float = 0.0
    metrics_tensor: Optional[torch.Tensor] = None


def clear_parameter_gradients(parameters) -> None:
    for p in parameters:
        p.grad = None
        mg = getattr(p, "main_grad", None)
        if mg is not None:
            mg.zero_()


def flat_sharded_adamw_step(parameters, parameter_shard: FlatParameterShard, optimizer: FlatAdamW,
                            data_comm: Collectives, data_group: Sequence[int], norm_comm: Collectives,
                            norm_group: Sequence[int], max_grad_norm: float = 0.0, average_gradients: bool = True,
                            require_grad: bool = True, apply_parameters: bool = True,
                            reduce_scatter_bucket_numel: int = 0, all_gather_bucket_numel: int = 0,
                            comm_dtype: Optional[torch.dtype] = None) -> FlatAdamWStepResult:
    """One sharded optimizer step with the reference's semantics (generic tensors, any backend)."""
    if max_grad_norm < 0:
        raise ValueError("flat_sharded_adamw_step max_grad_norm must be non-negative")
    gs = reduce_scatter_flat_gradient_shard(parameters, data_comm, data_group, average_gradients, require_grad,
                                            comm_dtype, reduce_scatter_bucket_numel)
    if (gs.original_numel, gs.padded_numel, gs.shard_begin, gs.shard_end) != (
            parameter_shard.original_numel, parameter_shard.padded_numel, parameter_shard.shard_begin,
            parameter_shard.shard_end):
        raise RuntimeError("flat_sharded_adamw_step parameter/gradient shard metadata mismatch")
    clear_parameter_gradients(parameters)
    g32 = gs.shard.float().contiguous()
    local_sq = optim_ops.sumsq(g32)
    if len(norm_group) == 1:
        Collectives.rank_index_in_group(norm_comm.rank(), norm_group, "norm group")
        global_sq = local_sq
    else:
        global_sq = norm_comm.all_reduce(local_sq, ReduceOp.SUM, norm_group)
    clip = optim_ops.clip_scale(global_sq, max_grad_norm)
    optimizer.step(g32, clip=clip if max_grad_norm > 0 else None)
    parameter_shard.shard.copy_(optimizer.parameter_shard.to(parameter_shard.shard.dtype))
    res = FlatAdamWStepResult(gradient_shard=gs)
    res.metrics_tensor = torch.cat([local_sq.reshape(1), global_sq.reshape(1), clip[:1]])
    m = res.metrics_tensor.detach().cpu()  # the step's single device->host copy
    res.local_grad_norm_sq = float(m[0])
    res.global_grad_norm = float(m[1]) ** 0.5
    res.grad_clip_scale = float(m[2]) if max_grad_norm > 0 else 1.0
    res.local_grad_norm = (res.local_grad_norm_sq ** 0.5) * res.grad_clip_scale
    if apply_parameters:
        all_gather_apply_flat_parameter_shard(parameter_shard, data_comm, data_group, parameters,
                                              all_gather_bucket_numel)
    return res


class FlatZeroOptimizer:
    """ZeRO-1/2 flat-shard AdamW over a ``FlatParams`` buffer (production path).

    ``dp_group`` / ``norm_group`` are ``torch.distributed`` process groups (None =
    single rank / world).  ``replica_scale`` divides the reduced gradient (mean
    over DP).  All scalars stay on the device; ``last_metrics`` is a 3-float
    device tensor ``[local_sq, global_sq, clip_scale]`` read by the trainer once
    per step together with its other metrics.
    """

    def __init__(self, flat_params, options: AdamWOptions, *, dp_group=None, dp_rank: int = 0, dp_size: int = 1,
                 norm_group=None, norm_world: int = 1, max_grad_norm: float = 1.0,
                 comm_dtype: Optional[torch.dtype] = None, fused_comm=None):
        self.fp = flat_params
        self.dp_group, self.dp_rank, self.dp_size = dp_group, dp_rank, dp_size
        self.norm_group, self.norm_world = norm_group, norm_world
        self.max_grad_norm = max_grad_norm
        self.comm_dtype = comm_dtype
        self.fused_comm = fused_comm
        n = flat_params.padded_numel
        if n % dp_size:
            raise ValueError("flat buffer must be padded to a multiple of the data-parallel size")
        self.shard_numel = n // dp_size
        self.begin = dp_rank * self.shard_numel
        self.end = self.begin + self.shard_numel
        self.adam = FlatAdamW(flat_params.flat[self.begin:self.end], options)
        dev = flat_params.flat.device
        self.grad_shard = (torch.zeros(self.shard_numel, dtype=torch.float32, device=dev) if dp_size > 1 else None)
        self.last_metrics = torch.zeros(3, dtype=torch.float32, device=dev)

    def shard_meta(self) -> FlatParameterShard:
        return FlatParameterShard(self.fp.numel, self.fp.padded_numel, self.begin, self.end, self.adam.parameter_shard)

    @torch.no_grad()
    def step(self) -> None:
        import torch.distributed as dist
        fp = self.fp
        if self.dp_size > 1 and self.fused_comm is not None:
            self._fused_step()
            return
        if self.dp_size > 1:
            if self.comm_dtype is not None and self.comm_dtype != torch.float32:
                src = fp.main_grad.to(self.comm_dtype)
                out = torch.empty(self.shard_numel, dtype=self.comm_dtype, device=src.device)
                dist.reduce_scatter_tensor(out, src, op=dist.ReduceOp.SUM, group=self.dp_group)
                self.grad_shard.copy_(out)
                self.grad_shard.div_(self.dp_size)
                gshard = self.grad_shard
            else:
                if fp.main_grad.is_cuda:
                    dist.reduce_scatter_tensor(self.grad_shard, fp.main_grad, op=dist.ReduceOp.AVG,
                                               group=self.dp_group)
                else:
                    self._gloo_reduce_scatter()
                gshard = self.grad_shard
            fp.main_grad.zero_()
        else:
            gshard = fp.main_grad
        local_sq = optim_ops.sumsq(gshard)
        global_sq = local_sq
        if self.norm_world > 1:
            global_sq = local_sq.clone()
            dist.all_reduce(global_sq, group=self.norm_group)
        clip = optim_ops.clip_scale(global_sq, self.max_grad_norm)
        self.adam.step(gshard, clip=clip if self.max_grad_norm > 0 else None, zero_grad=(self.dp_size == 1))
        self.last_metrics = torch.cat([local_sq.reshape(1), global_sq.reshape(1), clip[:1]])
        if self.dp_size > 1:
            shard = fp.flat[self.begin:self.end]
            if fp.flat.is_cuda:
                dist.all_gather_into_tensor(fp.flat, shard, group=self.dp_group)
            else:
                parts = [torch.empty_like(shard) for _ in range(self.dp_size)]
                dist.all_gather(parts, shard.clone(), group=self.dp_group)
                fp.flat.copy_(torch.cat(parts))

    def _fused_step(self) -> None:
        """Symmetric-memory step: the reduce-scatter pulls peers' gradients and produces the squared
        norm in the same pass; the AdamW kernel's stores are the parameter all-gather.  The only
        library collective left is the 1-float norm all-reduce."""
        import torch.distributed as dist
        fc = self.fused_comm
        if fc.param_flat is not self.fp.flat or fc.grad_flat is not self.fp.main_grad:
            raise RuntimeError("fused ZeRO path needs FlatParams allocated by FusedZeroComm.allocator")
        local_sq = fc.reduce_scatter_mean_sumsq(self.grad_shard, self.begin).clone()
        global_sq = local_sq
        if self.norm_world > 1:
            global_sq = local_sq.clone()
            dist.all_reduce(global_sq, group=self.norm_group)
        clip = optim_ops.clip_scale(global_sq, self.max_grad_norm)
        fc.adamw_allgather(self.adam, self.grad_shard, clip if self.max_grad_norm > 0 else None, self.begin)
        self.last_metrics = torch.cat([local_sq.reshape(1), global_sq.reshape(1), clip[:1]])

    def _gloo_reduce_scatter(self) -> None:
        import torch.distributed as dist
        full = self.fp.main_grad.clone()
        dist.all_reduce(full, group=self.dp_group)
        self.grad_shard.copy_(full[self.begin:self.end])
        self.grad_shard.div_(self.dp_size)

    # --- checkpoint state ------------------------------------------------------
    def state_dict(self) -> dict:
        return {"flat_param_shard": self.adam.parameter_shard.detach().clone(),
                "flat_exp_avg": self.adam.exp_avg.detach().clone(),
                "flat_exp_avg_sq": self.adam.exp_avg_sq.detach().clone(),
                "optim_step": torch.tensor(self.adam.step_count, dtype=torch.int64)}

    def load_state_dict(self, sd: dict) -> None:
        self.adam.load_state(sd["flat_param_shard"], sd["flat_exp_avg"], sd["flat_exp_avg_sq"],
                             int(sd["optim_step"]))
