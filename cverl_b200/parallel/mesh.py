"""Builds the ``ParallelContext`` of this rank: one ``torch.distributed`` group per axis.

The reference opens six independent communicators per process, each with its
own id file (tools/model/qwen3_5_pp_tp_ppo_trainer.cc:2000-2063); here every
axis is a sub-group of the one NCCL (or gloo) world, created collectively in a
fixed order so that all ranks agree.
"""
from __future__ import annotations

from typing import Optional

from .context import ParallelContext
from .topology import ClusterSpec, ParallelDims, Topology


def build_context(world: int, rank: int, *, tp: int = 1, dp: Optional[int] = None, pp: int = 1, cp: int = 1,
                  ep: int = 1, micro_batches: Optional[int] = None, gpus_per_node: int = 8,
                  fused_comm: bool = False) -> ParallelContext:
    if dp is None:
        dp = world // (tp * pp * cp * ep)
    dims = ParallelDims(data=dp, pipeline=pp, context=cp, tensor=tp, expert=ep,
                        micro_batches=micro_batches or max(pp, 1))
    topo = Topology(dims, ClusterSpec(world_size=world, rank=rank, gpus_per_node=max(gpus_per_node, tp)))
    info = topo.rank_info(rank)
    ctx = ParallelContext(tp_rank=info.tensor_rank, tp_size=tp, ep_rank=info.expert_rank, ep_size=ep,
                          cp_rank=info.context_rank, cp_size=cp, dp_rank=info.data_rank, dp_size=dp,
                          pp_rank=info.pipeline_rank, pp_size=pp, fused_comm=fused_comm)
    ctx.topology = topo
    ctx.rank_info = info
    if world == 1:
        return ctx
    import torch.distributed as dist
    for axis, attr, size in (("tensor", "tp_group", tp), ("expert", "ep_group", ep), ("context", "cp_group", cp),
                             ("data", "dp_group", dp)):
        if size == 1:
            continue
        mine = None
        for ranks in topo.all_groups(axis):  # every rank creates every group, in the same order
            g = dist.new_group(ranks)
            if rank in ranks:
                mine = g
        setattr(ctx, attr, mine)
    if dp > 1 and world // dp > 1:
        for ranks in topo.all_groups("model"):
            g = dist.new_group(ranks)
            if rank in ranks:
                ctx.model_group = g
    # first and last pipeline stage of every pipeline group: they share the tied embedding
    ctx.embed_group = None
    if pp > 1:
        for ranks in topo.all_groups("pipeline"):
            g = dist.new_group([ranks[0], ranks[-1]])
            if rank in (ranks[0], ranks[-1]):
                ctx.embed_group = g
    return ctx
