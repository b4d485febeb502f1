"""Autograd-aware collectives over ``torch.distributed`` groups.

The tensor-parallel pair is Megatron's f / g: ``copy_to_tp`` is the identity
forward and an all-reduce backward (the operator the reference omits, see
tools/model/qwen3_5_pp_tp_ppo_trainer.cc:545-558 for its averaging
work-around), ``reduce_from_tp`` is an all-reduce forward and the identity
backward (src/model/qwen3_5_text.cc:195-205).  ``all_to_all_rows`` is the
expert-parallel exchange whose backward is the reverse exchange
(src/distributed/expert_parallel.cc:43-81); ``all_gather_rows`` /
``reduce_scatter_rows`` are each other's backward (context parallel gather,
src/distributed/context_parallel.cc:101-141).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def _size(group) -> int:
    return 1 if group is None else dist.get_world_size(group)


class _CopyToTp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        y = x.contiguous().clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


def copy_to_tp(x: torch.Tensor, group) -> torch.Tensor:
    return x if _size(group) == 1 else _CopyToTp.apply(x, group)


def reduce_from_tp(x: torch.Tensor, group) -> torch.Tensor:
    return x if _size(group) == 1 else _ReduceFromTp.apply(x, group)


def all_reduce_sum_identity_bwd(x: torch.Tensor, group) -> torch.Tensor:
    return reduce_from_tp(x, group)


def all_reduce_max_nograd(x: torch.Tensor, group) -> torch.Tensor:
    if _size(group) == 1:
        return x
    y = x.detach().contiguous().clone()
    dist.all_reduce(y, op=dist.ReduceOp.MAX, group=group)
    return y


class _AllToAllRows(torch.autograd.Function):
    """Variable-size row exchange: rank r sends ``send_counts[p]`` rows to peer p."""

    @staticmethod
    def forward(ctx, x, send_counts: List[int], recv_counts: List[int], group):
        ctx.group, ctx.send_counts, ctx.recv_counts = group, send_counts, recv_counts
        out = x.new_empty((sum(recv_counts),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts,
                               group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.send_counts),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send_counts,
                               input_split_sizes=ctx.recv_counts, group=ctx.group)
        return out, None, None, None


def all_to_all_rows(x, send_counts, recv_counts, group):
    if _size(group) == 1:
        return x
    return _AllToAllRows.apply(x, list(send_counts), list(recv_counts), group)


class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        ws = dist.get_world_size(group)
        out = x.new_empty((ws * x.shape[0],) + tuple(x.shape[1:]))
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        ws = dist.get_world_size(ctx.group)
        out = g.new_empty((g.shape[0] // ws,) + tuple(g.shape[1:]))
        dist.reduce_scatter_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        ws = dist.get_world_size(group)
        out = x.new_empty((x.shape[0] // ws,) + tuple(x.shape[1:]))
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        ws = dist.get_world_size(ctx.group)
        out = g.new_empty((ws * g.shape[0],) + tuple(g.shape[1:]))
        dist.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


def all_gather_rows(x, group):
    return x if _size(group) == 1 else _AllGatherRows.apply(x, group)


def reduce_scatter_rows(x, group):
    return x if _size(group) == 1 else _ReduceScatterRows.apply(x, group)


class _SendRecvState(torch.autograd.Function):
    """Hand a tensor to the next rank of a chain; the gradient flows back the other way.

    Used for the context-parallel recurrent-state carry of linear attention
    (src/model/qwen3_5_text.cc:444-526): rank r receives from r-1 and sends to r+1.
    """

    @staticmethod
    def forward(ctx, x, src: Optional[int], dst: Optional[int], group, like):
        ctx.src, ctx.dst, ctx.group = src, dst, group
        if dst is not None:
            dist.send(x.contiguous(), dst=dst, group=group)
        if src is not None:
            out = torch.empty_like(like)
            dist.recv(out, src=src, group=group)
            return out
        return torch.zeros_like(like)

    @staticmethod
    def backward(ctx, g):
        gx = None
        if ctx.src is not None:
            dist.send(g.contiguous(), dst=ctx.src, group=ctx.group)
        if ctx.dst is not None:
            gx = torch.empty_like(g)
            dist.recv(gx, src=ctx.dst, group=ctx.group)
        else:
            gx = torch.zeros_like(g)
        return gx, None, None, None, None
