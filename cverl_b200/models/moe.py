"""Qwen3-MoE feed-forward: router, expert dispatch, grouped expert GEMMs, combine.

* ``router``: fp32 logits, top-k, weights = softmax over the top-k (``norm_topk_prob``) or
  the gathered entries of the full softmax (src/model/qwen3_5_text.cc:761-772).
* ``moe_mlp_dense_loop``: the reference's loop over all experts (:773-789) - the oracle.
* ``moe_mlp``: sort (token, k) pairs by expert, pad every expert's segment to 128 rows,
  run gate|up and down as grouped tcgen05 GEMMs, combine with the routing weights.  With
  expert parallelism the pairs first travel to the rank that owns their expert and the
  results travel back (all-to-all whose backward is the reverse all-to-all,
  src/distributed/expert_parallel.cc:43-140); the single host read per layer is the
  vector of per-rank row counts that sizes the exchange (the reference needs five syncs).
  The expert FFN dimension may additionally be split over tensor parallelism (:819-822).
"""
from __future__ import annotations

from typing import Tuple

import torch

from .. import ops
from ..ops.grouped_gemm import TILE_M, grouped_linear
from ..parallel.autograd_collectives import all_to_all_rows, copy_to_tp, reduce_from_tp


def router(x: torch.Tensor, gate_w: torch.Tensor, top_k: int, norm_topk_prob: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [T, H] -> (expert ids [T, k] int64, routing weights [T, k] fp32); fused kernel on CUDA."""
    from ..ops.router import route
    return route(x, gate_w, top_k, norm_topk_prob)


def _expert_ffn_ref(x, gate_up_w, down_w):
    gu = x.float() @ gate_up_w.float().t()
    return (ops.activation.swiglu_ref(gu) @ down_w.float().t())


def moe_mlp_dense_loop(x, gate_w, gate_up, down, top_k: int, norm_topk_prob: bool) -> torch.Tensor:
    """Oracle: every expert processes the tokens routed to it (single rank, full experts)."""
    idx, w = router(x, gate_w, top_k, norm_topk_prob)
    out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    for e in range(gate_up.shape[0]):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        y = _expert_ffn_ref(x[tok], gate_up[e], down[e])
        out.index_add_(0, tok, y * w[tok, slot].unsqueeze(-1))
    return out.to(x.dtype)


def sort_by_expert(expert_ids: torch.Tensor, num_experts: int):
    """Layout of expert-sorted, 128-row padded rows for a flat list of expert ids (no host sync).

    Returns ``(order, dest, tile_group, offsets, m_pad)``: ``order`` sorts the entries by expert,
    ``dest[j]`` is the padded row of sorted entry ``j``, ``tile_group`` the expert of each
    128-row tile (-1 = unused), ``offsets`` int32 [E+1] the padded segment bounds.
    """
    n = expert_ids.numel()
    dev = expert_ids.device
    order = torch.argsort(expert_ids, stable=True)
    sorted_e = expert_ids[order]
    counts = torch.bincount(expert_ids, minlength=num_experts)[:num_experts]
    padded = (counts + TILE_M - 1) // TILE_M * TILE_M
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64, device=dev)
    offsets[1:] = padded.cumsum(0)
    starts = torch.zeros(num_experts + 1, dtype=torch.int64, device=dev)
    starts[1:] = counts.cumsum(0)
    dest = offsets[sorted_e] + (torch.arange(n, device=dev) - starts[sorted_e])
    m_pad = (n + num_experts * (TILE_M - 1) + TILE_M - 1) // TILE_M * TILE_M      # static upper bound
    tile_starts = torch.arange(0, m_pad, TILE_M, device=dev)
    tile_group = torch.searchsorted(offsets[1:], tile_starts, right=True)
    tile_group = torch.where(tile_starts < offsets[-1], tile_group, torch.full_like(tile_group, -1))
    return order, dest, tile_group.to(torch.int32), offsets.to(torch.int32), m_pad


def expert_layout(expert_ids: torch.Tensor, num_experts: int, tile_m: int = TILE_M):
    """``(row, tile_group, offsets, m_pad)``: ``row[i]`` is the row of entry ``i`` in the expert-grouped matrix the
    grouped GEMM reads, every expert's segment padded to a multiple of ``tile_m`` (128) rows and the entries of one
    expert in their original order; ``tile_group`` is the expert of each ``tile_m``-row tile (-1 = unused),
    ``offsets`` int32 [E+1] the padded segment bounds, ``m_pad`` a static upper bound of the padded row count.
    On CUDA the table comes from ``cvb_expert_layout`` (four small launches, no sort, no host read); elsewhere
    from ``sort_by_expert``.  With ``tile_m=1`` it is a plain stable grouping (used for the expert-parallel
    destination rows)."""
    n = expert_ids.numel()
    dev = expert_ids.device
    m_pad = (n + num_experts * (tile_m - 1) + tile_m - 1) // tile_m * tile_m
    if expert_ids.is_cuda and expert_ids.dtype == torch.int64 and num_experts <= 256 and n > 0:
        from .. import _native as nv
        ids = expert_ids.contiguous()
        nblocks = (n + 255) // 256
        scratch = torch.empty(n + (nblocks + 1) * (num_experts + 1), dtype=torch.int32, device=dev)
        offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
        tile_group = torch.empty(m_pad // tile_m, dtype=torch.int32, device=dev)
        row = torch.empty(n, dtype=torch.int64, device=dev)
        nv.check(nv.cuda().cvb_expert_layout(ids.data_ptr(), n, num_experts, tile_m, scratch.data_ptr(),
                                             offsets.data_ptr(), tile_group.data_ptr(), m_pad // tile_m,
                                             row.data_ptr(), nv.status_word(dev).data_ptr(), nv.stream()),
                 "cvb_expert_layout")
        ops.launch_counter["n"] += 4
        return row, tile_group, offsets, m_pad
    if tile_m != TILE_M:
        raise ValueError("the tensor-op layout pads to 128 rows only")
    order, dest, tile_group, offsets, m_pad = sort_by_expert(expert_ids, num_experts)
    row = torch.empty_like(order)
    row[order] = dest
    return row, tile_group, offsets, m_pad


def _local_experts(rows: torch.Tensor, local_ids: torch.Tensor, gate_up, down, num_local: int) -> torch.Tensor:
    """Runs ``rows[j]`` through local expert ``local_ids[j]``; returns outputs in the input order."""
    row, tile_group, offsets, m_pad = expert_layout(local_ids, num_local)
    xp = rows.new_zeros((m_pad, rows.shape[1])).index_copy(0, row, rows)
    gu = grouped_linear(xp, gate_up, tile_group, offsets)
    act = ops.swiglu(gu)
    yp = grouped_linear(act, down, tile_group, offsets)
    return yp[row]


def moe_mlp(model, x: torch.Tensor, layer: int) -> torch.Tensor:
    cfg, ctx = model.cfg, model.ctx
    p = f"{cfg.layer_root}{layer}.mlp."
    from .qwen3_5 import _packed_moe_names
    gu_name, dn_name = _packed_moe_names(layer)
    gate_up, down = model.param(gu_name), model.param(dn_name)          # [E_local, 2I_local, H], [E_local, H, I_local]
    T, H = x.shape
    k = cfg.num_experts_per_tok
    e_local = cfg.num_experts // ctx.ep_size
    # Under tensor parallelism the expert outputs below are partial sums (the FFN dimension is split), so the
    # gradient that reaches the routing weights - and through them the router's input and its gate matrix - is this
    # rank's share only.  The router therefore reads the copied input (whose backward sums the shares of both
    # paths over the group), and the gate matrix is one of ``tp_partial_grad_names``.
    x_in = copy_to_tp(x, ctx.tp_group)
    idx, w = router(x_in, model.param(p + "gate.weight"), k, cfg.norm_topk_prob)
    rows = x_in.repeat_interleave(k, dim=0)                              # one row per (token, k) pair
    flat_e = idx.reshape(-1)
    if ctx.ep_size == 1:
        y = _local_experts(rows, flat_e, gate_up, down, e_local)
    elif ctx.ep_symm is not None and rows.is_cuda and rows.dtype == torch.bfloat16:
        # dispatch / combine by our own kernels over NVLink peer memory: no host read of the split sizes
        from ..parallel import ep_symm
        eps = ctx.ep_symm
        peer_rank, peer_row, recv_expert = eps.plan(flat_e // e_local, flat_e % e_local, e_local)
        got_rows = ep_symm.dispatch(rows, peer_rank, peer_row, eps)
        if eps.fuse_combine and down.shape[1] % 64 == 0 and rows.shape[0] <= eps.cap:
            # the down projection's epilogue stores every output row into its token's home rank: no separate
            # combine, the expert outputs are never materialised on the expert rank
            row, tile_group, offsets, m_pad = expert_layout(recv_expert, e_local)
            xp = got_rows.new_zeros((m_pad, got_rows.shape[1])).index_copy(0, row, got_rows)
            act = ops.swiglu(grouped_linear(xp, gate_up, tile_group, offsets))
            y = ep_symm.fused_down_combine(act, down, tile_group, offsets, row, peer_rank, peer_row, eps)
        else:
            got_y = _local_experts(got_rows, recv_expert, gate_up, down, e_local)
            y = ep_symm.combine(got_y, peer_rank, peer_row, eps)
    else:
        import torch.distributed as dist
        dst_rank = flat_e // e_local
        order = torch.argsort(dst_rank, stable=True)
        send_counts = torch.bincount(dst_rank, minlength=ctx.ep_size)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=ctx.ep_group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()             # the layer's one host read
        sent_rows = rows[order]
        sent_ids = (flat_e[order] % e_local).contiguous()
        got_rows = all_to_all_rows(sent_rows, sc, rc, ctx.ep_group)
        got_ids = torch.empty(sum(rc), dtype=sent_ids.dtype, device=x.device)
        dist.all_to_all_single(got_ids, sent_ids, output_split_sizes=rc, input_split_sizes=sc, group=ctx.ep_group)
        got_y = _local_experts(got_rows, got_ids, gate_up, down, e_local)
        back = all_to_all_rows(got_y, rc, sc, ctx.ep_group)
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=order.device)
        y = back[inv]
    y = (y.float().view(T, k, H) * w.unsqueeze(-1)).sum(1).to(x.dtype)
    return reduce_from_tp(y, ctx.tp_group)
