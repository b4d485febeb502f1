"""Fused LM-head log-probability: ``logp[r] = log_softmax(h[r] @ E.T)[target[r]]``
without materialising the ``[rows, vocab]`` logits in the forward pass.

Forward: one tcgen05 GEMM whose epilogue keeps a streaming max / sum-exp per
row and N tile and picks the target logit, then a tiny merge kernel.
Backward: the GEMM is replayed with an epilogue that writes
``g * (onehot - softmax)`` in bf16, followed by the two gradient GEMMs
(``dh`` and the fp32-accumulated ``dE``).  With ``vocab_lo``/``group`` the
vocabulary is sharded over a tensor-parallel group and the three per-row
statistics are exchanged instead of logits.
Reference: full fp32 logits + log_softmax + gather (src/model/qwen3_5_text.cc:
1590-1602) and the vocab-parallel variant (:1614-1629).
"""
from __future__ import annotations

import torch

from .. import _native as nv
from .gemm import count_launch, gemm_nn, gemm_raw, gemm_tn_acc, use_native, _row_major_2d


def lmhead_logprob_ref(h: torch.Tensor, emb: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    logits = h.float() @ emb.float().t()
    return torch.log_softmax(logits, dim=-1).gather(-1, targets.long().unsqueeze(-1)).squeeze(-1)


def _row_chunks(rows: int, vocab: int, budget_bytes: int = 8 << 30):
    """Row chunk size so that the bf16 softmax-gradient buffer stays under the budget."""
    per_row = vocab * 2
    chunk = max(128, (budget_bytes // per_row) // 128 * 128)
    return min(rows, chunk)


class _LmHeadLogProb(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, emb, targets, vocab_lo, group):
        h2 = _row_major_2d(h)
        emb2 = _row_major_2d(emb)
        M, K = h2.shape
        V = emb2.shape[0]
        dev = h2.device
        n_tiles = (V + 255) // 256
        local_t = (targets.long() - vocab_lo).contiguous()
        part_max = torch.empty((n_tiles, M), dtype=torch.float32, device=dev)
        part_sum = torch.empty((n_tiles, M), dtype=torch.float32, device=dev)
        tgt = torch.zeros(M, dtype=torch.float32, device=dev)
        gemm_raw(h2, emb2, None, M, V, K, a_mn=False, b_mn=False, epi=nv.EPI_LSE_PARTIAL, block_n=256,
                 targets=local_t, part_max=part_max, part_sum=part_sum, tgt_logit=tgt)
        lse = torch.empty(M, dtype=torch.float32, device=dev)
        logp = torch.empty(M, dtype=torch.float32, device=dev)
        lib = nv.cuda()
        if group is None:
            nv.check(lib.cvb_lse_combine(part_max.data_ptr(), part_sum.data_ptr(), tgt.data_ptr(), lse.data_ptr(),
                                         logp.data_ptr(), None, None, M, n_tiles, nv.stream()), "cvb_lse_combine")
            count_launch()
        else:
            import torch.distributed as dist
            rmax = torch.empty(M, dtype=torch.float32, device=dev)
            rsum = torch.empty(M, dtype=torch.float32, device=dev)
            nv.check(lib.cvb_lse_combine(part_max.data_ptr(), part_sum.data_ptr(), tgt.data_ptr(), None, None,
                                         rmax.data_ptr(), rsum.data_ptr(), M, n_tiles, nv.stream()),
                     "cvb_lse_combine")
            ws = dist.get_world_size(group)
            stats = torch.stack([rmax, rsum, tgt])  # [3, M]
            gathered = torch.empty((ws, 3, M), dtype=torch.float32, device=dev)
            dist.all_gather_into_tensor(gathered, stats, group=group)
            maxs = gathered[:, 0].contiguous()
            sums = gathered[:, 1].contiguous()
            tgts = gathered[:, 2].contiguous()
            nv.check(lib.cvb_lse_merge_ranks(maxs.data_ptr(), sums.data_ptr(), tgts.data_ptr(), lse.data_ptr(),
                                             logp.data_ptr(), M, ws, nv.stream()), "cvb_lse_merge_ranks")
            count_launch(2)
        ctx.save_for_backward(h2, emb, local_t, lse)
        ctx.group = group
        ctx.hshape = h.shape
        return logp.view(h.shape[:-1])

    @staticmethod
    def backward(ctx, dlogp):
        h2, emb, local_t, lse = ctx.saved_tensors
        emb2 = _row_major_2d(emb)
        M, K = h2.shape
        V = emb2.shape[0]
        dev = h2.device
        g = dlogp.reshape(-1).float().contiguous()
        dh = torch.empty((M, K), dtype=h2.dtype, device=dev)
        main_grad = getattr(emb, "main_grad", None)
        dE = main_grad if main_grad is not None else torch.zeros((V, K), dtype=torch.float32, device=dev)
        chunk = _row_chunks(M, V)
        dlog = torch.empty((chunk, V), dtype=torch.bfloat16, device=dev)
        for r0 in range(0, M, chunk):
            r1 = min(M, r0 + chunk)
            rows = r1 - r0
            d = dlog[:rows]
            gemm_raw(h2[r0:r1], emb2, d, rows, V, K, a_mn=False, b_mn=False, epi=nv.EPI_SOFTMAX_GRAD,
                     block_n=256, targets=local_t[r0:r1], lse=lse[r0:r1], gscale=g[r0:r1])
            gemm_nn(d, emb2, out=dh[r0:r1])          # dh = d @ E
            gemm_tn_acc(d, h2[r0:r1], dE)            # dE += d.T @ h
        # With a vocab-parallel group ``dh`` is this rank's partial sum over its vocabulary shard.  It is NOT
        # all-reduced here: the caller feeds ``h`` through ``copy_to_tp`` (identity forward, all-reduce backward),
        # as the PyTorch statement of this op does; reducing in both places would scale the gradient by the
        # group size.
        dEret = None if main_grad is not None else dE.to(emb.dtype)
        return dh.view(ctx.hshape), dEret, None, None, None


def lmhead_logprob(h: torch.Tensor, emb: torch.Tensor, targets: torch.Tensor, vocab_lo: int = 0,
                   group=None) -> torch.Tensor:
    """Per-row target log-probability under ``softmax(h @ emb.T)`` (fp32 result)."""
    if use_native(h) and emb.dtype == torch.bfloat16:
        return _LmHeadLogProb.apply(h, emb, targets, vocab_lo, group)
    if group is not None:
        return _lmhead_logprob_vocab_parallel_ref(h, emb, targets, vocab_lo, group)
    flat = lmhead_logprob_ref(h.reshape(-1, h.shape[-1]), emb, targets.reshape(-1))
    return flat.view(h.shape[:-1])


def _lmhead_logprob_vocab_parallel_ref(h, emb, targets, vocab_lo, group):
    """Vocab-parallel statement in PyTorch ops (max / sum-exp / target all-reduces)."""
    import torch.distributed as dist
    from ..parallel.autograd_collectives import all_reduce_sum_identity_bwd, all_reduce_max_nograd
    logits = h.float().reshape(-1, h.shape[-1]) @ emb.float().t()
    lmax = all_reduce_max_nograd(logits.max(dim=-1).values.detach(), group)
    ex = torch.exp(logits - lmax.unsqueeze(-1)).sum(-1)
    ex = all_reduce_sum_identity_bwd(ex, group)
    local = targets.reshape(-1).long() - vocab_lo
    ok = (local >= 0) & (local < emb.shape[0])
    tl = logits.gather(-1, local.clamp(0, emb.shape[0] - 1).unsqueeze(-1)).squeeze(-1) * ok
    tl = all_reduce_sum_identity_bwd(tl, group)
    return (tl - lmax - torch.log(ex)).view(h.shape[:-1])
