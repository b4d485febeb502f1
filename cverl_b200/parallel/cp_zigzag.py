"""Load-balanced context-parallel attention: zig-zag sequence sharding around the ring.

With a contiguous shard per rank, causal ring attention gives rank r the work of r + 1/2 key blocks: the last rank
does cp - 1/2 blocks while the first does half a block, and the step takes as long as the last rank.  Here the
sequence is cut into ``2 * cp`` half-chunks and rank i attends with half-chunks ``i`` and ``2 cp - 1 - i``.
Against the keys of owner j every rank then runs ONE attention-kernel launch per hop, all of the same size:

* j == i (own keys): both query halves against both key halves, causal over the local 2h x 2h block (with the
  local row / column numbers standing in for the positions: every key of the early half precedes every query of
  the late half, so the mask is exactly the causal one);
* j <  i: both query halves against the owner's EARLY key half, fully visible;
* j >  i: the LATE query half against both key halves of the owner, fully visible.

Each launch covers 2 h^2 score entries (the diagonal one 2 h^2 after masking), so all ranks finish together and the
attention time of the step drops from ``cp - 1/2`` to ``cp / 2 + 1/2`` block-units... of half the size squared:
about half the contiguous ring's critical path at cp = 8.  Partial results merge in fp32 with one kernel per hop
(``cuda/attn_merge.cu``).  K | V travel around the ring as one payload (NCCL send / recv posted before the hop's
attention so that the transfer overlaps it); the backward pass sends K | V with their fp32 gradient accumulators.

The layers around attention keep the contiguous shard (the Gated-DeltaNet state and the convolution halo pass
from rank to rank in sequence order), so ``zigzag_reshard`` moves q | k | v into the zig-zag layout before the
attention and the output back after it: two half-chunks out, two in, per rank and direction.

The reference shards contiguously and every rank walks all hops (src/distributed/context_parallel.cc:143-260).
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

from .context_parallel import _exchange, ring_schedule


# ---------------------------------------------------------------------------------------------------------------
# layout
# ---------------------------------------------------------------------------------------------------------------
def zigzag_chunks(rank: int, cp: int) -> Tuple[int, int]:
    """The two half-chunks (of ``2 * cp``) that zig-zag rank ``rank`` holds, early one first."""
    return rank, 2 * cp - 1 - rank


def zigzag_owner(chunk: int, cp: int) -> Tuple[int, int]:
    """(rank, slot) that holds half-chunk ``chunk`` in the zig-zag layout."""
    return (chunk, 0) if chunk < cp else (2 * cp - 1 - chunk, 1)


def _swap_halves(x: torch.Tensor, group, rank: int, cp: int, to_zigzag: bool) -> torch.Tensor:
    """x [B, T, C]: this rank's shard.  contiguous layout = half-chunks (2r, 2r+1); zig-zag = (r, 2cp-1-r)."""
    import torch.distributed as dist
    B, T, C = x.shape
    if T % 2:
        raise ValueError("zig-zag sharding needs an even shard length")
    h = T // 2
    out = torch.empty_like(x)
    halves = (x[:, :h], x[:, h:])
    sends: List[Tuple[int, torch.Tensor, int]] = []      # (chunk id, tensor, peer)
    recvs: List[Tuple[int, torch.Tensor, int]] = []      # (chunk id, buffer view, peer)
    if to_zigzag:
        mine_out = [(2 * rank + a, a) for a in (0, 1)]                  # chunk held now -> local half index
        mine_in = [(c, s) for s, c in enumerate(zigzag_chunks(rank, cp))]
        owner_now = lambda c: c // 2                                      # noqa: E731
        owner_then = lambda c: zigzag_owner(c, cp)[0]                     # noqa: E731
    else:
        mine_out = [(c, s) for s, c in enumerate(zigzag_chunks(rank, cp))]
        mine_in = [(2 * rank + a, a) for a in (0, 1)]
        owner_now = lambda c: zigzag_owner(c, cp)[0]                      # noqa: E731
        owner_then = lambda c: c // 2                                     # noqa: E731
    for c, a in mine_out:
        dst = owner_then(c)
        if dst == rank:
            slot = [s for cc, s in mine_in if cc == c][0]
            out[:, slot * h:(slot + 1) * h].copy_(halves[a])
        else:
            sends.append((c, halves[a].contiguous(), dst))
    bufs = []
    for c, s in mine_in:
        src = owner_now(c)
        if src != rank:
            buf = torch.empty((B, h, C), dtype=x.dtype, device=x.device)
            bufs.append((s, buf))
            recvs.append((c, buf, src))
    ops = []
    for c, t, peer in sorted(sends, key=lambda e: e[0]):
        ops.append(dist.P2POp(dist.isend, t, dist.get_global_rank(group, peer), group))
    for c, t, peer in sorted(recvs, key=lambda e: e[0]):
        ops.append(dist.P2POp(dist.irecv, t, dist.get_global_rank(group, peer), group))
    if ops:
        for r in dist.batch_isend_irecv(ops):
            r.wait()
    for s, buf in bufs:
        out[:, s * h:(s + 1) * h].copy_(buf)
    return out


class _Reshard(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, rank, cp, to_zigzag):
        ctx.cfg = (group, rank, cp, to_zigzag)
        return _swap_halves(x.contiguous(), group, rank, cp, to_zigzag)

    @staticmethod
    def backward(ctx, g):
        group, rank, cp, to_zigzag = ctx.cfg
        return _swap_halves(g.contiguous(), group, rank, cp, not to_zigzag), None, None, None, None


def zigzag_reshard(x: torch.Tensor, group, rank: int, cp: int, to_zigzag: bool) -> torch.Tensor:
    """Moves this rank's ``[B, T, C]`` shard between the contiguous and the zig-zag layout (differentiable)."""
    if cp == 1:
        return x
    return _Reshard.apply(x, group, rank, cp, to_zigzag)


# ---------------------------------------------------------------------------------------------------------------
# one hop: the attention kernels on CUDA bf16, a plain fp32 statement elsewhere (the tests' oracle)
# ---------------------------------------------------------------------------------------------------------------
def _native(q4: torch.Tensor, tq: int, tk: int) -> bool:
    if not (q4.is_cuda and q4.dtype == torch.bfloat16 and q4.shape[-1] in (128, 256)):
        return False
    from ..ops import attention_native
    return attention_native._enabled() and tq % 128 == 0 and tk % 128 == 0


def _scores(q4, k4, scale, causal):
    B, Tq, Hq, D = q4.shape
    Tk, Hkv = k4.shape[1], k4.shape[2]
    g = Hq // Hkv
    kf = k4.float().repeat_interleave(g, dim=2) if g > 1 else k4.float()
    s = torch.einsum("bqhd,bkhd->bhqk", q4.float(), kf) * scale
    if causal:      # local numbering: row r sees columns c <= r + (Tk - Tq)
        r = torch.arange(Tq, device=q4.device).unsqueeze(1) + (Tk - Tq)
        c = torch.arange(Tk, device=q4.device).unsqueeze(0)
        s = s.masked_fill(c > r, float("-inf"))
    return s


def hop_forward(q4, k4, v4, scale: float, causal: bool):
    """(out [B, Tq, Hq, D] in q's dtype, lse [B, Hq, Tq] fp32).  Causal means: local row r sees local columns
    c <= r + (Tk - Tq) (the diagonal hop has Tq == Tk)."""
    Tq, Tk = q4.shape[1], k4.shape[1]
    if _native(q4, Tq, Tk):
        from ..ops import attention_native as an
        return an._fwd(q4.contiguous(), k4.contiguous(), v4.contiguous(), scale, causal, Tk - Tq if causal else 0, 0)
    s = _scores(q4, k4, scale, causal)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    g = q4.shape[2] // v4.shape[2]
    vf = v4.float().repeat_interleave(g, dim=2) if g > 1 else v4.float()
    out = torch.einsum("bhqk,bkhd->bqhd", p, vf)
    return out.to(q4.dtype), lse


def hop_backward(q4, k4, v4, out, lse, do4, scale: float, causal: bool):
    """(dq, dk, dv) of one hop against the FINAL merged output and log-sum-exp of its query rows."""
    Tq, Tk = q4.shape[1], k4.shape[1]
    if _native(q4, Tq, Tk):
        from ..ops import attention_native as an
        return an._bwd(q4.contiguous(), k4.contiguous(), v4.contiguous(), out.contiguous(), lse.contiguous(),
                       do4.contiguous(), scale, causal, Tk - Tq if causal else 0, 0)
    B, _, Hq, D = q4.shape
    Hkv = k4.shape[2]
    g = Hq // Hkv
    s = _scores(q4, k4, scale, causal)
    p = torch.exp(s - lse.unsqueeze(-1))
    kf = k4.float().repeat_interleave(g, dim=2) if g > 1 else k4.float()
    vf = v4.float().repeat_interleave(g, dim=2) if g > 1 else v4.float()
    delta = (do4.float() * out.float()).sum(-1).transpose(1, 2)                # [B, Hq, Tq]
    dp = torch.einsum("bqhd,bkhd->bhqk", do4.float(), vf)
    ds = p * (dp - delta.unsqueeze(-1))
    dq = torch.einsum("bhqk,bkhd->bqhd", ds, kf) * scale
    dk = torch.einsum("bhqk,bqhd->bkhd", ds, q4.float()) * scale
    dv = torch.einsum("bhqk,bqhd->bkhd", p, do4.float())
    if g > 1:
        dk = dk.view(B, Tk, Hkv, g, D).sum(3)
        dv = dv.view(B, Tk, Hkv, g, D).sum(3)
    return dq.to(q4.dtype), dk.to(k4.dtype), dv.to(v4.dtype)


def merge_partial(acc: torch.Tensor, lse: torch.Tensor, part: torch.Tensor, lse_p: torch.Tensor, row0: int,
                  first: bool) -> None:
    """In place: rows ``[row0, row0 + Tp)`` of (acc [B,T,H,D] fp32, lse [B,H,T]) take in (part [B,Tp,H,D], lse_p)."""
    B, T, H, D = acc.shape
    Tp = part.shape[1]
    if acc.is_cuda and part.dtype == torch.bfloat16:
        from .. import _native as nv
        from ..ops.gemm import count_launch
        part, lse_p = part.contiguous(), lse_p.contiguous()
        nv.check(nv.cuda().cvb_attn_merge(acc.data_ptr(), lse.data_ptr(), part.data_ptr(), lse_p.data_ptr(), B, T, Tp,
                                          H, D, row0, int(first), nv.stream()), "cvb_attn_merge")
        count_launch()
        return
    a, l = acc[:, row0:row0 + Tp], lse[:, :, row0:row0 + Tp]
    if first:
        a.copy_(part.float())
        l.copy_(lse_p)
        return
    new = torch.logaddexp(l, lse_p)
    safe = torch.where(torch.isinf(new), torch.zeros_like(new), new)
    w0 = torch.exp(l - safe).transpose(1, 2).unsqueeze(-1)
    w1 = torch.exp(lse_p - safe).transpose(1, 2).unsqueeze(-1)
    a.copy_(a * w0 + part.float() * w1)
    l.copy_(new)


# ---------------------------------------------------------------------------------------------------------------
# the ring
# ---------------------------------------------------------------------------------------------------------------
def _hop_plan(owner: int, rank: int, h: int):
    """(query row range, key row range, causal) of the single launch against ``owner``'s keys."""
    if owner == rank:
        return (0, 2 * h), (0, 2 * h), True
    if owner < rank:
        return (0, 2 * h), (0, h), False
    return (h, 2 * h), (0, 2 * h), False


class _ZigzagRing(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q4, k4, v4, group, rank, cp, scale):
        B, T, Hq, D = q4.shape
        h = T // 2
        q4 = q4.contiguous()
        kv = torch.cat([k4, v4], dim=-1).contiguous()                       # [B, T, Hkv, 2D]: one payload per hop
        acc = torch.empty((B, T, Hq, D), dtype=torch.float32, device=q4.device)
        lse = torch.empty((B, Hq, T), dtype=torch.float32, device=q4.device)
        seen = [False, False]                                               # per query half: has a partial result
        for owner, send_to, recv_from in ring_schedule(rank, cp):
            nxt, reqs = None, []
            if cp > 1 and owner != (rank + 1) % cp:                         # not the last step: post the next hop
                nxt, reqs = _exchange(kv, send_to, recv_from, group)
            (q0, q1), (k0, k1), causal = _hop_plan(owner, rank, h)
            o_h, l_h = hop_forward(q4[:, q0:q1], kv[:, k0:k1, :, :D], kv[:, k0:k1, :, D:], scale, causal)
            halves = [x for x in (0, 1) if q0 <= x * h < q1]
            if all(seen[x] == seen[halves[0]] for x in halves):
                merge_partial(acc, lse, o_h, l_h, q0, first=not seen[halves[0]])
            else:                                                           # one half is new, the other is not
                for x in halves:
                    a, b = x * h - q0, (x + 1) * h - q0
                    merge_partial(acc, lse, o_h[:, a:b], l_h[:, :, a:b], x * h, first=not seen[x])
            for x in halves:
                seen[x] = True
            for r in reqs:
                r.wait()
            if nxt is not None:
                kv = nxt
        out = acc.to(q4.dtype)
        ctx.save_for_backward(q4, k4, v4, out, lse)
        ctx.cfg = (group, rank, cp, scale)
        return out

    @staticmethod
    def backward(ctx, do4):
        q4, k4, v4, out, lse = ctx.saved_tensors
        group, rank, cp, scale = ctx.cfg
        B, T, Hq, D = q4.shape
        h = T // 2
        do4 = do4.contiguous()
        dq = torch.zeros(q4.shape, dtype=torch.float32, device=q4.device)
        # payload: K | V | dK | dV of the block currently held (gradients in fp32); after cp hops it is home again
        pay = torch.cat([k4.float(), v4.float(), torch.zeros_like(k4, dtype=torch.float32),
                         torch.zeros_like(v4, dtype=torch.float32)], dim=-1).contiguous()
        for owner, send_to, recv_from in ring_schedule(rank, cp):
            (q0, q1), (k0, k1), causal = _hop_plan(owner, rank, h)
            kb = pay[:, k0:k1, :, :D].to(k4.dtype)
            vb = pay[:, k0:k1, :, D:2 * D].to(v4.dtype)
            dq_h, dk_h, dv_h = hop_backward(q4[:, q0:q1], kb, vb, out[:, q0:q1], lse[:, :, q0:q1], do4[:, q0:q1],
                                            scale, causal)
            dq[:, q0:q1] += dq_h.float()
            pay[:, k0:k1, :, 2 * D:3 * D] += dk_h.float()
            pay[:, k0:k1, :, 3 * D:] += dv_h.float()
            if cp > 1:
                nxt, reqs = _exchange(pay, send_to, recv_from, group)
                for r in reqs:
                    r.wait()
                pay = nxt
        dk = pay[..., 2 * D:3 * D].to(k4.dtype)
        dv = pay[..., 3 * D:].to(v4.dtype)
        return dq.to(q4.dtype), dk, dv, None, None, None, None


def zigzag_supported(shard_len: int, original_len: int, cp: int) -> bool:
    """Zig-zag needs a sequence without padding and half-chunks the attention kernels take (multiples of 128 on
    CUDA; any even shard elsewhere)."""
    return cp > 1 and original_len == shard_len * cp and shard_len % 2 == 0


def zigzag_ring_attention(q4: torch.Tensor, k4: torch.Tensor, v4: torch.Tensor, group, rank: int, cp: int,
                          scale: Optional[float] = None) -> torch.Tensor:
    """Causal GQA attention over a zig-zag sharded sequence.

    ``q4 [B, T, Hq, D]``, ``k4 / v4 [B, T, Hkv, D]``: rows ``[0, T/2)`` are half-chunk ``rank`` and rows
    ``[T/2, T)`` half-chunk ``2 cp - 1 - rank`` of the sequence (``zigzag_reshard`` produces that layout).
    Returns the attention output in the same layout.
    """
    scale = scale if scale is not None else 1.0 / math.sqrt(q4.shape[-1])
    return _ZigzagRing.apply(q4, k4, v4, group, rank, cp, scale)
