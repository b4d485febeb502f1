"""Context parallelism: sequence sharding, ring attention, linear-attention carries.

* ``shard_sequence`` / ``gather_sequence``: contiguous shards with zero padding
  (reference: src/distributed/context_parallel.cc:321-380).
* ``ring_schedule``: at step i a rank works on the K/V block of rank ``(local - i) mod cp``,
  sends to the next rank and receives from the previous one (:451-467).
* ``streaming_attention``: order-independent blockwise attention with a running max / sum /
  accumulator (:505-588) - the math of every ring step and the oracle of the kernels.
* ``ring_attention``: causal GQA attention over the ring.  Unlike the reference, which
  completes all hops, concatenates the remote K/V and only then runs one attention call
  (:160-176), every hop's transfer is posted before the block it overlaps is computed, and
  nothing is concatenated.  The backward pass sends each block round the ring again
  together with its gradient accumulator, which arrives at its owner after ``cp`` hops.
* ``conv_halo`` and ``carry_state``: what the Gated-DeltaNet layers need across shards - the
  ``kernel-1`` pre-convolution rows of the previous rank, and the ``[dk, dv]`` recurrent
  state handed from rank to rank with its gradient flowing back
  (src/model/qwen3_5_text.cc:444-526).  The reference instead ring-exchanges the full
  projected activations of every rank (:1274-1352).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


# ---------------------------------------------------------------------------------------------
# sharding helpers
# ---------------------------------------------------------------------------------------------
def padded_shard_len(seq_len: int, cp: int) -> int:
    return (seq_len + cp - 1) // cp


def shard_sequence(x: torch.Tensor, cp_rank: int, cp: int, dim: int = 1) -> torch.Tensor:
    """This rank's contiguous shard of ``x`` along ``dim`` (zero padded to ``cp * shard``)."""
    n = x.shape[dim]
    s = padded_shard_len(n, cp)
    if s * cp != n:
        pad = [0, 0] * (x.dim() - dim - 1) + [0, s * cp - n]
        x = F.pad(x, pad)
    return x.narrow(dim, cp_rank * s, s)


def gather_sequence(shard: torch.Tensor, group, dim: int = 1, original_len: Optional[int] = None) -> torch.Tensor:
    import torch.distributed as dist
    cp = dist.get_world_size(group)
    parts = [torch.empty_like(shard) for _ in range(cp)]
    dist.all_gather(parts, shard.contiguous(), group=group)
    full = torch.cat(parts, dim=dim)
    return full if original_len is None else full.narrow(dim, 0, original_len)


def ring_schedule(cp_rank: int, cp: int) -> List[Tuple[int, int, int]]:
    """``(block_owner, send_to, recv_from)`` for every ring step (group-local ranks)."""
    return [((cp_rank - i) % cp, (cp_rank + 1) % cp, (cp_rank - 1) % cp) for i in range(cp)]


# ---------------------------------------------------------------------------------------------
# blockwise attention math (fp32 statistics)
# ---------------------------------------------------------------------------------------------
def _block_scores(q, k, scale, q_pos, k_pos, k_valid_len):
    """q [B,Hq,Tq,D], k [B,Hkv,Tk,D] -> masked scores [B,Hq,Tq,Tk] (fp32)."""
    g = q.shape[1] // k.shape[1]
    kf = k.repeat_interleave(g, dim=1) if g > 1 else k
    s = torch.matmul(q.float(), kf.float().transpose(-1, -2)) * scale
    mask = (k_pos[None, :] > q_pos[:, None]) | (k_pos[None, :] >= k_valid_len)
    return s.masked_fill(mask, float("-inf"))


def streaming_attention(q, k_blocks: Sequence[torch.Tensor], v_blocks: Sequence[torch.Tensor], q_begin: int,
                        k_begins: Sequence[int], original_len: int, scale: Optional[float] = None):
    """Causal attention of ``q`` (positions ``q_begin ..``) over K/V blocks given in ANY order.

    Returns ``(out [B,Hq,Tq,Dv] in q's dtype, lse [B,Hq,Tq] fp32)``; fully masked rows give 0 / -inf.
    """
    B, Hq, Tq, D = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    q_pos = torch.arange(q_begin, q_begin + Tq, device=q.device)
    m = torch.full((B, Hq, Tq), float("-inf"), device=q.device)
    l = torch.zeros((B, Hq, Tq), device=q.device)
    acc = torch.zeros((B, Hq, Tq, v_blocks[0].shape[-1]), device=q.device)
    for k, v, kb in zip(k_blocks, v_blocks, k_begins):
        k_pos = torch.arange(kb, kb + k.shape[2], device=q.device)
        s = _block_scores(q, k, scale, q_pos, k_pos, original_len)
        m_new = torch.maximum(m, s.amax(-1))
        safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
        p = torch.exp(s - safe.unsqueeze(-1))
        alpha = torch.exp(torch.where(torch.isinf(m), torch.full_like(m, float("-inf")), m) - safe)
        g = q.shape[1] // v.shape[1]
        vf = v.repeat_interleave(g, dim=1) if g > 1 else v
        acc = acc * alpha.unsqueeze(-1) + torch.matmul(p, vf.float())
        l = l * alpha + p.sum(-1)
        m = m_new
    out = torch.where(l.unsqueeze(-1) > 0, acc / l.clamp_min(1e-38).unsqueeze(-1), torch.zeros_like(acc))
    lse = torch.where(l > 0, m + torch.log(l.clamp_min(1e-38)), torch.full_like(m, float("-inf")))
    return out.to(q.dtype), lse


def _exchange(send: torch.Tensor, send_to: int, recv_from: int, group):
    """Posts one ring hop; returns ``(recv_buffer, requests)`` so compute can overlap it."""
    import torch.distributed as dist
    recv = torch.empty_like(send)
    ops = [dist.P2POp(dist.isend, send.contiguous(), dist.get_global_rank(group, send_to), group),
           dist.P2POp(dist.irecv, recv, dist.get_global_rank(group, recv_from), group)]
    return recv, dist.batch_isend_irecv(ops)


def _native_hops(q, k, v, shard_len: int, original_len: int, cp: int) -> bool:
    """True when every hop can run on the tcgen05 attention kernels: CUDA bf16, head dim 128 / 256, shards of
    a multiple of 128 tokens and no padding inside the sequence."""
    if not q.is_cuda:
        return False
    from ..ops import attention_native
    return attention_native.supported(q, k, v, shard_len) and original_len == cp * shard_len and q.shape[2] == shard_len


def _ring_forward_native(ctx, q, k, v, group, cp_rank, cp, shard_len, original_len, scale):
    """Ring forward with one attention-kernel launch per visible hop: the hop of this rank's own block is
    causal, earlier blocks are fully visible, later ones are skipped; (out, lse) pairs merge in fp32."""
    from ..ops import attention_native as an
    q4 = q.transpose(1, 2).contiguous()                        # [B, Tq, Hq, D]
    kv = torch.cat([k.transpose(1, 2), v.transpose(1, 2)], dim=-1).contiguous()   # [B, Tk, Hkv, 2D], one payload
    D = q.shape[-1]
    out = lse = None
    for owner, send_to, recv_from in ring_schedule(cp_rank, cp):
        nxt, reqs = (None, [])
        if cp > 1 and owner != (cp_rank + 1) % cp:              # not the last step: post the next hop first
            nxt, reqs = _exchange(kv, send_to, recv_from, group)
        if owner <= cp_rank:
            o_h, l_h = an._fwd(q4, kv[..., :D].contiguous(), kv[..., D:].contiguous(), scale, owner == cp_rank,
                               cp_rank * shard_len, owner * shard_len)
            if out is None:
                out, lse = o_h.float(), l_h
            else:
                new = torch.logaddexp(lse, l_h)
                w0 = torch.exp(lse - new).transpose(1, 2).unsqueeze(-1)
                w1 = torch.exp(l_h - new).transpose(1, 2).unsqueeze(-1)
                out = out * w0 + o_h.float() * w1
                lse = new
        for r in reqs:
            r.wait()
        if nxt is not None:
            kv = nxt
    out = out.to(q.dtype)
    ctx.save_for_backward(q4, k, v, out, lse)
    ctx.cfg = (group, cp_rank, cp, shard_len, original_len, scale)
    return out.transpose(1, 2)


def _ring_backward_native(ctx, do):
    """Ring backward: K | V travel with their fp32 gradient accumulators; each visible hop runs the attention
    backward kernels against the FINAL (merged) output and log-sum-exp."""
    from ..ops import attention_native as an
    q4, k, v, out, lse = ctx.saved_tensors
    group, cp_rank, cp, shard_len, original_len, scale = ctx.cfg
    D = q4.shape[-1]
    do4 = do.transpose(1, 2).contiguous()
    dq = torch.zeros(q4.shape, dtype=torch.float32, device=q4.device)
    k4, v4 = k.transpose(1, 2), v.transpose(1, 2)
    pay = torch.cat([k4.float(), v4.float(), torch.zeros_like(k4, dtype=torch.float32),
                     torch.zeros_like(v4, dtype=torch.float32)], dim=-1).contiguous()
    for owner, send_to, recv_from in ring_schedule(cp_rank, cp):
        if owner <= cp_rank:
            kb = pay[..., :D].to(torch.bfloat16).contiguous()
            vb = pay[..., D:2 * D].to(torch.bfloat16).contiguous()
            dq_h, dk_h, dv_h = an._bwd(q4, kb, vb, out, lse, do4, scale, owner == cp_rank, cp_rank * shard_len,
                                       owner * shard_len)
            dq += dq_h.float()
            pay[..., 2 * D:3 * D] += dk_h.float()
            pay[..., 3 * D:] += dv_h.float()
        if cp > 1:                                              # cp hops bring every block home
            nxt, reqs = _exchange(pay, send_to, recv_from, group)
            for r in reqs:
                r.wait()
            pay = nxt
    dk = pay[..., 2 * D:3 * D].to(k.dtype).transpose(1, 2)
    dv = pay[..., 3 * D:].to(v.dtype).transpose(1, 2)
    return dq.to(q4.dtype).transpose(1, 2), dk, dv, None, None, None, None, None, None


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, group, cp_rank, cp, shard_len, original_len, scale, symm=None, key=None):
        B, Hq, Tq, D = q.shape
        ctx.native = _native_hops(q, k, v, shard_len, original_len, cp)
        ctx.pull = ctx.native and symm is not None and cp > 1
        if ctx.pull:       # K / V stay where they are: every hop pulls its tiles from the owner over NVLink
            from . import cp_symm
            return cp_symm.ring_forward(ctx, q, k, v, symm, key, shard_len, scale)
        if ctx.native:
            return _ring_forward_native(ctx, q, k, v, group, cp_rank, cp, shard_len, original_len, scale)
        q_begin = cp_rank * shard_len
        q_pos = torch.arange(q_begin, q_begin + Tq, device=q.device)
        m = torch.full((B, Hq, Tq), float("-inf"), device=q.device)
        l = torch.zeros((B, Hq, Tq), device=q.device)
        acc = torch.zeros((B, Hq, Tq, v.shape[-1]), device=q.device)
        kv = torch.cat([k, v], dim=-1).contiguous()        # K and V travel as one payload per hop
        for owner, send_to, recv_from in ring_schedule(cp_rank, cp):
            nxt, reqs = (None, [])
            if owner != (cp_rank + 1) % cp or cp == 1:      # not the last step: post the next hop first
                if cp > 1 and owner != (cp_rank - (cp - 1)) % cp:
                    nxt, reqs = _exchange(kv, send_to, recv_from, group)
            if owner <= cp_rank:                             # blocks from later ranks are fully masked
                kb, vb = kv[..., :D], kv[..., D:]
                k_pos = torch.arange(owner * shard_len, owner * shard_len + kb.shape[2], device=q.device)
                s = _block_scores(q, kb, scale, q_pos, k_pos, original_len)
                m_new = torch.maximum(m, s.amax(-1))
                safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
                p = torch.exp(s - safe.unsqueeze(-1))
                alpha = torch.exp(torch.where(torch.isinf(m), torch.full_like(m, float("-inf")), m) - safe)
                g = Hq // vb.shape[1]
                vf = vb.repeat_interleave(g, dim=1) if g > 1 else vb
                acc = acc * alpha.unsqueeze(-1) + torch.matmul(p, vf.float())
                l = l * alpha + p.sum(-1)
                m = m_new
            for r in reqs:
                r.wait()
            if nxt is not None:
                kv = nxt
        out = torch.where(l.unsqueeze(-1) > 0, acc / l.clamp_min(1e-38).unsqueeze(-1), torch.zeros_like(acc)).to(q.dtype)
        lse = torch.where(l > 0, m + torch.log(l.clamp_min(1e-38)), torch.full_like(m, float("-inf")))
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (group, cp_rank, cp, shard_len, original_len, scale)
        return out

    @staticmethod
    def backward(ctx, do):
        if ctx.pull:
            from . import cp_symm
            return cp_symm.ring_backward(ctx, do) + (None,) * 8
        if ctx.native:
            return _ring_backward_native(ctx, do) + (None, None)
        q, k, v, out, lse = ctx.saved_tensors
        group, cp_rank, cp, shard_len, original_len, scale = ctx.cfg
        B, Hq, Tq, D = q.shape
        Hkv = k.shape[1]
        g = Hq // Hkv
        q_begin = cp_rank * shard_len
        q_pos = torch.arange(q_begin, q_begin + Tq, device=q.device)
        delta = (do.float() * out.float()).sum(-1)                       # rowsum(dO * O)
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        # payload: K | V | dK | dV of the block currently held (gradients in fp32)
        pay = torch.cat([k.float(), v.float(), torch.zeros_like(k, dtype=torch.float32),
                         torch.zeros_like(v, dtype=torch.float32)], dim=-1).contiguous()
        Dv = v.shape[-1]
        lse_safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
        for owner, send_to, recv_from in ring_schedule(cp_rank, cp):
            if owner <= cp_rank:
                kb, vb = pay[..., :D], pay[..., D:D + Dv]
                k_pos = torch.arange(owner * shard_len, owner * shard_len + kb.shape[2], device=q.device)
                s = _block_scores(q, kb, scale, q_pos, k_pos, original_len)
                p = torch.exp(s - lse_safe.unsqueeze(-1))
                p = torch.where(torch.isinf(lse).unsqueeze(-1), torch.zeros_like(p), p)
                vf = vb.repeat_interleave(g, dim=1) if g > 1 else vb
                kf = kb.repeat_interleave(g, dim=1) if g > 1 else kb
                dp = torch.matmul(do.float(), vf.transpose(-1, -2))
                ds = p * (dp - delta.unsqueeze(-1))
                dq += torch.matmul(ds, kf) * scale
                dk_full = torch.matmul(ds.transpose(-1, -2), q.float()) * scale      # [B,Hq,Tk,D]
                dv_full = torch.matmul(p.transpose(-1, -2), do.float())
                if g > 1:
                    dk_full = dk_full.view(B, Hkv, g, -1, D).sum(2)
                    dv_full = dv_full.view(B, Hkv, g, -1, Dv).sum(2)
                pay[..., D + Dv:2 * D + Dv] += dk_full
                pay[..., 2 * D + Dv:] += dv_full
            if cp > 1:                                                     # cp hops bring every block home
                nxt, reqs = _exchange(pay, send_to, recv_from, group)
                for r in reqs:
                    r.wait()
                pay = nxt
        dk = pay[..., D + Dv:2 * D + Dv].to(k.dtype)
        dv = pay[..., 2 * D + Dv:].to(v.dtype)
        return dq.to(q.dtype), dk, dv, None, None, None, None, None, None, None, None


def ring_attention(q, k, v, group, cp_rank: int, cp: int, original_len: int, scale: Optional[float] = None,
                   symm=None, key=None):
    """Causal GQA attention of this rank's query shard over the whole (sharded) sequence.

    ``q [B,Hq,Tq,D]``, ``k/v [B,Hkv,Tq,D]`` are this rank's contiguous shard; positions are
    ``cp_rank*Tq + arange(Tq)``; keys at positions >= ``original_len`` are padding.  With ``symm`` (a
    ``cp_symm.CpSymm``) and a per-layer ``key`` the hops pull K / V from the owners' peer-mapped buffers instead
    of passing them around the ring.
    """
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return _RingAttention.apply(q, k, v, group, cp_rank, cp, q.shape[2], original_len, scale, symm, key)


# ---------------------------------------------------------------------------------------------
# Gated-DeltaNet carries
# ---------------------------------------------------------------------------------------------
class _ConvHalo(torch.autograd.Function):
    """Prepends the previous rank's last ``halo`` rows (zeros on rank 0) along dim 1."""

    @staticmethod
    def forward(ctx, x, group, cp_rank, cp, halo):
        import torch.distributed as dist
        ctx.cfg = (group, cp_rank, cp, halo)
        tail = x[:, -halo:].contiguous()
        head = torch.zeros_like(tail)
        ops = []
        if cp_rank + 1 < cp:
            ops.append(dist.P2POp(dist.isend, tail, dist.get_global_rank(group, cp_rank + 1), group))
        if cp_rank > 0:
            ops.append(dist.P2POp(dist.irecv, head, dist.get_global_rank(group, cp_rank - 1), group))
        for r in (dist.batch_isend_irecv(ops) if ops else []):
            r.wait()
        return torch.cat([head, x], dim=1)

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist
        group, cp_rank, cp, halo = ctx.cfg
        g_head = g[:, :halo].contiguous()
        g_x = g[:, halo:].clone()
        g_tail = torch.zeros_like(g_head)
        ops = []
        if cp_rank > 0:
            ops.append(dist.P2POp(dist.isend, g_head, dist.get_global_rank(group, cp_rank - 1), group))
        if cp_rank + 1 < cp:
            ops.append(dist.P2POp(dist.irecv, g_tail, dist.get_global_rank(group, cp_rank + 1), group))
        for r in (dist.batch_isend_irecv(ops) if ops else []):
            r.wait()
        if cp_rank + 1 < cp:
            g_x[:, -halo:] += g_tail
        return g_x, None, None, None, None


def conv_halo(x, group, cp_rank: int, cp: int, halo: int):
    return x if cp == 1 or halo == 0 else _ConvHalo.apply(x, group, cp_rank, cp, halo)


class _RecvState(torch.autograd.Function):
    """Initial recurrent state from the previous rank; its gradient is sent back there."""

    @staticmethod
    def forward(ctx, anchor, like, group, cp_rank):
        import torch.distributed as dist
        ctx.cfg = (group, cp_rank)
        if cp_rank == 0:
            return torch.zeros_like(like)
        s = torch.empty_like(like)
        dist.recv(s, src=dist.get_global_rank(group, cp_rank - 1), group=group)
        return s

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist
        group, cp_rank = ctx.cfg
        if cp_rank > 0:
            dist.send(g.contiguous(), dst=dist.get_global_rank(group, cp_rank - 1), group=group)
        return None, None, None, None


class _SendState(torch.autograd.Function):
    """Hands the final state to the next rank; returns a zero scalar that must join the loss so
    that the backward pass waits for the next rank's state gradient."""

    @staticmethod
    def forward(ctx, state, group, cp_rank, cp):
        import torch.distributed as dist
        ctx.cfg = (group, cp_rank, cp)
        ctx.shape, ctx.dtype = state.shape, state.dtype
        if cp_rank + 1 < cp:
            dist.send(state.contiguous(), dst=dist.get_global_rank(group, cp_rank + 1), group=group)
        return state.new_zeros(())

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist
        group, cp_rank, cp = ctx.cfg
        gs = torch.zeros(ctx.shape, dtype=ctx.dtype, device=g.device)
        if cp_rank + 1 < cp:
            dist.recv(gs, src=dist.get_global_rank(group, cp_rank + 1), group=group)
        return gs, None, None, None


def recv_initial_state(anchor: torch.Tensor, like: torch.Tensor, group, cp_rank: int) -> torch.Tensor:
    """``anchor`` is any tensor that requires grad; it ties the receive into the autograd graph."""
    return _RecvState.apply(anchor, like, group, cp_rank)


def send_final_state(state: torch.Tensor, group, cp_rank: int, cp: int) -> torch.Tensor:
    return _SendState.apply(state, group, cp_rank, cp)
