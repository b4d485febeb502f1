"""Context-parallel attention by peer pull: no ring send / recv.

Every rank keeps the K and V of its sequence shard in a peer-mapped buffer (one per attention layer, so that
the values are still there in the backward pass).  A rank's attention over an earlier rank's keys is then one
launch of the tcgen05 attention kernel whose K / V tensor maps point at that rank's buffer: the TMA loads pull
the tiles over NVLink as they are needed (plain TMA loads, no multicast).  The hops are independent launches
merged through their log-sum-exps.  In the backward pass each rank writes its dK | dV contribution for every
key owner into a local fp32 staging slot; after a flag barrier each owner pulls and sums its slot from all
peers (the same pull kernel as the ZeRO reduce-scatter).

The reference moves K / V around a ring with ncclSend / ncclRecv and concatenates them
(src/distributed/context_parallel.cc:143-260).
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from .. import _native as nv
from ..ops import attention_native as an
from ..ops.gemm import count_launch
from .symm import SymmBarrier, SymmetricHeap


class CpSymm:
    def __init__(self, group, device):
        self.heap = SymmetricHeap(group, device)
        self.world, self.rank = self.heap.world, self.heap.index
        self.device = torch.device(device)
        self.barrier = SymmBarrier(self.heap)
        self._kv: Dict[Tuple, tuple] = {}
        self._stage: Dict[Tuple, tuple] = {}

    def kv_buffers(self, key, shape, ):
        """(K buffer, V buffer) of ``shape`` [B, L, Hkv, D] bf16 for one layer / micro-batch slot (collective on
        first use)."""
        k = (key, tuple(shape))
        if k not in self._kv:
            n = 1
            for s in shape:
                n *= s
            bk, bv = self.heap.alloc(n * 2), self.heap.alloc(n * 2)
            self._kv[k] = (bk, bv, bk.tensor(n, torch.bfloat16).view(shape), bv.tensor(n, torch.bfloat16).view(shape))
        return self._kv[k]

    def stage(self, shape):
        """fp32 staging [world, 2, *shape] for the dK | dV contributions, shared by all layers."""
        k = tuple(shape)
        if k not in self._stage:
            n = 1
            for s in shape:
                n *= s
            b = self.heap.alloc(self.world * 2 * n * 4)
            self._stage[k] = (b, b.tensor(self.world * 2 * n, torch.float32).view(self.world, 2, *shape), 2 * n)
        return self._stage[k]


def ring_forward(ctx, q, k, v, cps: CpSymm, key, shard_len: int, scale: float):
    """q [B,Hq,L,D], k/v [B,Hkv,L,D] (this rank's shard).  Returns out [B,Hq,L,D]."""
    cp_rank, cp = cps.rank, cps.world
    q4 = q.transpose(1, 2).contiguous()
    k4, v4 = k.transpose(1, 2).contiguous(), v.transpose(1, 2).contiguous()
    bk, bv, kbuf, vbuf = cps.kv_buffers(key, k4.shape)
    cps.barrier()                                   # peers are done reading the previous contents of this slot
    kbuf.copy_(k4)
    vbuf.copy_(v4)
    cps.barrier()                                   # every shard is in place
    B, L, Hq, D = q4.shape
    Hkv = k4.shape[2]
    out = lse = None
    for owner in range(cp_rank, -1, -1):            # own block first (local), then earlier blocks by peer pull
        o_h = torch.empty_like(q4)
        l_h = torch.empty((B, Hq, L), dtype=torch.float32, device=q4.device)
        rc = nv.cuda().cvb_attention_fwd(q4.data_ptr(), bk.peer_ptrs[owner], bv.peer_ptrs[owner], o_h.data_ptr(),
                                         l_h.data_ptr(), B, L, L, Hq, Hkv, D, scale, int(owner == cp_rank),
                                         cp_rank * shard_len, owner * shard_len,
                                         nv.status_word(q4.device).data_ptr(), nv.stream())
        nv.check(rc, "cvb_attention_fwd (peer pull)")
        count_launch()
        if out is None:
            out, lse = o_h.float(), l_h
        else:
            new = torch.logaddexp(lse, l_h)
            out = out * torch.exp(lse - new).transpose(1, 2).unsqueeze(-1) + \
                o_h.float() * torch.exp(l_h - new).transpose(1, 2).unsqueeze(-1)
            lse = new
    out = out.to(q.dtype)
    ctx.save_for_backward(q4, out, lse)
    ctx.cps_state = (cps, key, k4.shape, shard_len, scale)
    return out.transpose(1, 2)


def ring_backward(ctx, do):
    q4, out, lse = ctx.saved_tensors
    cps, key, kshape, shard_len, scale = ctx.cps_state
    cp_rank, cp = cps.rank, cps.world
    bk, bv, kbuf, vbuf = cps.kv_buffers(key, kshape)
    sb, stage, slot_elems = cps.stage(kshape)
    B, L, Hq, D = q4.shape
    Hkv = kshape[2]
    do4 = do.transpose(1, 2).contiguous()
    dq = torch.zeros(q4.shape, dtype=torch.float32, device=q4.device)
    cps.barrier()                                   # the staging buffer is free (previous layer's pull is done)
    stage.zero_()
    lib = nv.cuda()
    for owner in range(cp_rank, -1, -1):
        delta = torch.empty((B, Hq, L), dtype=torch.float32, device=q4.device)
        dqt = torch.zeros((B, Hq, D, L), dtype=torch.float32, device=q4.device)
        dq_h = torch.empty_like(q4)
        dkh = torch.empty((B, L, Hkv, D), dtype=torch.bfloat16, device=q4.device)
        dvh = torch.empty((B, L, Hkv, D), dtype=torch.bfloat16, device=q4.device)
        rc = lib.cvb_attention_bwd(q4.data_ptr(), bk.peer_ptrs[owner], bv.peer_ptrs[owner], out.data_ptr(),
                                   do4.data_ptr(), lse.data_ptr(), delta.data_ptr(), dqt.data_ptr(), dq_h.data_ptr(),
                                   dkh.data_ptr(), dvh.data_ptr(), B, L, L, Hq, Hkv, D, scale, int(owner == cp_rank),
                                   cp_rank * shard_len, owner * shard_len, nv.status_word(q4.device).data_ptr(),
                                   nv.stream())
        nv.check(rc, "cvb_attention_bwd (peer pull)")
        count_launch(5)
        dq += dq_h.float()
        stage[owner, 0] = dkh.float()
        stage[owner, 1] = dvh.float()
    cps.barrier()                                   # every contribution is staged
    dkv = torch.empty((2,) + tuple(kshape), dtype=torch.float32, device=q4.device)
    sq = torch.zeros(1, dtype=torch.float32, device=q4.device)
    nv.check(lib.cvb_reduce_scatter_sumsq(sb.ptr_array(), cp, cp_rank, cp_rank * slot_elems, slot_elems, 1.0,
                                          dkv.data_ptr(), sq.data_ptr(), nv.stream()), "cp dK|dV pull")
    count_launch()
    dk = dkv[0].to(torch.bfloat16).transpose(1, 2)
    dv = dkv[1].to(torch.bfloat16).transpose(1, 2)
    return dq.to(q4.dtype).transpose(1, 2), dk, dv
