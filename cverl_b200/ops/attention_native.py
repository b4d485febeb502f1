"""Front end of the hand-written sm_100a attention kernels (cuda/attention_tcgen05.cu).

``attention_block(q, k, v, scale, causal, q_pos0, k_pos0) -> (out, lse)`` runs one (query range, key range)
block of attention and returns the un-normalised-merge pair: the normalised output of that key range and
its log-sum-exp, which is what ring attention merges across hops.  ``causal_attention`` is the plain
self-attention used by the model; its backward runs the tcgen05 backward kernels.
"""
from __future__ import annotations

import math
import os

import torch

from .. import _native as nv
from .gemm import count_launch


def _enabled() -> bool:
    return os.environ.get("CVERL_B200_ATTENTION", "auto") in ("auto", "native")


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq: int) -> bool:
    """bf16, head dim 128 or 256, sequence length a multiple of 128 (query blocks of 128, key blocks of 128)."""
    if not (_enabled() and q.is_cuda and q.dtype == k.dtype == v.dtype == torch.bfloat16):
        return False
    d = q.shape[-1]
    return d in (128, 256) and v.shape[-1] == d and k.shape[-1] == d and seq % 128 == 0 and \
        q.shape[-2] % k.shape[-2] == 0


def _fwd(q4, k4, v4, scale, causal, q_pos0, k_pos0):
    B, Sq, Hq, D = q4.shape
    Skv, Hkv = k4.shape[1], k4.shape[2]
    out = torch.empty_like(q4)
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q4.device)
    rc = nv.cuda().cvb_attention_fwd(q4.data_ptr(), k4.data_ptr(), v4.data_ptr(), out.data_ptr(), lse.data_ptr(), B, Sq,
                                     Skv, Hq, Hkv, D, scale, int(causal), q_pos0, k_pos0,
                                     nv.status_word(q4.device).data_ptr(), nv.stream())
    nv.check(rc, "cvb_attention_fwd")
    count_launch()
    return out, lse


def _bwd(q4, k4, v4, out, lse, dout, scale, causal, q_pos0, k_pos0):
    B, Sq, Hq, D = q4.shape
    Skv, Hkv = k4.shape[1], k4.shape[2]
    dev = q4.device
    delta = torch.empty((B, Hq, Sq), dtype=torch.float32, device=dev)
    dqt = torch.zeros((B, Hq, D, Sq), dtype=torch.float32, device=dev)
    dq = torch.empty_like(q4)
    dk = torch.empty((B, Skv, Hkv, D), dtype=torch.bfloat16, device=dev)   # summed over each GQA group in-kernel
    dv = torch.empty((B, Skv, Hkv, D), dtype=torch.bfloat16, device=dev)
    rc = nv.cuda().cvb_attention_bwd(q4.data_ptr(), k4.data_ptr(), v4.data_ptr(), out.data_ptr(), dout.data_ptr(),
                                     lse.data_ptr(), delta.data_ptr(), dqt.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                                     dv.data_ptr(), B, Sq, Skv, Hq, Hkv, D, scale, int(causal), q_pos0, k_pos0,
                                     nv.status_word(dev).data_ptr(), nv.stream())
    nv.check(rc, "cvb_attention_bwd")
    count_launch(4 if D == 128 else 5)
    return dq, dk, dv


class _AttentionBlock(torch.autograd.Function):
    """q [B,Sq,Hq,D], k/v [B,Skv,Hkv,D] -> (out [B,Sq,Hq,D], lse [B,Hq,Sq]); gradients flow through ``out``
    and, for merged hops, through ``lse`` (d lse adds P * dlse to dS, folded into delta)."""

    @staticmethod
    def forward(ctx, q4, k4, v4, scale, causal, q_pos0, k_pos0):
        q4, k4, v4 = q4.contiguous(), k4.contiguous(), v4.contiguous()
        out, lse = _fwd(q4, k4, v4, scale, causal, q_pos0, k_pos0)
        ctx.save_for_backward(q4, k4, v4, out, lse)
        ctx.cfg = (scale, causal, q_pos0, k_pos0)
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        q4, k4, v4, out, lse = ctx.saved_tensors
        scale, causal, q_pos0, k_pos0 = ctx.cfg
        dq, dk, dv = _bwd(q4, k4, v4, out, lse, dout.contiguous(), scale, causal, q_pos0, k_pos0)
        return dq, dk, dv, None, None, None, None


def attention_block(q4, k4, v4, scale: float, causal: bool = True, q_pos0: int = 0, k_pos0: int = 0):
    return _AttentionBlock.apply(q4, k4, v4, scale, causal, q_pos0, k_pos0)


def causal_attention(q, k, v, batch: int, seq: int, scale=None):
    """q [B*S, Hq, D], k/v [B*S, Hkv, D] -> [B*S, Hq, D] (causal self-attention per sequence)."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out, _ = attention_block(q.reshape(batch, seq, Hq, D), k.reshape(batch, seq, Hkv, D), v.reshape(batch, seq, Hkv, D),
                             float(scale), True, 0, 0)
    return out.reshape(T, Hq, D)
