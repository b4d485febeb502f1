"""Causal GQA attention on packed ``[B*S, heads, D]`` activations.

``causal_attention`` dispatches to the hand-written sm_100a kernel when it is
available for the shape (``cuda/attention_tcgen05.cu``); otherwise it runs the
library SDPA, which is the labelled baseline path, and on CPU the fp32 eager
statement below (the oracle of the tests).  The streaming (blockwise,
order-independent) softmax used by context parallelism lives in
``cverl_b200.parallel.context_parallel``.
Reference: at::scaled_dot_product_attention(causal, enable_gqa) in
src/model/qwen3_5_text.cc:1068-1075.
"""
from __future__ import annotations

import math
import os

import torch
import torch.nn.functional as F


def causal_attention_ref(q, k, v, batch: int, seq: int, scale: float | None = None):
    """q [B*S, Hq, D], k/v [B*S, Hkv, D] -> [B*S, Hq, D]; fp32 eager math."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().view(batch, seq, Hq, D).transpose(1, 2)
    kf = k.float().view(batch, seq, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    vf = v.float().view(batch, seq, Hkv, v.shape[-1]).transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    s = (qf @ kf.transpose(-1, -2)) * scale
    mask = torch.ones(seq, seq, dtype=torch.bool, device=q.device).triu(1)
    s = s.masked_fill(mask, float("-inf"))
    o = torch.softmax(s, dim=-1) @ vf
    return o.transpose(1, 2).reshape(T, Hq, v.shape[-1]).to(q.dtype)


def _sdpa(q, k, v, batch: int, seq: int, scale: float | None):
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    q4 = q.view(batch, seq, Hq, D).transpose(1, 2)
    k4 = k.view(batch, seq, Hkv, D).transpose(1, 2)
    v4 = v.view(batch, seq, Hkv, v.shape[-1]).transpose(1, 2)
    o = F.scaled_dot_product_attention(q4, k4, v4, is_causal=True, scale=scale, enable_gqa=(Hq != Hkv))
    return o.transpose(1, 2).reshape(T, Hq, v.shape[-1])


def causal_attention(q, k, v, batch: int, seq: int, scale: float | None = None):
    """Causal self-attention per sequence over a packed batch of equal-length sequences."""
    if q.is_cuda:
        backend = os.environ.get("CVERL_B200_ATTENTION", "auto")
        if backend != "sdpa":
            from . import attention_native
            if attention_native.supported(q, k, v, seq):
                return attention_native.causal_attention(q, k, v, batch, seq, scale)
            from ..utils import fallbacks
            fallbacks.note("causal_attention", f"dtype {q.dtype}, head dim {q.shape[-1]}, sequence length {seq}: the "
                                               f"tcgen05 kernels take bf16, head dim 128 / 256, length % 128 == 0")
        return _sdpa(q, k, v, batch, seq, scale)
    return causal_attention_ref(q, k, v, batch, seq, scale)
