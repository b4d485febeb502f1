"""Front end of the hand-written sm_100a attention kernels (cuda/attention_tcgen05.cu).

``supported`` reports whether the kernel library exports the attention entry
points and the shape is one they cover; until then ``causal_attention`` in
``attention.py`` runs the library SDPA baseline.
"""
from __future__ import annotations

import torch

from .. import _native as nv


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq: int) -> bool:
    lib = nv.cuda()
    return hasattr(lib, "cvb_attention_fwd") and q.dtype == torch.bfloat16 and q.shape[-1] in (128, 256) \
        and _enabled()


def _enabled() -> bool:
    return False


def causal_attention(q, k, v, batch, seq, scale=None):  # pragma: no cover - needs the kernel
    raise NotImplementedError
