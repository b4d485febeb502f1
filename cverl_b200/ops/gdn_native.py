"""Front end of the hand-written Gated-DeltaNet scan kernels (cuda/gdn_scan.cu)."""
from __future__ import annotations

import torch

from .. import _native as nv


def supported(q: torch.Tensor, v: torch.Tensor) -> bool:
    return False


def gated_delta_rule(q, k, v, beta, g, initial_state=None):  # pragma: no cover - needs the kernel
    raise NotImplementedError
