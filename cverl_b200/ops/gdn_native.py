"""Front end of the tcgen05 Gated-DeltaNet state-scan kernels (cuda/gdn_scan.cu).

``scan_fwd`` / ``scan_bwd`` have the contracts of ``scan_fwd_ref`` / ``scan_bwd_ref``
in ``gdn.py``; operands travel as bf16, the state stays fp32 in tensor memory.
"""
from __future__ import annotations

import os

import torch

from .. import _native as nv
from .gemm import count_launch


def scan_supported(W: torch.Tensor, U: torch.Tensor) -> bool:
    if os.environ.get("CVERL_B200_GDN", "native") != "native":
        return False
    return W.is_cuda and W.shape[-1] == 128 and U.shape[-1] == 128 and W.shape[-2] == 64


def _bf(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).contiguous()


def scan_fwd(W, U, Kdec, egam, S0):
    B, H, n = W.shape[:3]
    dev = W.device
    Wb, Ub, Kb = _bf(W), _bf(U), _bf(Kdec)
    eg = egam.float().contiguous()
    s0 = S0.float().contiguous() if S0 is not None else None
    Vn = torch.empty((B, H, n, 64, 128), dtype=torch.bfloat16, device=dev)
    SsT = torch.empty((B, H, n, 128, 128), dtype=torch.bfloat16, device=dev)
    Sf = torch.empty((B, H, 128, 128), dtype=torch.float32, device=dev)
    rc = nv.cuda().cvb_gdn_scan_fwd(Wb.data_ptr(), Ub.data_ptr(), Kb.data_ptr(), eg.data_ptr(), nv.ptr(s0),
                                    Sf.data_ptr(), Vn.data_ptr(), SsT.data_ptr(), B * H, n,
                                    nv.status_word(dev).data_ptr(), nv.stream())
    nv.check(rc, "cvb_gdn_scan_fwd")
    count_launch()
    return Vn, SsT.transpose(-1, -2), Sf


def scan_bwd(dVloc, Kdec, Qd, W, dO, egam, dSf):
    B, H, n = W.shape[:3]
    dev = W.device
    dVl, Kb, Qb, Wb, dOb = _bf(dVloc), _bf(Kdec), _bf(Qd), _bf(W), _bf(dO)
    eg = egam.float().contiguous()
    dsf = dSf.float().contiguous() if dSf is not None else None
    dVn = torch.empty((B, H, n, 64, 128), dtype=torch.bfloat16, device=dev)
    dSnT = torch.empty((B, H, n, 128, 128), dtype=torch.bfloat16, device=dev)
    dS0 = torch.empty((B, H, 128, 128), dtype=torch.float32, device=dev)
    rc = nv.cuda().cvb_gdn_scan_bwd(dVl.data_ptr(), Kb.data_ptr(), Qb.data_ptr(), Wb.data_ptr(), dOb.data_ptr(),
                                    eg.data_ptr(), nv.ptr(dsf), dS0.data_ptr(), dVn.data_ptr(), dSnT.data_ptr(),
                                    B * H, n, nv.status_word(dev).data_ptr(), nv.stream())
    nv.check(rc, "cvb_gdn_scan_bwd")
    count_launch()
    return dVn, dSnT.transpose(-1, -2), dS0


def supported(q: torch.Tensor, v: torch.Tensor) -> bool:
    return False


def gated_delta_rule(q, k, v, beta, g, initial_state=None):  # pragma: no cover
    raise NotImplementedError
