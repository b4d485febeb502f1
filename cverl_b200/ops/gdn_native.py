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


def scan_bwd(P, Kdec, Qd, W, dO, egam, dSf):
    """Reverse state scan; ``P^T dO`` is formed inside.  Returns (dVn, dS_next per chunk, dS0)."""
    B, H, n = W.shape[:3]
    dev = W.device
    Pb, Kb, Qb, Wb, dOb = _bf(P), _bf(Kdec), _bf(Qd), _bf(W), _bf(dO)
    eg = egam.float().contiguous()
    dsf = dSf.float().contiguous() if dSf is not None else None
    dVn = torch.empty((B, H, n, 64, 128), dtype=torch.bfloat16, device=dev)
    dSnT = torch.empty((B, H, n, 128, 128), dtype=torch.bfloat16, device=dev)
    dS0 = torch.empty((B, H, 128, 128), dtype=torch.float32, device=dev)
    rc = nv.cuda().cvb_gdn_scan_bwd(Pb.data_ptr(), Kb.data_ptr(), Qb.data_ptr(), Wb.data_ptr(), dOb.data_ptr(),
                                    eg.data_ptr(), nv.ptr(dsf), dS0.data_ptr(), dVn.data_ptr(), dSnT.data_ptr(),
                                    B * H, n, 0, nv.status_word(dev).data_ptr(), nv.stream())
    nv.check(rc, "cvb_gdn_scan_bwd")
    count_launch()
    return dVn, dSnT.transpose(-1, -2), dS0


def chunk_supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    """The chunk kernels read q/k/v in place: bf16 [B,T,H,128] views with unit inner stride, head stride
    128, one common token stride and batch stride T * token stride; T a multiple of 64."""
    if os.environ.get("CVERL_B200_GDN", "native") != "native" or os.environ.get("CVERL_B200_GDN_CHUNK", "1") != "1":
        return False
    if not (q.is_cuda and q.dtype == k.dtype == v.dtype == torch.bfloat16):
        return False
    B, T, H, D = q.shape
    if D != 128 or v.shape[-1] != 128 or T % 64 != 0 or k.shape != q.shape or v.shape != q.shape:
        return False
    ts = q.stride(1)
    for t in (q, k, v):
        if t.stride(3) != 1 or t.stride(2) != 128 or t.stride(1) != ts or (B > 1 and t.stride(0) != T * ts):
            return False
        if t.data_ptr() % 16 or ts % 8:
            return False
    return True


def chunk_bwd_enabled() -> bool:
    return os.environ.get("CVERL_B200_GDN_CHUNK_BWD", "1") == "1"


def chunk_prep(q, k, v, beta, g, scale: float, eps: float = 1e-6, want_aux: bool = False):
    """Runs the chunk-local prep kernel. Returns dict(W, U, Kd, Qd [BH,n,64,128] bf16, P [BH,n,64,64] bf16,
    egam [BH,n] fp32 and, when ``want_aux``, Tm [BH,n,64,64] and aux [BH,n,3,64] fp32)."""
    B, T, H, _ = q.shape
    n = T // 64
    dev = q.device
    mk = lambda *s, dt=torch.bfloat16: torch.empty(s, dtype=dt, device=dev)
    out = dict(W=mk(B, H, n, 64, 128), U=mk(B, H, n, 64, 128), Kd=mk(B, H, n, 64, 128), Qd=mk(B, H, n, 64, 128),
               P=mk(B, H, n, 64, 64), egam=mk(B, H, n, dt=torch.float32))
    Tm = mk(B, H, n, 64, 64, dt=torch.float32) if want_aux else None
    aux = mk(B, H, n, 3, 64, dt=torch.float32) if want_aux else None
    bf, gf = beta.float().contiguous(), g.float().contiguous()
    rc = nv.cuda().cvb_gdn_chunk_prep(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(1), bf.data_ptr(),
                                      gf.data_ptr(), B, T, H, scale, eps, out["W"].data_ptr(), out["U"].data_ptr(),
                                      out["Kd"].data_ptr(), out["Qd"].data_ptr(), out["P"].data_ptr(),
                                      out["egam"].data_ptr(), nv.ptr(Tm), nv.ptr(aux),
                                      nv.status_word(dev).data_ptr(), nv.stream())
    nv.check(rc, "cvb_gdn_chunk_prep")
    count_launch()
    out["Tm"], out["aux"] = Tm, aux
    return out


def state_mode() -> str:
    """What the backward pass gets of the per-chunk recurrent states: ``full`` (kept from the forward pass),
    ``recompute`` (regenerated by one more launch of the forward scan) or ``budget`` (kept while they fit a byte
    budget).  Same environment switches as the reference (src/model/qwen3_5_text.cc:288-339):
    ``CVERL_LINEAR_ATTN_STATE_MODE`` = none | recompute | full | chunk | checkpoint, ``CVERL_LINEAR_ATTN_SAVE_STATES=1``
    (= full), ``CVERL_LINEAR_ATTN_CHECKPOINT_MAX_BYTES_MB`` and ``CVERL_LINEAR_ATTN_CHECKPOINT_INTERVAL``.

    The reference's chunk mode keeps every k-th state and replays k chunks at a time; the scan kernel here replays
    a whole sequence from its initial state in one launch (0.26 ms for 32 x 1280 tokens), so intermediate
    checkpoints would shorten nothing: chunk mode keeps ALL states of a call while they fit the budget and none
    otherwise.  The interval is validated and otherwise unused."""
    import os
    mode = os.environ.get("CVERL_LINEAR_ATTN_STATE_MODE", "")
    interval = os.environ.get("CVERL_LINEAR_ATTN_CHECKPOINT_INTERVAL", "")
    if interval and int(interval) <= 0:
        raise ValueError("CVERL_LINEAR_ATTN_CHECKPOINT_INTERVAL must be positive")
    if mode:
        if mode in ("none", "recompute"):
            return "recompute"
        if mode == "full":
            return "full"
        if mode in ("chunk", "checkpoint"):
            return "budget"
        raise ValueError("CVERL_LINEAR_ATTN_STATE_MODE must be none|recompute|full|chunk|checkpoint")
    if os.environ.get("CVERL_LINEAR_ATTN_SAVE_STATES", "") == "1":
        return "full"
    return "budget"


def keep_states(B: int, H: int, n: int) -> bool:
    """Whether a call with ``n`` chunks per (batch, head) keeps its states (bf16 S_c 128 x 128 and V' 64 x 128)."""
    import os
    mode = state_mode()
    if mode != "budget":
        return mode == "full"
    budget = os.environ.get("CVERL_LINEAR_ATTN_CHECKPOINT_MAX_BYTES_MB", "")
    if not budget:
        return True
    if int(budget) <= 0:
        raise ValueError("CVERL_LINEAR_ATTN_CHECKPOINT_MAX_BYTES_MB must be positive")
    return B * H * n * (128 * 128 + 64 * 128) * 2 <= int(budget) * 1024 * 1024


def regenerate_states(W, U, Kd, egam, S0):
    """(V', S^T per chunk) again from the scan's inputs: the forward scan kernel, final state discarded."""
    B, H, n = W.shape[:3]
    dev = W.device
    s0 = S0.float().contiguous() if S0 is not None else None
    Vn = torch.empty((B, H, n, 64, 128), dtype=torch.bfloat16, device=dev)
    SsT = torch.empty((B, H, n, 128, 128), dtype=torch.bfloat16, device=dev)
    Sf = torch.empty((B, H, 128, 128), dtype=torch.float32, device=dev)
    rc = nv.cuda().cvb_gdn_scan_fwd(W.data_ptr(), U.data_ptr(), Kd.data_ptr(), egam.data_ptr(), nv.ptr(s0),
                                    Sf.data_ptr(), Vn.data_ptr(), SsT.data_ptr(), B * H, n,
                                    nv.status_word(dev).data_ptr(), nv.stream())
    nv.check(rc, "cvb_gdn_scan_fwd")
    count_launch()
    return Vn, SsT


def chunk_forward(q, k, v, beta, g, S0, scale: float, keep_prep: bool = False):
    """Full chunked forward on the three kernels. Returns (o [B,T,H,128] bf16, Sf fp32, Vn, SsT, prep) where
    ``prep`` is the prep kernel's output dict (with T and the per-token scalars when ``keep_prep``)."""
    B, T, H, _ = q.shape
    n = T // 64
    dev = q.device
    pre = chunk_prep(q, k, v, beta, g, scale, want_aux=keep_prep)
    s0 = S0.float().contiguous() if S0 is not None else None
    Vn = torch.empty((B, H, n, 64, 128), dtype=torch.bfloat16, device=dev)
    SsT = torch.empty((B, H, n, 128, 128), dtype=torch.bfloat16, device=dev)
    Sf = torch.empty((B, H, 128, 128), dtype=torch.float32, device=dev)
    lib = nv.cuda()
    rc = lib.cvb_gdn_scan_fwd(pre["W"].data_ptr(), pre["U"].data_ptr(), pre["Kd"].data_ptr(), pre["egam"].data_ptr(),
                              nv.ptr(s0), Sf.data_ptr(), Vn.data_ptr(), SsT.data_ptr(), B * H, n,
                              nv.status_word(dev).data_ptr(), nv.stream())
    nv.check(rc, "cvb_gdn_scan_fwd")
    o = torch.empty((B, T, H, 128), dtype=torch.bfloat16, device=dev)
    rc = lib.cvb_gdn_chunk_out(SsT.data_ptr(), pre["Qd"].data_ptr(), Vn.data_ptr(), pre["P"].data_ptr(), o.data_ptr(),
                               B, T, H, nv.status_word(dev).data_ptr(), nv.stream())
    nv.check(rc, "cvb_gdn_chunk_out")
    count_launch(2)
    return o, Sf, Vn, SsT, pre


def chunk_backward(q, k, v, beta, scale: float, pre, Vn, SsT, Sf, do, dSf, out=None):
    """Backward of ``chunk_forward`` on two kernels: the reverse state scan and the chunk-local backward.
    ``pre`` holds the forward's prep outputs (W, Kd, Qd, P, egam, Tm, aux).  ``out`` may give three bf16
    [B,T,H,128] views with one common token stride (column ranges of a packed gradient buffer) for dq, dk, dv.
    Returns (dq, dk, dv [B,T,H,128] bf16, dbeta, dg [B,T,H] fp32, dS0 fp32)."""
    B, T, H, _ = q.shape
    n = T // 64
    dev = q.device
    lib = nv.cuda()
    st = nv.status_word(dev).data_ptr()
    do = do.to(torch.bfloat16).contiguous()
    dsf = dSf.float().contiguous() if dSf is not None else None
    dVn = torch.empty((B, H, n, 64, 128), dtype=torch.bfloat16, device=dev)
    dSnT = torch.empty((B, H, n, 128, 128), dtype=torch.bfloat16, device=dev)
    dS0 = torch.empty((B, H, 128, 128), dtype=torch.float32, device=dev)
    rc = lib.cvb_gdn_scan_bwd(pre["P"].data_ptr(), pre["Kd"].data_ptr(), pre["Qd"].data_ptr(), pre["W"].data_ptr(),
                              do.data_ptr(), pre["egam"].data_ptr(), nv.ptr(dsf), dS0.data_ptr(), dVn.data_ptr(),
                              dSnT.data_ptr(), B * H, n, H, st, nv.stream())   # dO read token-major, in place
    nv.check(rc, "cvb_gdn_scan_bwd")
    if out is None:
        dq, dk, dv = (torch.empty((B, T, H, 128), dtype=torch.bfloat16, device=dev) for _ in range(3))
        d_stride = 0
    else:
        dq, dk, dv = out
        d_stride = dq.stride(1)
        for t in out:
            assert t.dtype == torch.bfloat16 and t.shape == (B, T, H, 128) and t.stride(3) == 1 and \
                t.stride(2) == 128 and t.stride(1) == d_stride and t.stride(0) == T * d_stride, "packed dq/dk/dv layout"
    dbeta = torch.empty((B, T, H), dtype=torch.float32, device=dev)
    dg = torch.empty((B, T, H), dtype=torch.float32, device=dev)
    dgam = torch.empty((B, H, n), dtype=torch.float32, device=dev)
    bf = beta.float().contiguous()
    SsT, Vn, Sf = SsT.contiguous(), Vn.contiguous(), Sf.float().contiguous()
    rc = lib.cvb_gdn_chunk_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(1), do.data_ptr(), bf.data_ptr(),
                               pre["Tm"].data_ptr(), pre["aux"].data_ptr(), Vn.data_ptr(), dVn.data_ptr(),
                               SsT.data_ptr(), dSnT.data_ptr(), Sf.data_ptr(), dgam.data_ptr(), B, T, H, scale,
                               dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), d_stride, dbeta.data_ptr(),
                               dg.data_ptr(), st, nv.stream())
    nv.check(rc, "cvb_gdn_chunk_bwd")
    count_launch(3)
    return dq, dk, dv, dbeta, dg, dS0
