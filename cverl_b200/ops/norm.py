"""RMSNorm family: residual-add + RMSNorm, gated RMSNorm, q/k head norm + RoPE.

CUDA bf16 tensors run ``cuda/norm_ops.cu``; everything else runs the fp32
PyTorch statement of the same math (``*_ref``), which is also the test oracle.
Weight gradients go to ``w.main_grad`` (fp32) when the parameter has one.
Reference math: src/model/qwen3_5_text.cc:698-711, :724-757, :1057-1066.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _native as nv
from .gemm import count_launch


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16


def _wgrad(w: torch.Tensor, dw32: torch.Tensor):
    """Route an fp32 weight gradient: accumulate into main_grad or hand it to autograd."""
    mg = getattr(w, "main_grad", None)
    if mg is not None:
        mg.add_(dw32.view_as(mg))
        return None
    return dw32.to(w.dtype).view_as(w)


def _wgrad_buffer(w: torch.Tensor):
    """fp32 buffer the backward kernel accumulates into, and whether it is the main_grad itself."""
    mg = getattr(w, "main_grad", None)
    if mg is not None:
        return mg, True
    return torch.zeros(w.shape, dtype=torch.float32, device=w.device), False


# ----------------------------------------------------------------------------
# reference math
# ----------------------------------------------------------------------------
def rmsnorm_ref(x, w, eps: float, w_offset: float, gate=None):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (w_offset + w.float())
    if gate is not None:
        y = y * F.silu(gate.float())
    return y.to(x.dtype)


def rope_tables(max_pos: int, rot: int, theta: float, device, offset: int = 0):
    """fp32 cos/sin tables [max_pos, rot/2] for positions offset .. offset+max_pos-1."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32, device=device) / rot))
    pos = torch.arange(offset, offset + max_pos, dtype=torch.float32, device=device)
    ang = torch.outer(pos, inv_freq)
    return ang.cos().contiguous(), ang.sin().contiguous()


def apply_rope_ref(x, cos, sin, positions, rot: int):
    """x [T, heads, D]; rotate_half on the first ``rot`` dims."""
    half = rot // 2
    c = cos[positions].unsqueeze(1)  # [T,1,half]
    s = sin[positions].unsqueeze(1)
    xf = x.float()
    x1, x2, rest = xf[..., :half], xf[..., half:rot], xf[..., rot:]
    o1 = x1 * c - x2 * s
    o2 = x2 * c + x1 * s
    return torch.cat([o1, o2, rest], dim=-1).to(x.dtype)


def headnorm_rope_ref(x, w, cos, sin, positions, rot, eps, w_offset, use_norm=True):
    y = rmsnorm_ref(x, w, eps, w_offset) if use_norm else x
    if rot > 0:
        y = apply_rope_ref(y, cos, sin, positions, rot)
    return y


# ----------------------------------------------------------------------------
# residual add + RMSNorm
# ----------------------------------------------------------------------------
class _AddRmsNorm(torch.autograd.Function):
    """h = x + resid (resid optional); y = rmsnorm(h). Returns (y, h)."""

    @staticmethod
    def forward(ctx, x, resid, w, eps, w_offset):
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        rows = x2.shape[0]
        if x2.stride(1) != 1 or x2.stride(0) % 8:
            x2 = x2.contiguous()
        y = torch.empty((rows, D), dtype=x.dtype, device=x.device)
        h = torch.empty((rows, D), dtype=x.dtype, device=x.device) if resid is not None else None
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        r2 = resid.reshape(-1, D).contiguous() if resid is not None else None
        rc = nv.cuda().cvb_rmsnorm_fwd(x2.data_ptr(), nv.ptr(r2), w.data_ptr(), None, y.data_ptr(), nv.ptr(h),
                                       rstd.data_ptr(), rows, D, x2.stride(0), 0, eps, w_offset, 0, 0, nv.stream())
        nv.check(rc, "cvb_rmsnorm_fwd")
        count_launch()
        hh = h if h is not None else x2
        ctx.save_for_backward(hh, w, rstd)
        ctx.w_offset = w_offset
        ctx.has_resid = resid is not None
        ctx.shape = x.shape
        if h is None:
            return y.view(x.shape)
        return y.view(x.shape), h.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dh=None):
        h, w, rstd = ctx.saved_tensors
        D = h.shape[-1]
        rows = h.shape[0]
        dy2 = dy.reshape(-1, D).contiguous()
        dres = dh.reshape(-1, D).contiguous() if dh is not None else None
        dx = torch.empty((rows, D), dtype=h.dtype, device=h.device)
        dwbuf, is_main = _wgrad_buffer(w)
        rc = nv.cuda().cvb_rmsnorm_bwd(dy2.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), None,
                                       nv.ptr(dres), dx.data_ptr(), None, dwbuf.data_ptr(), rows, D,
                                       h.stride(0), 0, D, ctx.w_offset, 0, 0, 0, 0, nv.stream())
        nv.check(rc, "cvb_rmsnorm_bwd")
        count_launch()
        dxv = dx.view(ctx.shape)
        dw = None if is_main else dwbuf.to(w.dtype)
        return dxv, (dxv if ctx.has_resid else None), dw, None, None


def add_rmsnorm(x, resid, w, eps: float = 1e-6, w_offset: float = 1.0):
    """Returns ``(rmsnorm(x + resid), x + resid)``; ``resid`` may be None."""
    if _native(x):
        if resid is None:
            return _AddRmsNorm.apply(x, None, w, eps, w_offset), x
        return _AddRmsNorm.apply(x, resid, w, eps, w_offset)
    h = x if resid is None else (x.float() + resid.float()).to(x.dtype)
    return rmsnorm_ref(h, w, eps, w_offset), h


def rmsnorm(x, w, eps: float = 1e-6, w_offset: float = 1.0):
    return add_rmsnorm(x, None, w, eps, w_offset)[0]


# ----------------------------------------------------------------------------
# gated RMSNorm: y = rmsnorm(x) * w * silu(z)   (rows = tokens*heads, D = head dim)
# ----------------------------------------------------------------------------
def _gate_layout(z, rows, D):
    """(tensor to read, row stride, block, block stride) for the gate of a [rows, D] gated norm.  A column range
    of a wider [tokens, width] tensor (the z group of the linear-attention projection) is read in place: its rows
    are (token, head) pairs, ``block`` heads per token."""
    if z.dim() >= 2 and z.stride(-1) == 1 and z.shape[-1] % D == 0 and z.shape[-1] != D:
        z2 = z.reshape(-1, z.shape[-1]) if z.dim() != 2 else z
        heads = z2.shape[1] // D
        if (z2.shape[0] * heads == rows and z2.stride(1) == 1 and z2.stride(0) % 8 == 0 and z2.data_ptr() % 16 == 0
                and z2.data_ptr() == z.data_ptr()):
            return z2, D, heads, z2.stride(0)
    z2 = z.reshape(-1, D)
    if z2.stride(1) != 1 or z2.stride(0) % 8:
        z2 = z2.contiguous()
    return z2, z2.stride(0), 0, 0


class _GatedRmsNorm(torch.autograd.Function):
    """y = rmsnorm(x) * w * silu(z).  ``z`` is [..., D] like ``x`` or [tokens..., heads * D] (a column range of
    the projection output, read in place).  If ``z`` carries ``_grad_sink`` (set by ``conv1d_silu_split``) its
    gradient is written straight into that op's projection-gradient buffer."""

    @staticmethod
    def forward(ctx, x, z, w, eps, sink):
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        if x2.stride(1) != 1 or x2.stride(0) % 8:
            x2 = x2.contiguous()
        rows = x2.shape[0]
        z2, zs, zb, zbs = _gate_layout(z, rows, D)
        y = torch.empty((rows, D), dtype=x.dtype, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        rc = nv.cuda().cvb_rmsnorm_fwd(x2.data_ptr(), None, w.data_ptr(), z2.data_ptr(), y.data_ptr(), None,
                                       rstd.data_ptr(), rows, D, x2.stride(0), zs, eps, 0.0, zb, zbs, nv.stream())
        nv.check(rc, "cvb_rmsnorm_fwd(gated)")
        count_launch()
        ctx.save_for_backward(x2, z2, w, rstd)
        ctx.xshape, ctx.zshape = x.shape, z.shape
        ctx.zlayout = (zs, zb, zbs)
        ctx.sink = sink
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, z2, w, rstd = ctx.saved_tensors
        rows, D = x2.shape
        zs, zb, zbs = ctx.zlayout
        dy2 = dy.reshape(-1, D).contiguous()
        dx = torch.empty((rows, D), dtype=x2.dtype, device=x2.device)
        dz = None
        if zb > 0 and ctx.sink is not None:
            dz = ctx.sink[0].view_for(ctx.sink[1], ctx.zshape)      # a column range of the projection gradient
        if dz is not None:
            ds, dbs = D, dz.reshape(-1, dz.shape[-1]).stride(0)
        elif zb > 0:
            dz = torch.empty(ctx.zshape, dtype=x2.dtype, device=x2.device)
            ds, dbs = D, zb * D
        else:
            dz = torch.empty((rows, D), dtype=x2.dtype, device=x2.device)
            ds, dbs = D, 0
        dwbuf, is_main = _wgrad_buffer(w)
        rc = nv.cuda().cvb_rmsnorm_bwd(dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                       z2.data_ptr(), None, dx.data_ptr(), dz.data_ptr(), dwbuf.data_ptr(),
                                       rows, D, x2.stride(0), zs, D, 0.0, zb, zbs, ds, dbs, nv.stream())
        nv.check(rc, "cvb_rmsnorm_bwd(gated)")
        count_launch()
        dw = None if is_main else dwbuf.to(w.dtype)
        return dx.view(ctx.xshape), (dz if zb > 0 else dz.view(ctx.zshape)), dw, None, None


def gated_rmsnorm(x, z, w, eps: float = 1e-6):
    if _native(x):
        return _GatedRmsNorm.apply(x, z, w, eps, getattr(z, "_grad_sink", None))
    if z.shape != x.shape:
        z = z.reshape(x.shape)
    return rmsnorm_ref(x, w, eps, 0.0, gate=z)


# ----------------------------------------------------------------------------
# per-head RMSNorm + partial RoPE on a [T, heads, D] view (may be strided)
# ----------------------------------------------------------------------------
class _HeadNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, cos, sin, positions, rot, eps, w_offset, use_norm):
        T, Hh, D = x.shape
        assert x.stride(2) == 1
        y = torch.empty((T, Hh, D), dtype=x.dtype, device=x.device)
        rstd = torch.empty(T * Hh, dtype=torch.float32, device=x.device)
        wp = w.data_ptr() if w is not None else None
        rc = nv.cuda().cvb_headnorm_rope_fwd(x.data_ptr(), wp, positions.data_ptr(), y.data_ptr(),
                                             rstd.data_ptr(), T, Hh, D, x.stride(0), x.stride(1), rot,
                                             nv.ptr(cos), nv.ptr(sin), 1, eps, w_offset, int(use_norm),
                                             nv.stream())
        nv.check(rc, "cvb_headnorm_rope_fwd")
        count_launch()
        ctx.save_for_backward(x, w if w is not None else x.new_zeros(1), rstd, cos if cos is not None else rstd,
                              sin if sin is not None else rstd, positions)
        ctx.cfg = (rot, w_offset, use_norm, w is not None)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd, cos, sin, positions = ctx.saved_tensors
        rot, w_offset, use_norm, has_w = ctx.cfg
        T, Hh, D = x.shape
        dy = dy.contiguous()
        dx = torch.empty((T, Hh, D), dtype=x.dtype, device=x.device)
        dwbuf, is_main = (None, True)
        if use_norm:
            dwbuf, is_main = _wgrad_buffer(w)
        # x is read with its own strides, dx is written densely as [T, heads, D]
        rc = nv.cuda().cvb_headnorm_rope_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                             positions.data_ptr(), dx.data_ptr(), nv.ptr(dwbuf), T, Hh, D,
                                             x.stride(0), x.stride(1), rot,
                                             cos.data_ptr() if rot > 0 else None,
                                             sin.data_ptr() if rot > 0 else None, 1, w_offset, int(use_norm),
                                             nv.stream())
        nv.check(rc, "cvb_headnorm_rope_bwd")
        count_launch()
        dw = None
        if use_norm and not is_main:
            dw = dwbuf.to(w.dtype)
        return dx, dw, None, None, None, None, None, None, None


def headnorm_rope(x, w, cos, sin, positions, rot: int, eps: float = 1e-6, w_offset: float = 1.0,
                  use_norm: bool = True):
    """x [T, heads, D] -> per-head RMSNorm (optional) then rotary on the first ``rot`` dims."""
    if _native(x):
        pos32 = positions if positions.dtype == torch.int32 else positions.to(torch.int32)
        return _HeadNormRope.apply(x, w, cos, sin, pos32, rot, eps, w_offset, use_norm)
    return headnorm_rope_ref(x, w, cos, sin, positions.long(), rot, eps, w_offset, use_norm)
