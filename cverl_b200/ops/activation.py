"""SwiGLU, sigmoid output gate, causal depthwise conv1d + SiLU, embedding.

CUDA bf16 tensors run ``cuda/elementwise_ops.cu``; other tensors run the fp32
PyTorch statement of the same math, which is the oracle of the tests.
Reference math: src/model/qwen3_5_text.cc:791-793, :1077-1079, :1241-1243, :692.
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from .. import _native as nv
from .gemm import count_launch
from .norm import _wgrad_buffer


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16


def _rows2d(t: torch.Tensor) -> torch.Tensor:
    t2 = t.reshape(-1, t.shape[-1])
    if t2.stride(1) != 1 or t2.stride(0) % 8 or t2.data_ptr() % 16:
        t2 = t2.contiguous()
    return t2


# ------------------------------ SwiGLU --------------------------------------
def swiglu_ref(gu: torch.Tensor) -> torch.Tensor:
    g, u = gu.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gu.dtype)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        gu2 = _rows2d(gu)
        rows, two_i = gu2.shape
        inter = two_i // 2
        y = torch.empty((rows, inter), dtype=gu.dtype, device=gu.device)
        nv.check(nv.cuda().cvb_swiglu_fwd(gu2.data_ptr(), y.data_ptr(), rows, inter, gu2.stride(0), nv.stream()),
                 "cvb_swiglu_fwd")
        count_launch()
        ctx.save_for_backward(gu2)
        ctx.shape = gu.shape
        return y.view(*gu.shape[:-1], inter)

    @staticmethod
    def backward(ctx, dy):
        (gu2,) = ctx.saved_tensors
        rows, two_i = gu2.shape
        inter = two_i // 2
        dy2 = dy.reshape(rows, inter).contiguous()
        dgu = torch.empty((rows, two_i), dtype=gu2.dtype, device=gu2.device)
        nv.check(nv.cuda().cvb_swiglu_bwd(dy2.data_ptr(), gu2.data_ptr(), dgu.data_ptr(), rows, inter,
                                          gu2.stride(0), nv.stream()), "cvb_swiglu_bwd")
        count_launch()
        return dgu.view(ctx.shape)


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    """``silu(gu[..., :I]) * gu[..., I:]``"""
    if _native(gu) and (gu.shape[-1] // 2) % 8 == 0:
        return _SwiGLU.apply(gu)
    return swiglu_ref(gu)


# --------------------------- sigmoid output gate ----------------------------
def siggate_ref(a, g):
    return (a.float() * torch.sigmoid(g.float())).to(a.dtype)


class _SigGate(torch.autograd.Function):
    """y = a * sigmoid(g) on [T, heads, D] views (unit inner stride)."""

    @staticmethod
    def forward(ctx, a, g):
        T, Hh, D = a.shape
        a_d = a if (a.stride(2) == 1 and a.stride(1) == D and a.stride(0) % 8 == 0) else a.contiguous()
        g_ok = g.stride(2) == 1 and g.stride(0) % 8 == 0 and g.stride(1) % 8 == 0
        g_d = g if g_ok else g.contiguous()
        y = torch.empty((T, Hh * D), dtype=a.dtype, device=a.device)
        nv.check(nv.cuda().cvb_siggate_fwd(a_d.data_ptr(), g_d.data_ptr(), y.data_ptr(), T, Hh * D,
                                           a_d.stride(0), g_d.stride(0), D, g_d.stride(1), nv.stream()),
                 "cvb_siggate_fwd")
        count_launch()
        ctx.save_for_backward(a_d, g_d)
        return y.view(T, Hh, D)

    @staticmethod
    def backward(ctx, dy):
        a_d, g_d = ctx.saved_tensors
        T, Hh, D = a_d.shape
        dy2 = dy.reshape(T, Hh * D).contiguous()
        da = torch.empty((T, Hh, D), dtype=a_d.dtype, device=a_d.device)
        dg = torch.empty((T, Hh, D), dtype=a_d.dtype, device=a_d.device)
        nv.check(nv.cuda().cvb_siggate_bwd(dy2.data_ptr(), a_d.data_ptr(), g_d.data_ptr(), da.data_ptr(),
                                           dg.data_ptr(), T, Hh * D, a_d.stride(0), g_d.stride(0), D,
                                           g_d.stride(1), Hh * D, Hh * D, D, nv.stream()), "cvb_siggate_bwd")
        count_launch()
        return da, dg


def siggate(a: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """``a * sigmoid(g)`` for [T, heads, D] tensors."""
    if _native(a) and a.shape[-1] % 8 == 0:
        return _SigGate.apply(a, g)
    return siggate_ref(a, g)


# ---------------------- causal depthwise conv1d + SiLU ----------------------
def conv1d_silu_ref(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [B,S,C], w [C,K]: y[b,s,c] = silu(sum_j w[c,j] x[b,s-(K-1)+j,c])."""
    B, S, Cc = x.shape
    K = w.shape[1]
    xt = x.float().transpose(1, 2)
    y = F.conv1d(xt, w.float().unsqueeze(1), padding=K - 1, groups=Cc)[..., :S]
    return F.silu(y).transpose(1, 2).to(x.dtype)


class _ConvSilu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        B, S, Cc = x.shape
        x3 = x if (x.stride(2) == 1 and x.stride(1) % 8 == 0 and x.stride(0) == S * x.stride(1)
                   and x.data_ptr() % 16 == 0) else x.contiguous()
        wc = w.contiguous()
        y = torch.empty((B, S, Cc), dtype=x.dtype, device=x.device)
        nv.check(nv.cuda().cvb_conv1d_silu_fwd(x3.data_ptr(), wc.data_ptr(), y.data_ptr(), B, S, Cc, wc.shape[1],
                                               x3.stride(1), nv.stream()), "cvb_conv1d_silu_fwd")
        count_launch()
        ctx.save_for_backward(x3, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        x3, w = ctx.saved_tensors
        B, S, Cc = x3.shape
        dx = torch.empty((B, S, Cc), dtype=x3.dtype, device=x3.device)
        dw = _conv_bwd_launch(dy, x3, w, dx)
        return dx, dw


def _conv_bwd_launch(dy, x3, w, dx):
    """Runs the convolution backward: ``x3`` [B,S,C] and ``dx`` [B,S,C] may be column ranges of wider tensors
    (unit inner stride, row strides multiples of 8).  Returns the weight gradient, or None when it was
    accumulated into the weight's fp32 main gradient."""
    B, S, Cc = x3.shape
    wc = w.contiguous()
    dy = dy.contiguous()
    dwbuf, is_main = _wgrad_buffer(w)
    # the TMA-tiled kernel answers -2 for layouts it does not take (C not a multiple of 64, odd strides)
    rc = -2
    if os.environ.get("CVERL_B200_CONV_BWD", "tma") == "tma":
        rc = nv.cuda().cvb_conv1d_silu_bwd_tma(dy.data_ptr(), x3.data_ptr(), wc.data_ptr(), dx.data_ptr(),
                                               dwbuf.data_ptr(), B, S, Cc, wc.shape[1], x3.stride(1), dx.stride(1),
                                               nv.status_word(x3.device).data_ptr(), nv.stream())
    if rc == -2:
        rc = nv.cuda().cvb_conv1d_silu_bwd(dy.data_ptr(), x3.data_ptr(), wc.data_ptr(), dx.data_ptr(),
                                           dwbuf.data_ptr(), B, S, Cc, wc.shape[1], x3.stride(1), dx.stride(1),
                                           nv.stream())
    nv.check(rc, "cvb_conv1d_silu_bwd")
    count_launch()
    return None if is_main else dwbuf.to(w.dtype)


class _GradSink:
    """The [B,S,W] projection-gradient buffer of one ``_ConvSiluSplit`` node, created by whoever needs it first
    in the backward pass: a consumer of one of the passed-through column groups may write its gradient straight
    into the group's columns (``view_for``) instead of returning a tensor that is copied there later."""

    def __init__(self, shape, dtype, device, sizes):
        self.shape, self.dtype, self.device, self.sizes = shape, dtype, device, sizes
        self.buf = None

    def buffer(self):
        if self.buf is None:
            self.buf = torch.empty(self.shape, dtype=self.dtype, device=self.device)
        return self.buf

    def columns(self, group):
        at = sum(self.sizes[:group])
        return self.buffer()[..., at:at + self.sizes[group]]

    def view_for(self, group, shape):
        v = self.columns(group)
        return v if tuple(v.shape) == tuple(shape) else None


class _ConvSiluSplit(torch.autograd.Function):
    """``proj`` [B,S,W] = [x | r1 | r2 ...]: returns (conv1d_silu(x), r1, r2, ...) with the r's as views.  The
    backward writes the convolution's input gradient straight into the first columns of one [B,S,W] buffer and
    copies the other gradients beside it, instead of concatenating W columns."""

    @staticmethod
    def forward(ctx, proj, w, *sizes):
        B, S, W = proj.shape
        Cc = sizes[0]
        x3 = proj[..., :Cc]
        y = torch.empty((B, S, Cc), dtype=proj.dtype, device=proj.device)
        nv.check(nv.cuda().cvb_conv1d_silu_fwd(x3.data_ptr(), w.contiguous().data_ptr(), y.data_ptr(), B, S, Cc,
                                               w.shape[1], W, nv.stream()), "cvb_conv1d_silu_fwd")
        count_launch()
        ctx.save_for_backward(proj, w)
        ctx.sizes = sizes
        ctx.sink = _GradSink(proj.shape, proj.dtype, proj.device, sizes)
        rest, at = [], Cc
        for n in sizes[1:]:
            rest.append(proj[..., at:at + n])
            at += n
        return (y, *rest)

    @staticmethod
    def backward(ctx, dy, *drest):
        proj, w = ctx.saved_tensors
        sizes = ctx.sizes
        Cc = sizes[0]
        dproj = ctx.sink.buffer()
        ctx.sink.buf = None   # a second backward through this node gets a fresh buffer
        dw = _conv_bwd_launch(dy, proj[..., :Cc], w, dproj[..., :Cc])
        at = Cc
        for n, d in zip(sizes[1:], drest):
            dst = dproj[..., at:at + n]
            if d is None:
                dst.zero_()
            elif not (d.data_ptr() == dst.data_ptr() and d.stride() == dst.stride() and d.shape == dst.shape):
                dst.copy_(d)  # (a consumer that wrote through the sink returns this very view: nothing to copy)
            at += n
        return (dproj, dw, *([None] * len(sizes)))


def conv1d_silu(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    if _native(x) and x.shape[-1] % 8 == 0 and w.shape[1] in (2, 3, 4):
        return _ConvSilu.apply(x, w)
    return conv1d_silu_ref(x, w)


def conv1d_silu_split(proj: torch.Tensor, w: torch.Tensor, sizes):
    """``proj`` [B,S,sum(sizes)]: conv1d + SiLU on the first ``sizes[0]`` columns, the other column groups are
    returned unchanged: ``(y, r1, r2, ...)``.  Same values and gradients as splitting first."""
    sizes = tuple(int(s) for s in sizes)
    if (_native(proj) and proj.is_contiguous() and sizes[0] % 8 == 0 and proj.shape[-1] % 8 == 0
            and w.shape[1] in (2, 3, 4) and proj.data_ptr() % 16 == 0):
        outs = _ConvSiluSplit.apply(proj, w, *sizes)
        node = outs[0].grad_fn
        if node is not None and hasattr(node, "sink"):
            for g, r in enumerate(outs[1:], start=1):
                r._grad_sink = (node.sink, g)
        return outs
    parts = proj.split(list(sizes), dim=-1)
    return (conv1d_silu(parts[0], w), *parts[1:])


# ------------------------------- embedding ----------------------------------
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, vocab_lo):
        flat = ids.reshape(-1).contiguous()
        T, H = flat.numel(), table.shape[1]
        out = torch.empty((T, H), dtype=table.dtype, device=table.device)
        nv.check(nv.cuda().cvb_embedding_fwd(flat.data_ptr(), table.data_ptr(), out.data_ptr(), T, H, vocab_lo,
                                             vocab_lo + table.shape[0], nv.stream()), "cvb_embedding_fwd")
        count_launch()
        ctx.save_for_backward(flat, table)
        ctx.vocab_lo = vocab_lo
        ctx.ids_shape = ids.shape
        return out.view(*ids.shape, H)

    @staticmethod
    def backward(ctx, dout):
        flat, table = ctx.saved_tensors
        T, H = flat.numel(), table.shape[1]
        d2 = dout.reshape(T, H).contiguous()
        dwbuf, is_main = _wgrad_buffer(table)
        nv.check(nv.cuda().cvb_embedding_bwd(flat.data_ptr(), d2.data_ptr(), dwbuf.data_ptr(), T, H, ctx.vocab_lo,
                                             ctx.vocab_lo + table.shape[0], nv.stream()), "cvb_embedding_bwd")
        count_launch()
        return None, (None if is_main else dwbuf.to(table.dtype)), None


def embedding(ids: torch.Tensor, table: torch.Tensor, vocab_lo: int = 0) -> torch.Tensor:
    """Row gather; ids outside ``[vocab_lo, vocab_lo + rows)`` give zeros (vocab-parallel shards)."""
    if _native(table) and table.shape[1] % 8 == 0:
        return _Embedding.apply(ids.long(), table, vocab_lo)
    local = ids.long() - vocab_lo
    ok = (local >= 0) & (local < table.shape[0])
    out = F.embedding(local.clamp(0, table.shape[0] - 1), table)
    return out * ok.unsqueeze(-1).to(out.dtype)
