"""MoE router: logits GEMM (tcgen05, fp32 epilogue) + fused top-k / softmax kernel with its backward.

``route(x, gate_w, top_k, norm_topk_prob) -> (expert ids [T, k] int64, weights [T, k] fp32)``.
On CUDA bf16 inputs the selection and both softmax variants run in ``cuda/router_ops.cu`` (one warp
per token); elsewhere the PyTorch statement below is used, which is also the test oracle.
Reference: src/model/qwen3_5_text.cc:713-760.
"""
from __future__ import annotations

from typing import Tuple

import torch

from .. import _native as nv
from . import gemm as G


def route_ref(x: torch.Tensor, gate_w: torch.Tensor, top_k: int, norm_topk_prob: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    logits = x.float() @ gate_w.float().t()
    top_val, top_idx = logits.topk(top_k, dim=-1)
    if norm_topk_prob:
        w = torch.softmax(top_val, dim=-1)
    else:
        w = torch.softmax(logits, dim=-1).gather(-1, top_idx)
    return top_idx, w


class _Route(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate_w, top_k, norm_topk):
        T, E = x.shape[0], gate_w.shape[0]
        logits = G.gemm_nt(x, gate_w, out_dtype=torch.float32)
        if not logits.is_contiguous():
            logits = logits.contiguous()
        idx = torch.empty((T, top_k), dtype=torch.int64, device=x.device)
        w = torch.empty((T, top_k), dtype=torch.float32, device=x.device)
        nv.check(nv.cuda().cvb_router_topk_fwd(logits.data_ptr(), T, E, top_k, int(norm_topk), idx.data_ptr(),
                                               w.data_ptr(), nv.stream()), "cvb_router_topk_fwd")
        G.count_launch()
        ctx.save_for_backward(x, gate_w, logits, idx, w)
        ctx.cfg = (top_k, norm_topk)
        ctx.mark_non_differentiable(idx)
        return idx, w

    @staticmethod
    def backward(ctx, _didx, dw):
        x, gate_w, logits, idx, w = ctx.saved_tensors
        top_k, norm_topk = ctx.cfg
        T, E = logits.shape
        dlogits = torch.empty_like(logits)
        nv.check(nv.cuda().cvb_router_topk_bwd(logits.data_ptr(), idx.data_ptr(), w.data_ptr(),
                                               dw.float().contiguous().data_ptr(), T, E, top_k, int(norm_topk),
                                               dlogits.data_ptr(), nv.stream()), "cvb_router_topk_bwd")
        G.count_launch()
        dl = dlogits.to(torch.bfloat16)
        dx = G.gemm_nn(dl, gate_w) if ctx.needs_input_grad[0] else None
        dgw = None
        if ctx.needs_input_grad[1]:
            main_grad = getattr(gate_w, "main_grad", None)
            if main_grad is not None:
                G.gemm_tn_acc(dl, x, main_grad)
            else:
                acc = torch.zeros(gate_w.shape, dtype=torch.float32, device=x.device)
                G.gemm_tn_acc(dl, x, acc)
                dgw = acc.to(gate_w.dtype)
        return dx, dgw, None, None


def route(x: torch.Tensor, gate_w: torch.Tensor, top_k: int, norm_topk_prob: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    E = gate_w.shape[0]
    if G.use_native(x) and gate_w.dtype == torch.bfloat16 and E <= 256 and top_k <= 32 and E % 8 == 0:
        return _Route.apply(x.contiguous(), gate_w, top_k, bool(norm_topk_prob))
    return route_ref(x, gate_w, top_k, norm_topk_prob)
