"""Flat-shard optimizer kernels: squared norm, clip scale, fused FlatAdamW step.

CUDA fp32 shards run ``cuda/optim_ops.cu``; CPU shards run the same update in
PyTorch ops.  Update and clip rules: src/torch/fp32_master_adamw.cc:284-308
and src/distributed/optimizer_sharding.cc:701-709 of the reference.
"""
from __future__ import annotations

import torch

from .. import _native as nv
from .gemm import count_launch


def sumsq(grad: torch.Tensor, scale: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[0] += sum((grad*scale)^2)`` as a 1-element fp32 tensor on the grad's device."""
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=grad.device)
    if grad.is_cuda and grad.dtype == torch.float32:
        g = grad.reshape(-1)
        nv.check(nv.cuda().cvb_sumsq_f32(g.data_ptr(), g.numel(), scale, out.data_ptr(), nv.stream()),
                 "cvb_sumsq_f32")
        count_launch()
    else:
        out += (grad.float() * scale).pow(2).sum()
    return out


def clip_scale(global_sq: torch.Tensor, max_norm: float) -> torch.Tensor:
    """``[scale, norm]`` with scale = max/(norm+1e-6) when norm is finite and > max, else 1."""
    clip = torch.empty(2, dtype=torch.float32, device=global_sq.device)
    if global_sq.is_cuda:
        nv.check(nv.cuda().cvb_clip_scale(global_sq.data_ptr(), float(max_norm), clip.data_ptr(), nv.stream()),
                 "cvb_clip_scale")
        count_launch()
    else:
        norm = global_sq[0].sqrt()
        s = torch.ones(())
        if max_norm > 0 and torch.isfinite(norm) and norm > max_norm:
            s = max_norm / (norm + 1.0e-6)
        clip[0], clip[1] = s, norm
    return clip


def flat_adamw_step(grad, master, model, exp_avg, exp_avg_sq, *, clip=None, grad_scale: float = 1.0, lr: float,
                    beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
                    zero_grad: bool = False) -> None:
    """One fused AdamW update of a flat shard (all tensors 1-D, same length).

    ``master`` (fp32) may be None; ``model`` is the shard in model dtype (bf16 or
    fp32) and is always rewritten; ``clip`` is an optional device scalar tensor
    multiplied into the gradient together with ``grad_scale``.
    """
    n = grad.numel()
    if grad.is_cuda and grad.dtype == torch.float32:
        model_bf16 = model if (model is not None and model.dtype == torch.bfloat16) else None
        model_f32 = model if (model is not None and model.dtype == torch.float32) else None
        if model is not None and model_bf16 is None and model_f32 is None:
            raise TypeError("flat_adamw_step: model shard must be bf16 or fp32")
        nv.check(nv.cuda().cvb_flat_adamw(grad.data_ptr(), nv.ptr(master), nv.ptr(model_bf16), nv.ptr(model_f32),
                                          exp_avg.data_ptr(), exp_avg_sq.data_ptr(), nv.ptr(clip), n, grad_scale,
                                          lr, beta1, beta2, eps, weight_decay, step, int(zero_grad), nv.stream()),
                 "cvb_flat_adamw")
        count_launch()
        return
    g = grad.float() * grad_scale
    if clip is not None:
        g = g * clip[0]
    p = master if master is not None else model.float()
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    exp_avg.mul_(beta1).add_(g, alpha=1.0 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    if weight_decay != 0.0:
        p = p.mul_(1.0 - lr * weight_decay) if master is not None else p * (1.0 - lr * weight_decay)
    denom = (exp_avg_sq / bc2).sqrt_().add_(eps)
    if master is not None:
        master.addcdiv_(exp_avg, denom, value=-lr / bc1)
        if model is not None:
            model.copy_(master.to(model.dtype))
    else:
        p = p.addcdiv(exp_avg, denom, value=-lr / bc1)
        model.copy_(p.to(model.dtype))
    if zero_grad:
        grad.zero_()
