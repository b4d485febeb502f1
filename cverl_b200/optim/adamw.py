"""AdamW with fp32 state: per-tensor (``Fp32MasterAdamW``) and flat-shard (``FlatAdamW``).

Behaviour follows the reference (src/torch/fp32_master_adamw.cc:68-329):
bias-corrected Adam moments kept in fp32, decoupled weight decay
``p *= 1 - lr*wd``, optional fp32 master copy of the parameters (without it the
parameters stay in model dtype and round-trip through fp32 each step), fp32
``main_grad`` accumulation across micro-batches, device-tensor gradient norms
(no host sync), and ``load_state`` for resume.  On CUDA the update is one fused
kernel (``cuda/optim_ops.cu``); the reference issues eight elementwise ops.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..ops import optim as optim_ops


@dataclass
class AdamWOptions:
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.01
    use_master_weights: bool = True

    def validate(self, who: str) -> None:
        if self.lr < 0 or not (0 <= self.beta1 < 1) or not (0 <= self.beta2 < 1) or self.eps < 0 \
                or self.weight_decay < 0:
            raise ValueError(f"{who}: invalid AdamW options")


def clone_detached(params: Sequence[torch.Tensor]) -> List[torch.Tensor]:
    return [p.detach().clone() for p in params]


def parameter_delta_sum(before: Sequence[torch.Tensor], after: Sequence[torch.Tensor]) -> torch.Tensor:
    """Sum of absolute parameter changes as a device scalar ("did the parameters move")."""
    total = None
    for b, a in zip(before, after):
        d = (a.detach().float() - b.detach().float()).abs().sum()
        total = d if total is None else total + d
    return total if total is not None else torch.zeros(())


class FlatAdamW:
    """AdamW over ONE flat 1-D shard (reference: fp32_master_adamw.cc:270-329)."""

    def __init__(self, parameter_shard: torch.Tensor, options: AdamWOptions):
        options.validate("FlatAdamW")
        if parameter_shard.dim() != 1 or not parameter_shard.is_contiguous():
            raise ValueError("FlatAdamW: parameter shard must be a contiguous 1-D tensor")
        self.options = options
        self.model_shard = parameter_shard.detach()  # aliases the caller's storage: updated in place
        self.master = parameter_shard.detach().float().clone() if options.use_master_weights else None
        self.exp_avg = torch.zeros(parameter_shard.shape, dtype=torch.float32, device=parameter_shard.device)
        self.exp_avg_sq = torch.zeros_like(self.exp_avg)
        self.step_count = 0

    @property
    def parameter_shard(self) -> torch.Tensor:
        """The authoritative shard: fp32 master when kept, else the model-dtype shard."""
        return self.master if self.master is not None else self.model_shard

    def step(self, gradient_shard: torch.Tensor, *, clip: Optional[torch.Tensor] = None, grad_scale: float = 1.0,
             zero_grad: bool = False) -> None:
        if gradient_shard.numel() != self.model_shard.numel():
            raise ValueError("FlatAdamW.step: gradient shard shape mismatch")
        self.step_count += 1
        o = self.options
        g = gradient_shard.reshape(-1)
        if g.dtype != torch.float32:
            g = g.float()
            zero_grad = False
        optim_ops.flat_adamw_step(g, self.master, self.model_shard, self.exp_avg, self.exp_avg_sq, clip=clip,
                                  grad_scale=grad_scale, lr=o.lr, beta1=o.beta1, beta2=o.beta2, eps=o.eps,
                                  weight_decay=o.weight_decay, step=self.step_count, zero_grad=zero_grad)

    def load_state(self, parameter_value: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor,
                   step: int) -> None:
        if step < 0:
            raise ValueError("FlatAdamW.load_state: negative step")
        n = self.model_shard.numel()
        if parameter_value.numel() != n or exp_avg.numel() != n or exp_avg_sq.numel() != n:
            raise ValueError("FlatAdamW.load_state: state shape mismatch")
        dev = self.model_shard.device
        if self.master is not None:
            self.master.copy_(parameter_value.detach().to(dev, torch.float32).reshape(-1))
            self.model_shard.copy_(self.master.to(self.model_shard.dtype))
        else:
            self.model_shard.copy_(parameter_value.detach().to(dev, self.model_shard.dtype).reshape(-1))
        self.exp_avg.copy_(exp_avg.detach().to(dev, torch.float32).reshape(-1))
        self.exp_avg_sq.copy_(exp_avg_sq.detach().to(dev, torch.float32).reshape(-1))
        self.step_count = int(step)


class Fp32MasterAdamW:
    """Per-tensor AdamW with optional fp32 master weights and fp32 main-grad accumulation
    (reference: fp32_master_adamw.cc:68-268)."""

    def __init__(self, params: Sequence[torch.Tensor], options: AdamWOptions,
                 main_grads: Optional[Sequence[torch.Tensor]] = None):
        """``main_grads``: existing fp32 gradient accumulators to adopt (views of a flat gradient buffer that
        the backward kernels fill) instead of allocating one per parameter."""
        options.validate("Fp32MasterAdamW")
        self.options = options
        self.params = list(params)
        self.master = [p.detach().float().clone() if options.use_master_weights else None for p in self.params]
        self.exp_avg = [torch.zeros(p.shape, dtype=torch.float32, device=p.device) for p in self.params]
        self.exp_avg_sq = [torch.zeros(p.shape, dtype=torch.float32, device=p.device) for p in self.params]
        if main_grads is not None:
            if len(main_grads) != len(self.params) or any(g.shape != p.shape or g.dtype != torch.float32
                                                          for g, p in zip(main_grads, self.params)):
                raise ValueError("Fp32MasterAdamW: main_grads must be fp32 tensors shaped like the parameters")
            self.main_grad = list(main_grads)
        else:
            self.main_grad = [torch.zeros(p.shape, dtype=torch.float32, device=p.device) for p in self.params]
        self.has_main_grad = main_grads is not None
        self.step_count = 0

    # --- gradients -----------------------------------------------------------
    def accumulate_model_grads(self, clear_model_grads: bool = True) -> None:
        """main_grad += p.grad in fp32 (micro-batch accumulation)."""
        for p, mg in zip(self.params, self.main_grad):
            if p.grad is not None:
                mg.add_(p.grad.detach().float())
                if clear_model_grads:
                    p.grad = None
        self.has_main_grad = True

    def _grads(self) -> List[Optional[torch.Tensor]]:
        if self.has_main_grad:
            return list(self.main_grad)
        return [None if p.grad is None else p.grad.detach().float() for p in self.params]

    def grad_l2_norm_sq_tensor(self) -> torch.Tensor:
        total = None
        for g in self._grads():
            if g is None:
                continue
            s = g.pow(2).sum()
            total = s if total is None else total + s
        return total if total is not None else torch.zeros(())

    def grad_norm_sum_tensor(self) -> torch.Tensor:
        """Sum of per-tensor L2 norms (the reference's health metric)."""
        total = None
        for g in self._grads():
            if g is None:
                continue
            s = g.pow(2).sum().sqrt()
            total = s if total is None else total + s
        return total if total is not None else torch.zeros(())

    def scale_gradients(self, scale) -> None:
        """Multiply every gradient by a float or a device scalar tensor."""
        if self.has_main_grad:
            for g in self.main_grad:
                g.mul_(scale)
        else:
            for p in self.params:
                if p.grad is not None:
                    p.grad.mul_(scale if not torch.is_tensor(scale) else scale.to(p.grad.dtype))

    def zero_grad(self) -> None:
        for p, mg in zip(self.params, self.main_grad):
            p.grad = None
            mg.zero_()
        self.has_main_grad = False

    # --- update ----------------------------------------------------------------
    @torch.no_grad()
    def step(self) -> None:
        self.step_count += 1
        o = self.options
        grads = self._grads()
        for i, p in enumerate(self.params):
            g = grads[i]
            if g is None:
                continue
            model = p.data.reshape(-1)
            master = self.master[i].reshape(-1) if self.master[i] is not None else None
            optim_ops.flat_adamw_step(g.reshape(-1).contiguous(), master, model, self.exp_avg[i].reshape(-1),
                                      self.exp_avg_sq[i].reshape(-1), lr=o.lr, beta1=o.beta1, beta2=o.beta2,
                                      eps=o.eps, weight_decay=o.weight_decay, step=self.step_count)
        self.zero_grad()

    def master_or_param(self, i: int) -> torch.Tensor:
        return self.master[i] if self.master[i] is not None else self.params[i].data

    def load_state(self, param_values: Sequence[torch.Tensor], exp_avg: Sequence[torch.Tensor],
                   exp_avg_sq: Sequence[torch.Tensor], step: int) -> None:
        if step < 0 or len(param_values) != len(self.params):
            raise ValueError("Fp32MasterAdamW.load_state: bad state")
        for i, p in enumerate(self.params):
            if self.master[i] is not None:
                self.master[i].copy_(param_values[i].detach().to(p.device, torch.float32).view_as(p))
                p.data.copy_(self.master[i].to(p.dtype))
            else:
                p.data.copy_(param_values[i].detach().to(p.device, p.dtype).view_as(p))
            self.exp_avg[i].copy_(exp_avg[i].detach().to(p.device, torch.float32).view_as(p))
            self.exp_avg_sq[i].copy_(exp_avg_sq[i].detach().to(p.device, torch.float32).view_as(p))
        self.step_count = int(step)
