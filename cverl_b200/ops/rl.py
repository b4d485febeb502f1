"""RL math: masked reductions, KL penalties, GAE, GRPO advantages, PPO loss.

Three interchangeable implementations of one contract
(reference: src/torch/core_algos_torch.cc:9-193):

* ``*_torch``   differentiable PyTorch statements (oracle of the tests; used
                when a caller wants autograd through the loss),
* ``c_abi.*``   the public C ABI served by ``libcverl.so`` on CPU fp32 buffers,
* ``fused_*``   sm_100a kernels on CUDA fp32 tensors (``cuda/rl_loss.cu``); the
                PPO kernel returns the loss metrics and d(loss)/d(log_prob) in
                one pass so that the trainer never builds an autograd graph for
                the loss.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

from typing import Optional

import torch

from .. import _native as nv
from .gemm import count_launch

EPS = 1.0e-8
AGG_TOKEN_MEAN, AGG_SEQ_MEAN_TOKEN_SUM, AGG_SEQ_MEAN_TOKEN_MEAN = 0, 1, 2
KL_K1, KL_ABS, KL_K2, KL_K3 = 0, 1, 2, 3
_KL_NAMES = {"k1": KL_K1, "kl": KL_K1, "abs": KL_ABS, "k2": KL_K2, "mse": KL_K2, "k3": KL_K3, "low_var_kl": KL_K3}
_AGG_NAMES = {"token-mean": 0, "token_mean": 0, "seq-mean-token-sum": 1, "seq_mean_token_sum": 1,
              "seq-mean-token-mean": 2, "seq_mean_token_mean": 2}


def kl_kind(name) -> int:
    return name if isinstance(name, int) else _KL_NAMES[name]


def agg_mode(name) -> int:
    return name if isinstance(name, int) else _AGG_NAMES[name]


# ----------------------------------------------------------------------------
# differentiable PyTorch statements
# ----------------------------------------------------------------------------
def masked_sum(values, mask):
    return (values * mask.to(values.dtype)).sum()


def masked_mean(values, mask):
    return masked_sum(values, mask) / (mask.sum() + EPS)


def masked_whiten(values, mask, shift_mean: bool = True):
    mean = masked_mean(values, mask)
    centered = values - mean
    var = masked_mean(centered.pow(2), mask)
    msum = mask.sum()
    var = var * msum / (msum - 1.0)
    out = centered * torch.rsqrt(var + EPS)
    return out if shift_mean else out + mean


def kl_penalty(logprob, ref_logprob, penalty="k1"):
    kind = kl_kind(penalty)
    diff = logprob - ref_logprob
    if kind == KL_K1:
        return diff
    if kind == KL_ABS:
        return diff.abs()
    if kind == KL_K2:
        return 0.5 * diff.square()
    kl = torch.clamp(ref_logprob - logprob, -20.0, 20.0)
    return torch.clamp(torch.exp(kl) - kl - 1.0, -10.0, 10.0)


@torch.no_grad()
def gae_advantage_return(token_level_rewards, values, response_mask, gamma: float, lam: float):
    """Returns ``(whitened advantages, returns)``."""
    rows, cols = token_level_rewards.shape
    adv = torch.empty_like(token_level_rewards)
    next_value = token_level_rewards.new_zeros(rows)
    last = token_level_rewards.new_zeros(rows)
    for c in range(cols - 1, -1, -1):
        m = response_mask[:, c]
        delta = token_level_rewards[:, c] + gamma * next_value - values[:, c]
        cand = delta + gamma * lam * last
        next_value = values[:, c] * m + (1.0 - m) * next_value
        last = cand * m + (1.0 - m) * last
        adv[:, c] = last
    return masked_whiten(adv, response_mask), adv + values


@torch.no_grad()
def grpo_outcome_advantage(token_level_rewards, response_mask, group_ids, epsilon: float = 1e-6,
                           norm_adv_by_std: bool = True):
    """Returns ``(advantages, returns)`` (identical tensors, as in the reference)."""
    scores = token_level_rewards.sum(-1)
    _, inverse, counts = torch.unique(group_ids.to(scores.device).long(), sorted=True, return_inverse=True,
                                      return_counts=True)
    cnt = counts.to(scores.dtype)
    sums = torch.zeros_like(cnt).index_add_(0, inverse, scores)
    means = torch.where(cnt > 1, sums / cnt.clamp_min(1.0), torch.zeros_like(sums))
    scal = scores - means[inverse]
    if norm_adv_by_std:
        sq = torch.zeros_like(cnt).index_add_(0, inverse, scal.square())
        std = torch.where(cnt > 1, torch.sqrt(sq / (cnt - 1.0).clamp_min(1.0)), torch.ones_like(sq))
        scal = scal / (std[inverse] + epsilon)
    adv = scal.unsqueeze(-1) * response_mask
    return adv, adv


def aggregate_loss(loss_mat, loss_mask, mode=AGG_TOKEN_MEAN):
    mode = agg_mode(mode)
    if mode == AGG_TOKEN_MEAN:
        return masked_sum(loss_mat, loss_mask) / (loss_mask.sum() + EPS)
    cnt = loss_mask.sum(-1)
    seq_mask = (cnt > 0).to(loss_mat.dtype)
    seq_losses = (loss_mat * loss_mask).sum(-1)
    if mode == AGG_SEQ_MEAN_TOKEN_MEAN:
        seq_losses = seq_losses / (cnt + EPS)
    return masked_sum(seq_losses, seq_mask) / (seq_mask.sum() + EPS)


@dataclass
class PpoLossResult:
    pg_loss: torch.Tensor
    pg_clipfrac: torch.Tensor
    ppo_kl: torch.Tensor
    pg_clipfrac_lower: torch.Tensor


def ppo_clipped_loss(old_log_prob, log_prob, advantages, response_mask, clip_ratio: float = 0.2,
                     clip_ratio_low: float = -1.0, clip_ratio_high: float = -1.0, clip_ratio_c: float = 3.0,
                     agg=AGG_TOKEN_MEAN) -> PpoLossResult:
    if not clip_ratio_c > 1.0:
        raise ValueError("clip_ratio_c must be > 1.0")
    lo = clip_ratio if clip_ratio_low < 0 else clip_ratio_low
    hi = clip_ratio if clip_ratio_high < 0 else clip_ratio_high
    nak = torch.clamp(log_prob - old_log_prob, -20.0, 20.0)
    ratio = torch.exp(nak)
    ppo_kl = masked_mean(-nak, response_mask)
    l1 = -advantages * ratio
    l2 = -advantages * torch.clamp(ratio, 1.0 - lo, 1.0 + hi)
    m1 = torch.maximum(l1, l2)
    clipfrac = masked_mean((l2 > l1).to(response_mask.dtype), response_mask)
    l3 = -advantages * clip_ratio_c
    m2 = torch.minimum(l3, m1)
    lower = masked_mean(((m1 > l3) & (advantages < 0)).to(response_mask.dtype), response_mask)
    losses = torch.where(advantages < 0, m2, m1)
    return PpoLossResult(aggregate_loss(losses, response_mask, agg), clipfrac, ppo_kl, lower)


# ----------------------------------------------------------------------------
# public C ABI through ctypes (CPU fp32)
# ----------------------------------------------------------------------------
class _T2(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int), ("device", C.c_int), ("rows", C.c_int64),
                ("cols", C.c_int64)]


class _PpoOut(C.Structure):
    _fields_ = [("pg_loss", C.c_float), ("pg_clipfrac", C.c_float), ("ppo_kl", C.c_float),
                ("pg_clipfrac_lower", C.c_float)]


def _view(t: torch.Tensor) -> _T2:
    assert t.dtype == torch.float32 and t.dim() == 2 and t.is_contiguous() and not t.is_cuda
    return _T2(t.data_ptr(), 0, 0, t.shape[0], t.shape[1])


class _CAbi:
    """Thin ctypes front end of the ``cverl_*_f32_cpu`` entry points."""

    def __init__(self, library_path: Optional[str] = None):
        """``library_path``: another library exporting the same ten symbols (the reference's ``libcverl``), bound
        instead of this package's - for side-by-side checks."""
        self._lib = None
        self._path = library_path

    @property
    def lib(self):
        if self._lib is None:
            lib = C.CDLL(self._path) if self._path else nv.host()
            two = [_T2, _T2]
            lib.cverl_masked_sum_f32_cpu.argtypes = two + [C.POINTER(C.c_float)]
            lib.cverl_masked_mean_f32_cpu.argtypes = two + [C.POINTER(C.c_float)]
            lib.cverl_masked_whiten_f32_cpu.argtypes = two + [C.c_int, _T2]
            lib.cverl_kl_penalty_f32_cpu.argtypes = two + [C.c_int, _T2]
            lib.cverl_kl_penalty_backward_f32_cpu.argtypes = two + [C.c_int, _T2]
            lib.cverl_gae_advantage_return_f32_cpu.argtypes = [_T2, _T2, _T2, C.c_float, C.c_float, _T2, _T2]
            lib.cverl_grpo_outcome_advantage_f32_cpu.argtypes = [_T2, _T2, C.c_void_p, C.c_float, C.c_int, _T2, _T2]
            lib.cverl_ppo_clipped_loss_f32_cpu.argtypes = [_T2] * 4 + [C.c_float] * 4 + [C.c_int, C.POINTER(_PpoOut)]
            lib.cverl_ppo_clipped_loss_backward_f32_cpu.argtypes = [_T2] * 4 + [C.c_float] * 4 + [C.c_int, _T2]
            lib.cverl_status_string.restype = C.c_char_p
            self._lib = lib
        return self._lib

    @staticmethod
    def _ok(rc: int, what: str):
        if rc != 0:
            raise ValueError(f"{what}: status {rc}")

    def masked_sum(self, v, m) -> float:
        out = C.c_float()
        self._ok(self.lib.cverl_masked_sum_f32_cpu(_view(v), _view(m), C.byref(out)), "masked_sum")
        return out.value

    def masked_mean(self, v, m) -> float:
        out = C.c_float()
        self._ok(self.lib.cverl_masked_mean_f32_cpu(_view(v), _view(m), C.byref(out)), "masked_mean")
        return out.value

    def masked_whiten(self, v, m, shift_mean=True):
        out = torch.empty_like(v)
        self._ok(self.lib.cverl_masked_whiten_f32_cpu(_view(v), _view(m), int(shift_mean), _view(out)), "whiten")
        return out

    def kl_penalty(self, lp, ref, penalty, backward=False):
        out = torch.empty_like(lp)
        fn = self.lib.cverl_kl_penalty_backward_f32_cpu if backward else self.lib.cverl_kl_penalty_f32_cpu
        self._ok(fn(_view(lp), _view(ref), kl_kind(penalty), _view(out)), "kl_penalty")
        return out

    def gae(self, rew, val, mask, gamma, lam):
        adv, ret = torch.empty_like(rew), torch.empty_like(rew)
        self._ok(self.lib.cverl_gae_advantage_return_f32_cpu(_view(rew), _view(val), _view(mask), gamma, lam,
                                                             _view(adv), _view(ret)), "gae")
        return adv, ret

    def grpo(self, rew, mask, gid, eps=1e-6, norm=True):
        adv, ret = torch.empty_like(rew), torch.empty_like(rew)
        gid = gid.to(torch.int64).contiguous()
        self._ok(self.lib.cverl_grpo_outcome_advantage_f32_cpu(_view(rew), _view(mask), gid.data_ptr(), eps,
                                                               int(norm), _view(adv), _view(ret)), "grpo")
        return adv, ret

    def ppo_loss(self, old, lp, adv, mask, clip=0.2, low=-1.0, high=-1.0, c=3.0, agg=0):
        out = _PpoOut()
        self._ok(self.lib.cverl_ppo_clipped_loss_f32_cpu(_view(old), _view(lp), _view(adv), _view(mask), clip, low,
                                                         high, c, agg_mode(agg), C.byref(out)), "ppo_loss")
        return out.pg_loss, out.pg_clipfrac, out.ppo_kl, out.pg_clipfrac_lower

    def ppo_loss_backward(self, old, lp, adv, mask, clip=0.2, low=-1.0, high=-1.0, c=3.0, agg=0):
        g = torch.empty_like(lp)
        self._ok(self.lib.cverl_ppo_clipped_loss_backward_f32_cpu(_view(old), _view(lp), _view(adv), _view(mask),
                                                                  clip, low, high, c, agg_mode(agg), _view(g)),
                 "ppo_loss_backward")
        return g


c_abi = _CAbi()


# ----------------------------------------------------------------------------
# fused CUDA kernels
# ----------------------------------------------------------------------------
_ws_cache = {}


def _workspace(device) -> torch.Tensor:
    key = (device.type, device.index)
    ws = _ws_cache.get(key)
    if ws is None:
        ws = torch.zeros(16, dtype=torch.float64, device=device)
        _ws_cache[key] = ws
    return ws


def _f32c(t):
    return t.to(torch.float32).contiguous()


def fused_masked_mean(values, mask, mean: bool = True) -> torch.Tensor:
    v, m = _f32c(values), _f32c(mask)
    out = torch.empty(1, dtype=torch.float32, device=v.device)
    nv.check(nv.cuda().cvb_masked_sum_mean(v.data_ptr(), m.data_ptr(), v.numel(), int(mean), out.data_ptr(),
                                           _workspace(v.device).data_ptr(), nv.stream()), "cvb_masked_sum_mean")
    count_launch(2)
    return out[0]


def fused_masked_whiten(values, mask, shift_mean: bool = True) -> torch.Tensor:
    v, m = _f32c(values), _f32c(mask)
    out = torch.empty_like(v)
    nv.check(nv.cuda().cvb_masked_whiten(v.data_ptr(), m.data_ptr(), v.numel(), int(shift_mean), out.data_ptr(),
                                         _workspace(v.device).data_ptr(), nv.stream()), "cvb_masked_whiten")
    count_launch(3)
    return out


def fused_kl_penalty(logprob, ref_logprob, penalty="k1", backward: bool = False) -> torch.Tensor:
    lp, ref = _f32c(logprob), _f32c(ref_logprob)
    out = torch.empty_like(lp)
    nv.check(nv.cuda().cvb_kl_penalty(lp.data_ptr(), ref.data_ptr(), out.data_ptr(), lp.numel(), kl_kind(penalty),
                                      int(backward), nv.stream()), "cvb_kl_penalty")
    count_launch()
    return out


def fused_gae(token_level_rewards, values, response_mask, gamma: float, lam: float):
    rew, val, msk = _f32c(token_level_rewards), _f32c(values), _f32c(response_mask)
    rows, cols = rew.shape
    raw, adv, ret = torch.empty_like(rew), torch.empty_like(rew), torch.empty_like(rew)
    nv.check(nv.cuda().cvb_gae(rew.data_ptr(), val.data_ptr(), msk.data_ptr(), raw.data_ptr(), adv.data_ptr(),
                               ret.data_ptr(), rows, cols, gamma, lam, _workspace(rew.device).data_ptr(),
                               nv.stream()), "cvb_gae")
    count_launch(4)
    return adv, ret


def fused_grpo_advantage(token_level_rewards, response_mask, group_ids, epsilon: float = 1e-6,
                         norm_adv_by_std: bool = True):
    rew, msk = _f32c(token_level_rewards), _f32c(response_mask)
    gid = group_ids.to(device=rew.device, dtype=torch.int64).contiguous()
    rows, cols = rew.shape
    adv = torch.empty_like(rew)
    scratch = torch.empty(2 * rows, dtype=torch.float32, device=rew.device)
    nv.check(nv.cuda().cvb_grpo_advantage(rew.data_ptr(), msk.data_ptr(), gid.data_ptr(), epsilon,
                                          int(norm_adv_by_std), adv.data_ptr(), None, scratch.data_ptr(), rows,
                                          cols, nv.stream()), "cvb_grpo_advantage")
    count_launch(3)
    return adv, adv


def fused_ppo_loss(old_log_prob, log_prob, advantages, response_mask, ref_log_prob=None, *,
                   clip_ratio: float = 0.2, clip_ratio_low: float = -1.0, clip_ratio_high: float = -1.0,
                   clip_ratio_c: float = 3.0, agg=AGG_TOKEN_MEAN, kl_coef: float = 0.0, kl_penalty_kind="k1",
                   loss_scale: float = 1.0, want_grad: bool = True):
    """One pass: returns ``(metrics[6], grad)``.

    ``metrics`` = pg_loss, clipfrac, ppo_kl, clipfrac_lower, mean KL to the
    reference (0 without one), token count; ``grad`` = loss_scale *
    d(pg_loss + kl_coef * token_mean(KL)) / d log_prob.
    """
    old, lp, adv, msk = _f32c(old_log_prob), _f32c(log_prob), _f32c(advantages), _f32c(response_mask)
    ref = _f32c(ref_log_prob) if ref_log_prob is not None else None
    rows, cols = lp.shape
    grad = torch.empty_like(lp) if want_grad else None
    metrics = torch.empty(6, dtype=torch.float32, device=lp.device)
    rowcnt = torch.empty(rows, dtype=torch.float32, device=lp.device)
    nv.check(nv.cuda().cvb_ppo_loss(old.data_ptr(), lp.data_ptr(), adv.data_ptr(), msk.data_ptr(), nv.ptr(ref),
                                    nv.ptr(grad), metrics.data_ptr(), rowcnt.data_ptr(), rows, cols, clip_ratio,
                                    clip_ratio_low, clip_ratio_high, clip_ratio_c, agg_mode(agg), kl_coef,
                                    kl_kind(kl_penalty_kind), loss_scale, _workspace(lp.device).data_ptr(),
                                    nv.stream()), "cvb_ppo_loss")
    count_launch(3)
    return metrics, grad


def actor_loss(old_log_prob, log_prob, advantages, response_mask, ref_log_prob=None, **kw):
    """Device-agnostic ``fused_ppo_loss``: CUDA kernels on GPU tensors, PyTorch math otherwise."""
    if log_prob.is_cuda:
        return fused_ppo_loss(old_log_prob, log_prob, advantages, response_mask, ref_log_prob, **kw)
    want_grad = kw.pop("want_grad", True)
    kl_coef = kw.pop("kl_coef", 0.0)
    kind = kw.pop("kl_penalty_kind", "k1")
    loss_scale = kw.pop("loss_scale", 1.0)
    agg = kw.pop("agg", AGG_TOKEN_MEAN)
    lp = log_prob.detach().float().clone().requires_grad_(want_grad)
    res = ppo_clipped_loss(old_log_prob.float(), lp, advantages.float(), response_mask.float(), agg=agg,
                           clip_ratio=kw.pop("clip_ratio", 0.2), clip_ratio_low=kw.pop("clip_ratio_low", -1.0),
                           clip_ratio_high=kw.pop("clip_ratio_high", -1.0),
                           clip_ratio_c=kw.pop("clip_ratio_c", 3.0))
    total = res.pg_loss
    klm = torch.zeros(())
    if ref_log_prob is not None:
        klm = masked_mean(kl_penalty(lp, ref_log_prob.float(), kind), response_mask.float())
        total = total + kl_coef * klm
    grad = None
    if want_grad:
        (grad,) = torch.autograd.grad(total * loss_scale, lp)
    metrics = torch.stack([res.pg_loss.detach(), res.pg_clipfrac, res.ppo_kl.detach(), res.pg_clipfrac_lower,
                           klm.detach(), response_mask.float().sum()]).float()
    return metrics, grad
