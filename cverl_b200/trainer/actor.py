"""Actor update engine: PPO / GRPO policy loss or SFT over micro-batches, then
one sharded optimizer step.

One ``update`` is the reference trainer's hot loop for a single pipeline stage
(tools/model/qwen3_5_pp_tp_ppo_trainer.cc:2272-2451): per micro-batch a forward
to response log-probs, the clipped PPO loss (+ optional KL term) or the SFT
negative log-likelihood, each divided by the number of micro-batches, backward
into the flat fp32 gradient buffer; then gradient reduce-scatter, global-norm
clip, FlatAdamW and parameter all-gather.  The loss never builds an autograd
graph: a fused kernel returns the metrics and d(loss)/d(log_prob), which seeds
the model backward.  Metrics stay on the device and are read once per step.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import rl


@dataclass
class ActorConfig:
    mode: str = "ppo"                 # "ppo" (GRPO/PPO policy loss) or "sft"
    micro_batch_size: int = 8         # sequences per micro-batch
    clip_ratio: float = 0.2
    clip_ratio_low: float = -1.0
    clip_ratio_high: float = -1.0
    clip_ratio_c: float = 3.0
    loss_agg: str = "token-mean"
    kl_coef: float = 0.0
    kl_penalty: str = "k1"
    advantage_scale: float = 1.0      # used when a batch carries no advantages


METRIC_NAMES = ("pg_loss", "pg_clipfrac", "ppo_kl", "pg_clipfrac_lower", "kl_loss", "tokens")


class ActorEngine:
    def __init__(self, model, optimizer, cfg: ActorConfig):
        self.model = model
        self.optimizer = optimizer
        self.cfg = cfg
        self._pinned: Dict[str, torch.Tensor] = {}
        self._device_batch: Dict[str, torch.Tensor] = {}

    @property
    def device(self):
        return self.model.flat.flat.device

    # ------------------------------------------------------------------
    def update(self, batch: Dict[str, torch.Tensor], prompt_len: int) -> torch.Tensor:
        """One optimizer step over ``batch`` (device tensors). Returns a device tensor of
        ``len(METRIC_NAMES) + 3`` floats: the metric sums over micro-batches (loss terms
        already carry the 1/num_micro factor), then [local_sq, global_sq, clip_scale]."""
        cfg = self.cfg
        ids = batch["input_ids"]
        n = ids.shape[0]
        mb = min(cfg.micro_batch_size, n)
        if n % mb:
            raise ValueError("batch size must be a multiple of the micro-batch size")
        num_micro = n // mb
        ctx = getattr(self.model, "ctx", None)
        cp = ctx.cp_size if ctx is not None else 1
        # under context parallelism every rank evaluates the same loss on the gathered log-probs and
        # back-propagates only its shard: 1/cp here makes the CP-summed gradient the true one
        grad_scale = 1.0 / (num_micro * cp)
        total = torch.zeros(len(METRIC_NAMES), dtype=torch.float32, device=ids.device)
        for m in range(num_micro):
            sl = slice(m * mb, (m + 1) * mb)
            lp = self.model.response_logprobs(ids[sl], prompt_len)
            mask = batch["response_mask"][sl]
            if cfg.mode == "sft":
                denom = mask.sum() + rl.EPS
                dlogp = (-mask / denom) * grad_scale
                nll = -(lp.detach() * mask).sum() / denom
                metrics = torch.stack([nll, nll.new_zeros(()), nll.new_zeros(()), nll.new_zeros(()),
                                       nll.new_zeros(()), mask.sum()])
            else:
                adv = batch.get("advantages")
                adv = adv[sl] if adv is not None else torch.full_like(lp, cfg.advantage_scale).detach()
                old = batch.get("old_log_probs")
                old = old[sl] if old is not None else lp.detach()
                ref = batch.get("ref_log_probs")
                ref = ref[sl] if (ref is not None and cfg.kl_coef != 0.0) else None
                metrics, dlogp = rl.actor_loss(old, lp.detach(), adv, mask, ref, clip_ratio=cfg.clip_ratio,
                                               clip_ratio_low=cfg.clip_ratio_low,
                                               clip_ratio_high=cfg.clip_ratio_high, clip_ratio_c=cfg.clip_ratio_c,
                                               agg=cfg.loss_agg, kl_coef=cfg.kl_coef,
                                               kl_penalty_kind=cfg.kl_penalty, loss_scale=grad_scale)
            lp.backward(dlogp.to(lp.dtype))
            scale = torch.tensor([1.0 / num_micro] * 5 + [1.0], device=total.device)
            total += metrics.to(total.device) * scale
        self.fold_autograd_grads()
        if hasattr(self.model, "sync_replicated_grads"):
            self.model.sync_replicated_grads()
        if cp > 1:
            import torch.distributed as dist
            dist.all_reduce(self.model.flat.main_grad, group=ctx.cp_group)
        self.optimizer.step()
        return torch.cat([total, self.optimizer.last_metrics.to(total.device)])

    def fold_autograd_grads(self) -> None:
        """Ops without a native kernel on this device leave ``.grad``; fold it into main_grad."""
        params = list(self.model.flat.params.values()) + list(getattr(self.model, "fused", {}).values())
        for p in params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.float())
                p.grad = None

    # ------------------------------------------------------------------
    def pin_batch(self, batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """Page-locked host copies of a batch (the staging area a data loader would own)."""
        out = {}
        for k, v in batch.items():
            t = v.detach().cpu().contiguous()
            out[k] = t.pin_memory() if torch.cuda.is_available() else t
        return out

    def update_from_host(self, host_batch: Dict[str, torch.Tensor], prompt_len: int):
        """End-to-end step: H2D of the inputs, ``update``, D2H of the metrics (a host sync)."""
        dev = self.device
        dbatch = {k: v.to(dev, non_blocking=True) for k, v in host_batch.items()}
        out = self.update(dbatch, prompt_len)
        return out.cpu()

    @staticmethod
    def host_batch_bytes(host_batch: Dict[str, torch.Tensor]) -> int:
        return sum(v.numel() * v.element_size() for v in host_batch.values())


def synthetic_rl_batch(num_seqs: int, prompt_len: int, response_len: int, vocab: int, device="cpu",
                       seed: int = 0, group_size: int = 8) -> Dict[str, torch.Tensor]:
    """Synthetic GRPO batch: uniform token ids, Bernoulli(0.5) outcome rewards in groups,
    GRPO advantages, old log-probs unset (ratio 1), random response lengths."""
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(1, vocab, (num_seqs, prompt_len + response_len), generator=g)
    lens = torch.randint(max(1, response_len // 2), response_len + 1, (num_seqs,), generator=g)
    mask = (torch.arange(response_len)[None, :] < lens[:, None]).float()
    rewards = torch.zeros(num_seqs, response_len)
    outcome = torch.bernoulli(torch.full((num_seqs,), 0.5), generator=g)
    rewards[torch.arange(num_seqs), lens - 1] = outcome
    gid = torch.arange(num_seqs) // group_size
    adv, _ = rl.grpo_outcome_advantage(rewards, mask, gid)
    batch = {"input_ids": ids, "response_mask": mask, "advantages": adv}
    return {k: v.to(device) for k, v in batch.items()}
