"""The small GRPO loop shared by the demo trainers and the tiny-policy benchmark.

A policy maps a ``[batch, seq]`` grid of target ids to logits over an action set.  Every step samples actions from
the current policy, rewards a sequence with the share of positions where the action equals the target (placed on
the last token), forms GRPO outcome advantages within each prompt's group and runs ``ppo_epochs`` clipped-PPO
updates with AdamW.  This is the loop of the reference's demo programs (tools/model/
hf_embedding_grpo_trainer.cc:120-176, tools/bench/cverl_gsm8k_grpo_bench.cc:165-207), written once.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ..ops import rl


@dataclass
class StepStats:
    step: int
    loss: float
    avg_reward: float
    success_rate: float
    ppo_kl: float
    clipfrac: float


def action_log_probs(logits: torch.Tensor, actions: torch.Tensor) -> torch.Tensor:
    return torch.log_softmax(logits, -1).gather(-1, actions.unsqueeze(-1)).squeeze(-1)


def accuracy_grpo_step(policy: Callable[[torch.Tensor], torch.Tensor], optimizer, prompt_targets: torch.Tensor,
                       responses: int, ppo_epochs: int, step: int, clip_ratio: float = 0.2,
                       generator: Optional[torch.Generator] = None) -> StepStats:
    """One step on ``prompt_targets`` ``[prompts, seq]``; every prompt gets ``responses`` sampled sequences."""
    prompts, seq = prompt_targets.shape
    dev = prompt_targets.device
    batch = prompts * responses
    targets = prompt_targets.repeat_interleave(responses, 0)
    mask = torch.ones(batch, seq, device=dev)
    group_ids = torch.arange(prompts, device=dev).repeat_interleave(responses)
    with torch.no_grad():
        old_logits = policy(targets)
        probs = torch.softmax(old_logits, -1)
        actions = probs.reshape(batch * seq, -1).multinomial(1, generator=generator).reshape(batch, seq)
        old_lp = action_log_probs(old_logits, actions)
    scalar = ((actions == targets).float() * mask).sum(-1) / mask.sum(-1)
    token_rewards = torch.zeros(batch, seq, device=dev)
    token_rewards[:, seq - 1] = scalar
    adv, _ = rl.grpo_outcome_advantage(token_rewards, mask, group_ids, 1e-6, True)
    res = None
    for _ in range(ppo_epochs):
        lp = action_log_probs(policy(targets), actions)
        res = rl.ppo_clipped_loss(old_lp, lp, adv, mask, clip_ratio, -1.0, -1.0, 3.0)
        optimizer.zero_grad()
        res.pg_loss.backward()
        optimizer.step()
    return StepStats(step, float(res.pg_loss.detach()), float(scalar.mean()), float((scalar >= 0.999).float().mean()),
                     float(res.ppo_kl), float(res.pg_clipfrac))


CSV_HEADER = "step,loss,avg_reward,success_rate,ppo_kl,clipfrac"


def csv_row(s: StepStats) -> str:
    return f"{s.step},{s.loss:.6g},{s.avg_reward:.6g},{s.success_rate:.6g},{s.ppo_kl:.6g},{s.clipfrac:.6g}"
