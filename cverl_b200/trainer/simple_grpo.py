"""Self-contained toy GRPO loop: the smallest end-to-end use of the RL math.

Task: each prompt is a sequence of target symbols shown one-hot to an MLP policy; the policy
samples one action per position; the reward is the fraction of positions where the action equals
the target, paid on the last token; advantages are GRPO outcome advantages within the group of
responses to one prompt; the policy is improved by a few PPO-clip epochs.

Same behaviour and checkpoint files (``<prefix>.model.pt``, ``.optim.pt``, ``.meta.pt``) as the
reference (src/torch/simple_grpo_trainer.cc:66-173); the archives here are written by
``utils.checkpoint.save_archive``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch
from torch import nn

from ..ops import rl
from ..utils.checkpoint import load_archive, save_archive


@dataclass
class SimpleGrpoTrainerConfig:
    steps: int = 32
    prompts_per_batch: int = 8
    responses_per_prompt: int = 4
    seq_len: int = 8
    action_dim: int = 8
    hidden_dim: int = 64
    ppo_epochs: int = 2
    learning_rate: float = 3.0e-3
    clip_ratio: float = 0.2
    entropy_coef: float = 0.0
    seed: int = 17


@dataclass
class SimpleGrpoTrainerMetrics:
    step: int = 0
    loss: float = 0.0
    avg_reward: float = 0.0
    success_rate: float = 0.0
    ppo_kl: float = 0.0
    clipfrac: float = 0.0


def _action_log_probs(logits: torch.Tensor, actions: torch.Tensor) -> torch.Tensor:
    return torch.log_softmax(logits, -1).gather(-1, actions.unsqueeze(-1)).squeeze(-1)


def _entropy(logits: torch.Tensor) -> torch.Tensor:
    lp = torch.log_softmax(logits, -1)
    return -(lp.exp() * lp).sum(-1)


class SimpleGrpoTrainer:
    def __init__(self, config: SimpleGrpoTrainerConfig):
        if min(config.prompts_per_batch, config.responses_per_prompt, config.seq_len, config.action_dim,
               config.hidden_dim) <= 0 or config.ppo_epochs <= 0:
            raise ValueError("SimpleGrpoTrainer: sizes must be positive")
        self.config = config
        self.gen = torch.Generator().manual_seed(config.seed)
        torch.manual_seed(config.seed)
        self.policy = nn.Sequential(nn.Linear(config.action_dim, config.hidden_dim), nn.Tanh(),
                                    nn.Linear(config.hidden_dim, config.action_dim))
        self.optimizer = torch.optim.AdamW(self.policy.parameters(), lr=config.learning_rate)
        self.step = 0

    def current_step(self) -> int:
        return self.step

    def train_step(self) -> SimpleGrpoTrainerMetrics:
        c = self.config
        batch = c.prompts_per_batch * c.responses_per_prompt
        prompt_targets = torch.randint(c.action_dim, (c.prompts_per_batch, c.seq_len), generator=self.gen)
        targets = prompt_targets.repeat_interleave(c.responses_per_prompt, 0)
        obs = torch.nn.functional.one_hot(targets, c.action_dim).float()
        mask = torch.ones(batch, c.seq_len)
        group_ids = torch.arange(c.prompts_per_batch).repeat_interleave(c.responses_per_prompt)
        with torch.no_grad():
            old_logits = self.policy(obs)
            probs = torch.softmax(old_logits, -1).reshape(batch * c.seq_len, c.action_dim)
            actions = torch.multinomial(probs, 1, generator=self.gen).reshape(batch, c.seq_len)
            old_lp = _action_log_probs(old_logits, actions)
        scalar_rewards = ((actions == targets).float() * mask).sum(-1) / mask.sum(-1)
        token_rewards = torch.zeros(batch, c.seq_len)
        token_rewards[:, -1] = scalar_rewards
        advantages, _ = rl.grpo_outcome_advantage(token_rewards, mask, group_ids, 1.0e-6, True)
        m = SimpleGrpoTrainerMetrics()
        for _ in range(c.ppo_epochs):
            logits = self.policy(obs)
            lp = _action_log_probs(logits, actions)
            res = rl.ppo_clipped_loss(old_lp, lp, advantages, mask, c.clip_ratio, -1.0, -1.0, 3.0, rl.AGG_TOKEN_MEAN)
            loss = res.pg_loss
            if c.entropy_coef != 0.0:
                loss = loss - c.entropy_coef * rl.masked_mean(_entropy(logits), mask)
            self.optimizer.zero_grad()
            loss.backward()
            self.optimizer.step()
            m.loss, m.ppo_kl, m.clipfrac = loss.item(), res.ppo_kl.item(), res.pg_clipfrac.item()
        self.step += 1
        m.step = self.step
        m.avg_reward = float(scalar_rewards.mean())
        m.success_rate = float((scalar_rewards >= 0.999).float().mean())
        return m

    def train(self) -> List[SimpleGrpoTrainerMetrics]:
        return [self.train_step() for _ in range(self.config.steps)]

    # ------------------------------------------------------------------ checkpoint
    def save_checkpoint(self, prefix: str) -> None:
        save_archive(prefix + ".model.pt", {k: v.detach() for k, v in self.policy.state_dict().items()})
        flat = {}
        for i, p in enumerate(self.policy.parameters()):
            st = self.optimizer.state.get(p, {})
            if st:
                flat[f"{i}.step"] = torch.as_tensor(st["step"]).detach().clone().reshape(())
                flat[f"{i}.exp_avg"] = st["exp_avg"].detach()
                flat[f"{i}.exp_avg_sq"] = st["exp_avg_sq"].detach()
        save_archive(prefix + ".optim.pt", flat)
        save_archive(prefix + ".meta.pt", {"step": torch.tensor(self.step, dtype=torch.int64),
                                           "seed": torch.tensor(self.config.seed, dtype=torch.int64),
                                           "rng_state": self.gen.get_state()})

    def load_checkpoint(self, prefix: str) -> None:
        self.policy.load_state_dict(load_archive(prefix + ".model.pt"))
        flat = load_archive(prefix + ".optim.pt")
        for i, p in enumerate(self.policy.parameters()):
            if f"{i}.exp_avg" in flat:
                self.optimizer.state[p] = {"step": flat[f"{i}.step"].clone().float(),
                                           "exp_avg": flat[f"{i}.exp_avg"].clone(),
                                           "exp_avg_sq": flat[f"{i}.exp_avg_sq"].clone()}
        meta = load_archive(prefix + ".meta.pt")
        self.step = int(meta["step"])
        if "rng_state" in meta:
            self.gen.set_state(meta["rng_state"].to(torch.uint8))
