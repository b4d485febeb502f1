"""One PPO step on a tiny MLP policy: the smallest end-to-end use of the RL math.

``python -m cverl_b200.cli.minimal_ppo_step``

Random observations ``[8, 4, 6]``, a 6-16-5 MLP, random actions, the last token masked out, GRPO outcome
advantages over groups of two, one clipped-PPO update with AdamW; prints the loss, clip fraction, approximate
KL and the parameter change (reference: tools/torch/minimal_ppo_step.cc).
"""
from __future__ import annotations

import sys

import torch

from ..ops import rl
from ..trainer.accuracy_grpo import action_log_probs


def main(argv=None) -> int:
    torch.manual_seed(11)
    batch, seq, obs_dim, hidden, actions_n = 8, 4, 6, 16, 5
    policy = torch.nn.Sequential(torch.nn.Linear(obs_dim, hidden), torch.nn.ReLU(), torch.nn.Linear(hidden, actions_n))
    opt = torch.optim.AdamW(policy.parameters(), lr=1e-3)
    obs = torch.randn(batch, seq, obs_dim)
    actions = torch.randint(actions_n, (batch, seq))
    mask = torch.ones(batch, seq)
    mask[:, seq - 1] = 0.0
    with torch.no_grad():
        old_lp = action_log_probs(policy(obs), actions)
    token_rewards = torch.randn(batch, seq) * mask
    group_ids = torch.arange(batch) // 2
    adv, _ = rl.grpo_outcome_advantage(token_rewards, mask, group_ids, 1e-6, True)
    before = [p.detach().clone() for p in policy.parameters()]
    res = rl.ppo_clipped_loss(old_lp, action_log_probs(policy(obs), actions), adv, mask, 0.2, -1.0, -1.0, 3.0)
    opt.zero_grad()
    res.pg_loss.backward()
    grad_norm = float(torch.cat([p.grad.reshape(-1) for p in policy.parameters()]).norm())
    opt.step()
    delta = float(sum((p.detach() - b).abs().sum() for p, b in zip(policy.parameters(), before)))
    print(f"pg_loss={float(res.pg_loss.detach()):.6f} pg_clipfrac={float(res.pg_clipfrac):.6f} ppo_kl={float(res.ppo_kl):.6f} "
          f"grad_norm={grad_norm:.6f} param_delta={delta:.6f}")
    return 0 if (grad_norm > 0 and delta > 0) else 1


if __name__ == "__main__":
    sys.exit(main())
