"""Throughput of a tiny-MLP GRPO loop over a prompt / answer JSONL: ``train_tokens_per_second``.

``python -m cverl_b200.cli.gsm8k_grpo_bench --dataset data.jsonl [--steps 20] [--prompts 8] [--responses 4]
[--seq-len 16] [--action-dim 32] [--hidden-dim 64] [--ppo-epochs 2] [--lr 1e-3] [--seed 1] [--device cpu]``

Targets are derived from each example's text (FNV-1a of ``prompt + "\\n" + answer`` seeding an xorshift stream),
observations are their one-hot codes, the policy is Linear-ReLU-Linear.  Prints ``key,value`` lines: the shape,
``seconds``, ``sequences_per_second``, ``train_tokens_per_second`` (= steps x prompts x responses x seq_len x
ppo_epochs / seconds) and the last step's loss / reward / KL / clip fraction - the fields the reference's bench
prints (tools/bench/cverl_gsm8k_grpo_bench.cc:165-228), so the two can be set side by side on the same file.
"""
from __future__ import annotations

import argparse
import sys
import time

import torch

from ..data import load_prompt_answer_jsonl
from ..trainer.accuracy_grpo import accuracy_grpo_step

_MASK = (1 << 64) - 1


def _fnv1a64(text: str, seed: int) -> int:
    h = (1469598103934665603 ^ seed) & _MASK
    for ch in text.encode("utf-8"):
        h ^= ch
        h = (h * 1099511628211) & _MASK
    return h


def make_targets(data, step: int, prompts: int, seq_len: int, action_dim: int, seed: int, device) -> torch.Tensor:
    rows = []
    for row in range(prompts):
        ex = data[(step * prompts + row) % len(data)]
        state = _fnv1a64(ex.prompt + "\n" + ex.answer, seed + step)
        vals = []
        for _ in range(seq_len):
            state ^= state >> 12
            state ^= (state << 25) & _MASK
            state ^= state >> 27
            vals.append(((state * 2685821657736338717) & _MASK) % action_dim)
        rows.append(vals)
    return torch.tensor(rows, dtype=torch.int64, device=device)


class OneHotMlp(torch.nn.Module):
    def __init__(self, action_dim: int, hidden_dim: int):
        super().__init__()
        self.action_dim = action_dim
        self.fc1 = torch.nn.Linear(action_dim, hidden_dim)
        self.fc2 = torch.nn.Linear(hidden_dim, action_dim)

    def forward(self, targets: torch.Tensor) -> torch.Tensor:
        obs = torch.nn.functional.one_hot(targets, self.action_dim).float()
        return self.fc2(torch.relu(self.fc1(obs)))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--dataset", required=True)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--prompts", type=int, default=8)
    ap.add_argument("--responses", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=16)
    ap.add_argument("--action-dim", type=int, default=32)
    ap.add_argument("--hidden-dim", type=int, default=64)
    ap.add_argument("--ppo-epochs", type=int, default=2)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args(argv)
    if min(a.steps, a.prompts, a.seq_len, a.hidden_dim, a.ppo_epochs) <= 0 or a.responses <= 1 or a.action_dim <= 1:
        print("invalid benchmark shape", file=sys.stderr)
        return 2
    torch.manual_seed(a.seed)
    dev = torch.device(a.device)
    data = load_prompt_answer_jsonl(a.dataset)
    if not data:
        print("dataset is empty", file=sys.stderr)
        return 2
    policy = OneHotMlp(a.action_dim, a.hidden_dim).to(dev)
    opt = torch.optim.AdamW(policy.parameters(), lr=a.lr)
    last = None
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    for step in range(a.steps):
        targets = make_targets(data, step, a.prompts, a.seq_len, a.action_dim, a.seed, dev)
        last = accuracy_grpo_step(policy, opt, targets, a.responses, a.ppo_epochs, step)
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)
    seconds = time.perf_counter() - t0
    sequences = a.steps * a.prompts * a.responses
    tokens = sequences * a.seq_len * a.ppo_epochs
    for k, v in (("backend", "cverl_b200"), ("dataset_rows", len(data)), ("steps", a.steps), ("prompts", a.prompts),
                 ("responses", a.responses), ("seq_len", a.seq_len), ("action_dim", a.action_dim),
                 ("hidden_dim", a.hidden_dim), ("ppo_epochs", a.ppo_epochs), ("device", a.device),
                 ("seconds", f"{seconds:.6f}"), ("sequences_per_second", f"{sequences / seconds:.6f}"),
                 ("train_tokens_per_second", f"{tokens / seconds:.6f}"), ("last_loss", f"{last.loss:.6f}"),
                 ("last_avg_reward", f"{last.avg_reward:.6f}"), ("last_ppo_kl", f"{last.ppo_kl:.6f}"),
                 ("last_clipfrac", f"{last.clipfrac:.6f}")):
        print(f"{k},{v}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
