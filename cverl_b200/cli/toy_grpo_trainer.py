"""The self-contained toy GRPO trainer as a program.

``python -m cverl_b200.cli.toy_grpo_trainer [steps [prompts [responses]]] [--save-prefix P] [--load-prefix P]``

Runs ``SimpleGrpoTrainer`` (one-hot observation MLP policy, sampled actions, accuracy reward, GRPO advantages,
PPO epochs) and prints one CSV row per step; ``--save-prefix`` / ``--load-prefix`` write and read its
``.model.pt / .optim.pt / .meta.pt`` checkpoint (reference: tools/torch/toy_grpo_trainer.cc).
"""
from __future__ import annotations

import sys

from ..trainer.simple_grpo import SimpleGrpoTrainer, SimpleGrpoTrainerConfig


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    cfg = SimpleGrpoTrainerConfig()
    positional = []
    save_prefix = load_prefix = ""
    i = 0
    while i < len(argv):
        if argv[i] == "--save-prefix" and i + 1 < len(argv):
            save_prefix, i = argv[i + 1], i + 2
        elif argv[i] == "--load-prefix" and i + 1 < len(argv):
            load_prefix, i = argv[i + 1], i + 2
        else:
            positional.append(argv[i])
            i += 1
    for name, value in zip(("steps", "prompts_per_batch", "responses_per_prompt"), positional):
        setattr(cfg, name, int(value))
    trainer = SimpleGrpoTrainer(cfg)
    if load_prefix:
        trainer.load_checkpoint(load_prefix)
    print("step,loss,avg_reward,success_rate,ppo_kl,clipfrac")
    for m in trainer.train():
        print(f"{m.step},{m.loss:.6g},{m.avg_reward:.6g},{m.success_rate:.6g},{m.ppo_kl:.6g},{m.clipfrac:.6g}")
    if save_prefix:
        trainer.save_checkpoint(save_prefix)
    return 0


if __name__ == "__main__":
    sys.exit(main())
