"""Static trainer / rollout split on one node: the first T ranks train, the last R ranks generate.

``torchrun --nproc-per-node 8 -m cverl_b200.cli.static_split --trainers 4 --steps 5 [--backend gloo]``

Every step, in lock step over the whole world:

1. each rollout rank samples ``--n`` responses per prompt from its copy of the policy (cached decode for the
   Qwen policy), scores them with the GSM8K rule reward and sends one ``GpuRolloutBatch`` (ids, mask, rewards,
   old log-probs, group ids, the ``weight_version`` it generated with) to its trainer rank;
2. each trainer rank receives its batches into a ``TrainerIngressQueue``, forms GRPO advantages, runs the PPO
   epochs with gradients averaged over the trainer group, and bumps the weight version;
3. the new weights go back: trainer ``i`` pushes its parameters to the rollout ranks it serves
   (``send_parameter_shards`` / ``recv_parameter_shards``, bucketed), so the next rollouts are on-policy.

The reference documents this 4 + 4 layout but has no live weight push in its multi-GPU trainer; its library
functions are src/distributed/weight_sync.cc:86-189 and src/rollout/nccl_gpu_batch_transport.cc:119-344.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch

from ..models.policy import CausalLmPolicyOptions, make_causal_lm_policy
from ..ops import rl
from ..parallel.collectives import ReduceOp, TorchDistCollectives
from ..parallel.weight_sync import module_parameter_views, recv_parameter_shards, send_parameter_shards
from ..reward.gsm8k import Gsm8kRewardOptions
from ..rollout.gpu_batch_transport import GpuBatchReceiver, GpuBatchSender, GpuRolloutBatch, TrainerIngressQueue
from ..rollout.rollout_batch import build_gsm8k_rollout_batch
from ..rollout.worker import GenerationConfig, PolicyRolloutWorker
from ..text.tokenizer import ByteTokenizer
from ..trainer.gsm8k_grpo import generate_samples


def _problems(n: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(1, 20, (n, 2), generator=g).tolist()
    return [f"What is {x}+{y}?" for x, y in a], [f"#### {x + y}" for x, y in a]


def main(argv=None) -> int:
    import torch.distributed as dist
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--trainers", type=int, default=0, help="number of trainer ranks (default: half the world)")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--prompts", type=int, default=4, help="prompts per rollout rank per step")
    ap.add_argument("--n", type=int, default=4)
    ap.add_argument("--max-prompt-tokens", type=int, default=24)
    ap.add_argument("--max-response-tokens", type=int, default=8)
    ap.add_argument("--ppo-epochs", type=int, default=1)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--clip-ratio", type=float, default=0.2)
    ap.add_argument("--hidden-dim", type=int, default=32)
    ap.add_argument("--policy", default="tiny", choices=["tiny", "qwen"])
    ap.add_argument("--model-dir", default="")
    ap.add_argument("--backend", default="nccl", choices=["nccl", "gloo"])
    ap.add_argument("--seed", type=int, default=17)
    ap.add_argument("--weight-push", default="nccl", choices=["nccl", "symm", "nvls"],
                    help="trainer -> rollout weights: library send / recv per bucket, stores into peer-mapped receive "
                         "buffers by this package's kernel, or one multicast store through the NVSwitch (CUDA only)")
    a = ap.parse_args(argv)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if a.backend == "nccl":
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=device)
    else:
        device = torch.device("cpu")
        dist.init_process_group("gloo")
    comm = TorchDistCollectives()
    rank, world = comm.rank(), comm.world_size()
    T = a.trainers or world // 2
    R = world - T
    if T <= 0 or R <= 0 or R % T:
        raise SystemExit("need at least one trainer and a rollout count that is a multiple of the trainer count")
    is_trainer = rank < T
    trainer_group = list(range(T))
    comm.pg(trainer_group)       # sub-groups are created collectively: the rollout ranks take part, then never use it
    my_trainer = (rank - T) % T if not is_trainer else rank
    my_rollouts = [T + j for j in range(R) if j % T == rank] if is_trainer else []

    tok = ByteTokenizer()
    torch.manual_seed(a.seed)                                  # identical initial weights everywhere
    policy = make_causal_lm_policy(CausalLmPolicyOptions(
        kind="tiny" if a.policy == "tiny" else "qwen3_5", vocab_size=tok.vocab_size, hidden_size=a.hidden_dim,
        pad_id=max(tok.pad_id, 0), model_dir=a.model_dir)).to_device(device)
    params = module_parameter_views(policy)
    pusher = None
    if a.weight_push != "nccl":
        if a.backend != "nccl":
            raise SystemExit("--weight-push symm / nvls needs --backend nccl (CUDA peer memory)")
        from ..parallel.weight_sync import PeerMemoryWeightPush
        pusher = PeerMemoryWeightPush(params, device, T, world, a.weight_push)
    version = 0
    if is_trainer:
        opt = torch.optim.AdamW(policy.parameters(), lr=a.lr)
        queue = TrainerIngressQueue(capacity=max(2, len(my_rollouts)))
        receiver = GpuBatchReceiver(comm, device)
    else:
        worker = PolicyRolloutWorker(policy)
        sender = GpuBatchSender(comm, device)

    for step in range(1, a.steps + 1):
        t0 = time.time()
        if not is_trainer:
            prompts, answers = _problems(a.prompts, a.seed * 1000 + step * 64 + rank)
            gen = GenerationConfig(max_new_tokens=a.max_response_tokens, eos_token_id=tok.eos_id, eos_check_interval=8,
                                   seed=a.seed + step + rank)
            samples = generate_samples(worker, tok, prompts, a.n, gen, a.max_prompt_tokens, device)
            rb = build_gsm8k_rollout_batch(tok, prompts, answers, samples, a.max_prompt_tokens, a.max_response_tokens,
                                           Gsm8kRewardOptions(method="flexible")).to(device)
            with torch.no_grad():
                old_lp = policy.response_log_probs(rb.prompt_ids, rb.response_ids).float()
            sender.send(GpuRolloutBatch(step, version, a.max_prompt_tokens, a.max_response_tokens, {
                "prompt_ids": rb.prompt_ids, "response_ids": rb.response_ids, "response_mask": rb.response_mask,
                "old_log_probs": old_lp, "rewards": rb.rewards, "group_ids": rb.group_ids}), my_trainer)
            line = f"rollout rank {rank} step {step} sent {len(samples)} sequences weight_version={version}"
        else:
            for src in my_rollouts:
                if not queue.push(receiver.recv(src)):
                    raise RuntimeError("ingress queue overflow")
            stats = torch.zeros(3, device=device)               # loss, reward sum, sequences
            opt.zero_grad(set_to_none=True)
            stale = 0
            while len(queue):
                b = queue.pop()
                stale = max(stale, version - b.weight_version)
                t = b.tensors
                mask = t["response_mask"]
                tr = torch.zeros_like(mask)
                last = (mask.sum(-1).long() - 1).clamp_min(0)
                tr[torch.arange(mask.shape[0], device=device), last] = t["rewards"]
                adv, _ = rl.grpo_outcome_advantage(tr, mask, t["group_ids"], 1e-6, True)
                for _ in range(a.ppo_epochs):
                    lp = policy.response_log_probs(t["prompt_ids"], t["response_ids"]).float()
                    res = rl.ppo_clipped_loss(t["old_log_probs"], lp, adv, mask, a.clip_ratio)
                    (res.pg_loss / max(1, len(my_rollouts))).backward()
                stats += torch.stack([res.pg_loss.detach(), t["rewards"].sum(), torch.tensor(float(mask.shape[0]), device=device)])
            for p in policy.parameters():                        # data parallel over the trainer ranks
                if p.grad is None:
                    p.grad = torch.zeros_like(p)
                p.grad.copy_(comm.all_reduce(p.grad, ReduceOp.SUM, trainer_group) / T)
            opt.step()
            version += 1
            stats = comm.all_reduce(stats, ReduceOp.SUM, trainer_group)
            line = (f"trainer rank {rank} step {step} loss={float(stats[0]) / T:.5f} "
                    f"mean_reward={float(stats[1] / stats[2].clamp_min(1)):.4f} sequences={int(stats[2])} "
                    f"max_staleness={stale} weight_version={version}")
        # ---- weight push: each trainer to the rollout ranks it serves ------------------------------------
        if pusher is not None:
            pusher.push(rank, my_rollouts)
            if not is_trainer:
                version += 1
        elif is_trainer:
            for dst in my_rollouts:
                send_parameter_shards(params, comm, dst)
        else:
            recv_parameter_shards(params, comm, my_trainer)
            version += 1
        comm.barrier()
        if rank == 0 or rank == T:
            print(f"{line} step_time_s={time.time() - t0:.3f}", flush=True)
    # every rank must end with the same weights
    check = torch.cat([p.tensor.detach().reshape(-1).float() for p in params]).sum().reshape(1)
    lo = comm.all_reduce(check.clone(), ReduceOp.MIN)
    hi = comm.all_reduce(check.clone(), ReduceOp.MAX)
    if rank == 0:
        print(f"static split finished: trainers={T} rollout={R} weights_in_sync={bool(torch.allclose(lo, hi))}", flush=True)
    dist.destroy_process_group()
    return 0 if bool(torch.allclose(lo, hi)) else 3


if __name__ == "__main__":
    sys.exit(main())
