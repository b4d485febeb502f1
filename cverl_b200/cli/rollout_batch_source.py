"""Synthetic rollout rank: sends a deterministic ``GpuRolloutBatch`` to the listed trainer ranks every step.

Launch it as one rank of a ``torch.distributed`` job (``torchrun`` sets RANK / WORLD_SIZE / LOCAL_RANK):

``python -m cverl_b200.cli.rollout_batch_source --target-ranks 0,1 --steps 4 --batch 4 --prompt-len 32 --response-len 8``

The batch contents follow the reference source rank (tools/rollout/nccl_rollout_batch_source.cc:38-84):
``prompt_ids = 1..B*P``, ``response_ids = 100..``, an all-ones mask, advantages +1 on even rows and -1 on odd
rows, zero old log-probs, rewards 1/0 alternating, group ids ``row // 2``; ``weight_version`` advances with the
step.  Trainer ranks receive with ``GpuBatchReceiver`` (``--receive-from R`` turns this process into such a
receiver and prints what arrived, for smoke tests).

Started on its own (no ``torchrun``), it joins the trainer ranks through a rendezvous file instead, as the
reference's source does with its NCCL-id file (tools/distributed/run_rollout_nccl_to_pp_tp_ppo.sh):

``python -m cverl_b200.cli.rollout_batch_source --id-file /tmp/rollout.id --rank 0 --world-size 3 --target-ranks 1,2``

with the trainer ranks given ``--rollout-nccl-id-file /tmp/rollout.id --rollout-nccl-world-size 3
--rollout-nccl-rank-offset 1 --rollout-nccl-source-rank 0``.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

from ..parallel.collectives import TorchDistCollectives
from ..rollout.gpu_batch_transport import GpuBatchReceiver, GpuBatchSender, GpuRolloutBatch


def make_batch(step: int, batch_size: int, prompt_len: int, response_len: int, weight_version: int,
               device, with_ref_log_probs: bool = False) -> GpuRolloutBatch:
    if min(batch_size, prompt_len, response_len) <= 0:
        raise ValueError("batch, prompt_len, and response_len must be positive")
    row = torch.arange(batch_size, device=device)
    even = (row % 2 == 0)
    ones = torch.ones(batch_size, response_len, device=device)
    extra = {"ref_log_probs": torch.full((batch_size, response_len), -1.0, device=device)} if with_ref_log_probs else {}
    return GpuRolloutBatch(step, weight_version, prompt_len, response_len, {
        "prompt_ids": torch.arange(1, batch_size * prompt_len + 1, device=device).view(batch_size, prompt_len),
        "response_ids": torch.arange(100, 100 + batch_size * response_len, device=device).view(batch_size,
                                                                                                 response_len),
        "response_mask": ones.clone(),
        "advantages": torch.where(even.view(-1, 1), ones, -ones),
        "old_log_probs": torch.zeros(batch_size, response_len, device=device),
        "rewards": even.float(),
        "group_ids": row // 2,
        **extra,
    })


def main(argv=None) -> int:
    import torch.distributed as dist
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--target-ranks", default="")
    ap.add_argument("--receive-from", type=int, default=-1)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--prompt-len", type=int, default=32)
    ap.add_argument("--response-len", type=int, default=8)
    ap.add_argument("--weight-version", type=int, default=0)
    ap.add_argument("--backend", default="nccl", choices=["nccl", "gloo"])
    ap.add_argument("--id-file", default="", help="rendezvous file: join a communicator without torchrun")
    ap.add_argument("--rank", type=int, default=0, help="with --id-file: this process's rank in that communicator")
    ap.add_argument("--world-size", type=int, default=0, help="with --id-file: its size")
    ap.add_argument("--device", type=int, default=0, help="with --id-file and nccl: CUDA device index")
    ap.add_argument("--with-ref-log-probs", action="store_true", help="also send reference log-probs (for --kl-coef)")
    a = ap.parse_args(argv)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    local = int(os.environ.get("LOCAL_RANK", str(a.device)))
    if a.id_file:
        from ..parallel.file_rendezvous import FileRendezvousCollectives
        device = torch.device("cuda", local) if a.backend == "nccl" else torch.device("cpu")
        comm = FileRendezvousCollectives(a.id_file, a.rank, a.world_size, device)
    elif a.backend == "nccl":
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=device)
        comm = TorchDistCollectives()
    else:
        device = torch.device("cpu")
        dist.init_process_group("gloo")
        comm = TorchDistCollectives()
    rank, world = comm.rank(), comm.world_size()
    targets = [int(t) for t in a.target_ranks.split(",") if t]
    for step in range(1, a.steps + 1):
        if a.receive_from >= 0:
            b = GpuBatchReceiver(comm, device).recv(a.receive_from)
            print(f"trainer rank {rank} step {b.step} received batch={b.batch} weight_version={b.weight_version} "
                  f"reward_sum={float(b.tensors['rewards'].sum()):.1f}", flush=True)
        else:
            batch = make_batch(step, a.batch, a.prompt_len, a.response_len, a.weight_version + step, device,
                               a.with_ref_log_probs)
            sender = GpuBatchSender(comm, device)
            for peer in targets:
                if not (0 <= peer < world) or peer == rank:
                    raise ValueError("invalid target rank")
                sender.send(batch, peer)
            print(f"rollout source step {step} sent batch={a.batch} prompt_len={a.prompt_len} "
                  f"response_len={a.response_len} targets={len(targets)}", flush=True)
        comm.barrier()
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
