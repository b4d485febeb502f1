"""Every collective of a communication backend checked against its closed-form result, one process per rank.

    # the native NCCL communicator, formed through an id file - no launcher needed beyond starting the processes
    python -m cverl_b200.cli.collectives_smoke --rank R --world-size N --device D --id-file /tmp/nccl.id
    # torch.distributed (NCCL on GPUs, gloo on CPU), under torchrun or any launcher that sets RANK / WORLD_SIZE
    python -m cverl_b200.cli.collectives_smoke --backend torch [--cpu]

Checks (reference: tests/distributed/test_nccl_collectives.cc:76-352, run by tools/distributed/run_nccl_smoke.sh):
all-reduce sum / mean / max in fp32 and bf16, broadcast from a non-zero root, all-gather and reduce-scatter on
dim 0, all-to-all, send / recv in both directions, the ring ``send_recv``, refusal of non-contiguous inputs and of a
dim 0 the group does not divide, a sub-group (the first half of the world: all-reduce and reduce-scatter inside it,
refusal for a non-member), int64 payloads, a barrier.  Prints ``collectives smoke passed`` on rank 0.
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import List, Optional, Sequence

import torch

from ..parallel.collectives import Collectives, ReduceOp


def run_checks(comm: Collectives, dev: torch.device, ensure_group=None) -> List[str]:
    """Runs every check on ``comm``; returns the list of check names that ran (raises on a mismatch)."""
    rank, world = comm.rank(), comm.world_size()
    done: List[str] = []
    close = torch.testing.assert_close
    base = torch.arange(8, device=dev, dtype=torch.float32)
    x = base + rank * 10
    close(comm.all_reduce(x, ReduceOp.SUM), base * world + 10.0 * sum(range(world)))
    close(comm.all_reduce(x.bfloat16(), ReduceOp.MEAN).float(), base + 5.0 * (world - 1), rtol=1e-2, atol=1e-1)
    assert float(comm.all_reduce(x, ReduceOp.MAX)[0]) == 10.0 * (world - 1)
    done += ["all_reduce_sum", "all_reduce_mean_bf16", "all_reduce_max"]
    root = world - 1
    close(comm.broadcast(x, root), base + 10.0 * root)
    done.append("broadcast")
    g = comm.all_gather(x.view(2, 4))
    assert g.shape == (2 * world, 4) and [float(g[2 * p, 0]) for p in range(world)] == [10.0 * p for p in range(world)]
    rs = comm.reduce_scatter(torch.ones(4 * world, 3, device=dev) * (rank + 1), ReduceOp.SUM)
    assert rs.shape == (4, 3) and float(rs[0, 0]) == sum(r + 1 for r in range(world))
    a2a = comm.all_to_all(torch.full((2 * world, 2), float(rank), device=dev))
    assert [float(a2a[2 * p, 0]) for p in range(world)] == [float(p) for p in range(world)]
    done += ["all_gather", "reduce_scatter", "all_to_all"]
    if world > 1:
        ids = torch.arange(6, device=dev, dtype=torch.int64) + 100 * rank
        peer = rank ^ 1
        if peer < world:                       # pairs (0,1), (2,3), ...: the even rank sends first
            if rank % 2 == 0:
                comm.send(ids, peer)
                got = comm.recv_like(ids, peer)
            else:
                got = comm.recv_like(ids, peer)
                comm.send(ids, peer)
            assert int(got[0]) == 100 * peer and got.dtype == torch.int64
        ring = comm.send_recv(x, (rank + 1) % world, x, (rank - 1) % world)
        assert float(ring[0]) == 10.0 * ((rank - 1) % world)
        done += ["send_recv_pairs_int64", "ring_send_recv"]
    for bad, what in ((lambda: comm.all_reduce(x.view(2, 4).t()), "non-contiguous input"),
                      (lambda: comm.reduce_scatter(torch.ones(world + 1, device=dev)) if world > 1 else _raise(),
                       "dim 0 not divisible by the group")):
        try:
            bad()
        except (ValueError, RuntimeError):
            continue
        raise AssertionError(f"{what} was not refused")
    done.append("refusals")
    half: Sequence[int] = list(range(max(world // 2, 1)))
    if ensure_group is not None:
        ensure_group(half)                     # collective over the world: members and non-members both call it
    if rank in half:
        close(comm.all_reduce(x, ReduceOp.SUM, group=half), base * len(half) + 10.0 * sum(half))
        sub = comm.reduce_scatter(torch.ones(2 * len(half), device=dev) * (rank + 1), ReduceOp.SUM, group=half)
        assert sub.shape == (2,) and float(sub[0]) == sum(r + 1 for r in half)
    elif ensure_group is not None:
        try:
            comm.all_reduce(x, ReduceOp.SUM, group=half)
        except (ValueError, RuntimeError):
            pass
        else:
            raise AssertionError("a non-member used a sub-group")
    done.append("sub_group")
    comm.barrier()
    done.append("barrier")
    return done


def _raise():
    raise ValueError("skipped at world size 1")


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--backend", default="native", choices=["native", "torch"])
    ap.add_argument("--rank", type=int, default=int(os.environ.get("RANK", "0")))
    ap.add_argument("--world-size", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--device", type=int, default=int(os.environ.get("LOCAL_RANK", "0")))
    ap.add_argument("--id-file", default=os.environ.get("CVERL_NCCL_ID_FILE", ""))
    ap.add_argument("--id-timeout-s", type=float, default=60.0)
    ap.add_argument("--sync-after-op", action="store_true", help="native backend: synchronise after every collective")
    ap.add_argument("--cpu", action="store_true", help="torch backend on gloo / CPU")
    a = ap.parse_args(argv)
    if a.backend == "native":
        if not a.id_file:
            raise SystemExit("--backend native needs --id-file (rank 0 writes it, the others wait for it)")
        from ..parallel.nccl_backend import NcclCollectives
        dev = torch.device("cuda", a.device)
        torch.cuda.set_device(dev)
        comm = NcclCollectives(a.rank, a.world_size, dev, id_file=a.id_file, sync_after_op=a.sync_after_op,
                               id_timeout_s=a.id_timeout_s)
        try:
            done = run_checks(comm, dev, ensure_group=comm.ensure_group)
            torch.cuda.synchronize()
        finally:
            comm.close()
    else:
        import torch.distributed as dist
        from ..parallel.collectives import TorchDistCollectives
        use_cuda = torch.cuda.is_available() and not a.cpu
        dev = torch.device("cuda", a.device) if use_cuda else torch.device("cpu")
        if use_cuda:
            torch.cuda.set_device(dev)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29530")
        dist.init_process_group("nccl" if use_cuda else "gloo", rank=a.rank, world_size=a.world_size)
        comm = TorchDistCollectives()
        done = run_checks(comm, dev, ensure_group=lambda g: comm.pg(g))
        dist.barrier()
        dist.destroy_process_group()
    if a.rank == 0:
        print(f"collectives smoke passed: backend={a.backend} world={a.world_size} checks={','.join(done)}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
