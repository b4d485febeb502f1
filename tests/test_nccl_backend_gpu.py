"""The native NCCL communicator (``nccl/nccl_backend.cc`` + ``parallel/nccl_backend.py``) on two GPUs: rendezvous
through an id file, every collective in both completion modes, a split sub-communicator."""
import os
import tempfile

import pytest
import torch

from tests.dist_utils import run_ranks

pytestmark = pytest.mark.gpu


def _nccl_backend_rank(rank, world, id_dir):
    from cverl_b200.parallel.collectives import ReduceOp
    from cverl_b200.parallel.nccl_backend import NcclCollectives
    dev = torch.device("cuda", rank)
    for mode, sync in (("async", False), ("sync", True)):
        comm = NcclCollectives(rank, world, dev, id_file=os.path.join(id_dir, f"nccl_{mode}.id"), sync_after_op=sync,
                               id_timeout_s=30.0)
        assert comm.rank() == rank and comm.world_size() == world
        x = torch.arange(8, device=dev, dtype=torch.float32) + rank * 10
        s = comm.all_reduce(x, ReduceOp.SUM)
        torch.testing.assert_close(s, torch.arange(8, device=dev).float() * world + 10.0 * sum(range(world)))
        m = comm.all_reduce(x.bfloat16(), ReduceOp.MEAN)
        torch.testing.assert_close(m.float(), (torch.arange(8, device=dev).float() + 5.0), rtol=1e-2, atol=1e-2)
        assert float(comm.all_reduce(x, ReduceOp.MAX)[0]) == 10.0 * (world - 1)
        b = comm.broadcast(x, 1)
        torch.testing.assert_close(b, torch.arange(8, device=dev).float() + 10.0)
        g = comm.all_gather(x.view(2, 4))
        assert g.shape == (2 * world, 4) and float(g[2, 0]) == 10.0
        rs = comm.reduce_scatter(torch.ones(4 * world, 3, device=dev) * (rank + 1), ReduceOp.SUM)
        assert rs.shape == (4, 3) and float(rs[0, 0]) == sum(r + 1 for r in range(world))
        a2a = comm.all_to_all(torch.full((2 * world, 2), float(rank), device=dev))
        assert [float(a2a[2 * p, 0]) for p in range(world)] == [float(p) for p in range(world)]
        ids = torch.arange(6, device=dev, dtype=torch.int64) + 100 * rank
        if rank == 0:
            comm.send(ids, 1)
            got = comm.recv_like(ids, 1)
        else:
            got = comm.recv_like(ids, 0)
            comm.send(ids, 0)
        assert int(got[0]) == 100 * (1 - rank)
        ring = comm.send_recv(x, (rank + 1) % world, x, (rank - 1) % world)
        assert float(ring[0]) == 10.0 * ((rank - 1) % world)
        with pytest.raises(ValueError):
            comm.all_reduce(x.view(2, 4).t())                    # non-contiguous input is refused
        with pytest.raises(ValueError):
            comm.reduce_scatter(torch.ones(3, device=dev))        # dim 0 not divisible by the group
        # a sub-communicator of one rank: collective split, the non-member gets nothing
        comm.ensure_group([0])
        if rank == 0:
            solo = comm.all_reduce(x, ReduceOp.SUM, group=[0])
            torch.testing.assert_close(solo, x)
        else:
            with pytest.raises(ValueError):
                comm.all_reduce(x, ReduceOp.SUM, group=[0])
        comm.barrier()
        torch.cuda.synchronize()
        comm.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_native_nccl_backend_two_gpus():
    with tempfile.TemporaryDirectory() as d:
        run_ranks(_nccl_backend_rank, 2, d, backend="nccl", timeout=240)


def test_nccl_id_file_round_trip_and_timeout(tmp_path):
    """The id-file rendezvous itself needs only the library: atomic write, read back, and a bounded wait."""
    from cverl_b200.parallel import nccl_backend as nb
    uid = nb.create_unique_id()
    assert len(uid) == 128
    path = str(tmp_path / "comm.id")
    nb.write_unique_id_file(path, uid)
    assert nb.read_unique_id_file(path, timeout_s=1.0) == uid and not os.path.exists(path + ".tmp")
    with pytest.raises(TimeoutError):
        nb.read_unique_id_file(str(tmp_path / "never.id"), timeout_s=0.2)
