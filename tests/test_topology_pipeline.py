"""Topology bijection, groups, layer ranges, NCCL env, 1F1B schedule (Python and the C++ twin)."""
import ctypes as C
import subprocess

import pytest

from cverl_b200 import _native as nv
from cverl_b200.parallel.pipeline import (PipelineActionType, pipeline_1f1b_schedule, pipeline_peers,
                                          pipeline_schedule_max_live_activations)
from cverl_b200.parallel.topology import (ClusterSpec, NetworkPolicy, ParallelDims, Topology,
                                          cluster_spec_from_env)


def _topo(dp, pp, cp, tp, ep, rank=0, mb=None, gpn=8):
    d = ParallelDims(dp, pp, cp, tp, ep, 1, mb or pp)
    return Topology(d, ClusterSpec(world_size=d.world, rank=rank, gpus_per_node=gpn))


def test_rank_bijection_32_and_64():
    for dims in [(2, 2, 2, 2, 2), (4, 2, 1, 4, 2)]:
        t = _topo(*dims)
        seen = set()
        for r in range(t.dims.world):
            dp, pp, cp, tp, ep = t.coords_of(r)
            assert t.rank_of(dp, pp, cp, tp, ep) == r
            seen.add((dp, pp, cp, tp, ep))
        assert len(seen) == t.dims.world


def test_ep_innermost_then_tp():
    t = _topo(2, 2, 1, 2, 2)
    assert t.coords_of(1) == (0, 0, 0, 0, 1)
    assert t.coords_of(2) == (0, 0, 0, 1, 0)
    info = t.rank_info(5)
    assert info.expert_group == [4, 5]
    assert info.tensor_group == [5, 7] or info.tensor_group == [4 + 1 - 0, 7]  # tp stride = ep size
    assert sorted(info.model_group) == list(range(0, 8))
    assert info.data_group == [5, 13]


def test_groups_partition_world():
    t = _topo(2, 2, 2, 2, 1)
    for axis in ("data", "pipeline", "context", "tensor"):
        flat = sorted(r for g in t.all_groups(axis) for r in g)
        assert flat == list(range(16))


def test_invalid_configs():
    with pytest.raises(ValueError):
        Topology(ParallelDims(2, 1, 1, 1, 1), ClusterSpec(world_size=3))
    with pytest.raises(ValueError):
        Topology(ParallelDims(1, 1, 1, 16, 1), ClusterSpec(world_size=16, gpus_per_node=8))
    with pytest.raises(ValueError):
        Topology(ParallelDims(1, 4, 1, 1, 1, 1, 2), ClusterSpec(world_size=4))
    with pytest.raises(ValueError):
        Topology(ParallelDims(1, 1, 1, 4, 1, 3, 1), ClusterSpec(world_size=4))


def test_layer_ranges_remainder_early():
    t = _topo(1, 4, 1, 1, 1, mb=4)
    assert [t.pipeline_layer_range(26, r) for r in range(4)] == [(0, 7), (7, 14), (14, 20), (20, 26)]
    with pytest.raises(ValueError):
        t.pipeline_layer_range(3, 0)


def test_nccl_env_and_cluster_env():
    t = Topology(ParallelDims(), ClusterSpec(), network=NetworkPolicy(enable_nvls=False, socket_ifname="eth0"))
    env = t.nccl_env()
    assert env["NCCL_NVLS_ENABLE"] == "0" and env["NCCL_SOCKET_IFNAME"] == "eth0"
    assert env["NCCL_ASYNC_ERROR_HANDLING"] == "1"
    c = cluster_spec_from_env({"WORLD_SIZE": "16", "RANK": "9", "CVERL_GPUS_PER_NODE": "8"})
    assert (c.world_size, c.rank, c.local_rank, c.node_rank) == (16, 9, 1, 1)


def test_1f1b_schedule_and_live():
    s = pipeline_1f1b_schedule(0, 4, 6)
    assert [a.micro_batch for a in s[:3]] == [0, 1, 2] and all(a.type == PipelineActionType.FORWARD for a in s[:3])
    assert pipeline_schedule_max_live_activations(s, 6) == 4
    last = pipeline_1f1b_schedule(3, 4, 6)
    assert pipeline_schedule_max_live_activations(last, 6) == 1
    assert [(a.type.value[0], a.micro_batch) for a in last[:4]] == [("f", 0), ("b", 0), ("f", 1), ("b", 1)]
    with pytest.raises(ValueError):
        pipeline_1f1b_schedule(0, 4, 3)
    with pytest.raises(ValueError):
        pipeline_schedule_max_live_activations(s[:-1], 6)
    p = pipeline_peers([3, 7, 11], 1)
    assert (p.prev_rank, p.next_rank) == (3, 11)
    assert pipeline_peers([3, 7, 11], 0).prev_rank == -1


def test_cpp_twin_matches_python():
    lib = nv.host()
    dims = (C.c_int64 * 7)(2, 2, 2, 2, 2, 1, 2)
    t = _topo(2, 2, 2, 2, 2)
    for rank in (0, 5, 13, 31):
        out = (C.c_int64 * 5)()
        assert lib.cverl_topology_coords(dims, C.c_int64(32), C.c_int64(8), C.c_int64(rank), out) == 0
        assert tuple(out) == t.coords_of(rank)
        for axis, name in enumerate(["data", "pipeline", "context", "tensor", "expert"]):
            buf, cnt = (C.c_int64 * 64)(), C.c_int64()
            assert lib.cverl_topology_group(dims, C.c_int64(32), C.c_int64(8), C.c_int64(rank), axis, buf,
                                            C.c_int64(64), C.byref(cnt)) == 0
            assert list(buf[:cnt.value]) == getattr(t.rank_info(rank), name + "_group")
    types, micro = (C.c_int32 * 64)(), (C.c_int64 * 64)()
    cnt, live = C.c_int64(), C.c_int64()
    assert lib.cverl_pipeline_1f1b(C.c_int64(1), C.c_int64(4), C.c_int64(6), types, micro, C.c_int64(64),
                                   C.byref(cnt), C.byref(live)) == 0
    py = pipeline_1f1b_schedule(1, 4, 6)
    assert [(int(types[i]), int(micro[i])) for i in range(cnt.value)] == \
        [(0 if a.type == PipelineActionType.FORWARD else 1, a.micro_batch) for a in py]
    assert live.value == pipeline_schedule_max_live_activations(py, 6)
    assert lib.cverl_pipeline_1f1b(C.c_int64(0), C.c_int64(4), C.c_int64(2), types, micro, C.c_int64(64),
                                   C.byref(cnt), C.byref(live)) == 1


def test_cpp_twin_agrees_on_random_layouts():
    """The C++ planner and the Python one over 300 random layouts, valid and invalid: same verdict on validity,
    same coordinates, same groups on every axis, same layer ranges, same 1F1B action list and peak live count."""
    import random
    rng = random.Random(7)
    lib = nv.host()
    axes = ["data", "pipeline", "context", "tensor", "expert"]
    valid = invalid = 0
    for _ in range(300):
        dp, pp, cp, tp, ep = (rng.choice([1, 1, 2, 3, 4]) for _ in range(5))
        sp = rng.choice([1, 1, 1, tp, 2])
        mb = rng.choice([pp, pp, pp + 1, 2 * pp, max(pp - 1, 0), 0])
        gpn = rng.choice([1, 2, 4, 8])
        world = dp * pp * cp * tp * ep
        if rng.random() < 0.1:
            world += 1                                  # a world that the layout does not tile
        dims = (C.c_int64 * 7)(dp, pp, cp, tp, ep, sp, mb)
        rank = rng.randrange(0, max(world, 1))
        out = (C.c_int64 * 5)()
        rc = lib.cverl_topology_coords(dims, C.c_int64(world), C.c_int64(gpn), C.c_int64(rank), out)
        try:
            t = Topology(ParallelDims(dp, pp, cp, tp, ep, sp, mb), ClusterSpec(world_size=world, rank=rank, gpus_per_node=gpn))
            py_ok = True
        except ValueError:
            py_ok = False
        assert (rc == 0) == py_ok, (dp, pp, cp, tp, ep, sp, mb, gpn, world, rc, py_ok)
        if not py_ok:
            invalid += 1
            continue
        valid += 1
        assert tuple(out) == t.coords_of(rank)
        info = t.rank_info(rank)
        for axis, name in enumerate(axes):
            buf, cnt = (C.c_int64 * 256)(), C.c_int64()
            assert lib.cverl_topology_group(dims, C.c_int64(world), C.c_int64(gpn), C.c_int64(rank), axis, buf,
                                            C.c_int64(256), C.byref(cnt)) == 0
            assert list(buf[:cnt.value]) == getattr(info, name + "_group")
        layers = rng.randrange(pp, 70)
        b, e = C.c_int64(), C.c_int64()
        assert lib.cverl_pipeline_layer_range(C.c_int64(layers), C.c_int64(pp), C.c_int64(info.pipeline_rank),
                                              C.byref(b), C.byref(e)) == 0
        assert (b.value, e.value) == tuple(t.pipeline_layer_range(layers, info.pipeline_rank))
        types, micro = (C.c_int32 * 128)(), (C.c_int64 * 128)()
        cnt, live = C.c_int64(), C.c_int64()
        assert lib.cverl_pipeline_1f1b(C.c_int64(info.pipeline_rank), C.c_int64(pp), C.c_int64(mb), types, micro,
                                       C.c_int64(128), C.byref(cnt), C.byref(live)) == 0
        py = pipeline_1f1b_schedule(info.pipeline_rank, pp, mb)
        assert [(int(types[i]), int(micro[i])) for i in range(cnt.value)] == \
            [(0 if a.type == PipelineActionType.FORWARD else 1, a.micro_batch) for a in py]
        assert live.value == pipeline_schedule_max_live_activations(py, mb)
    assert valid > 60 and invalid > 30, (valid, invalid)


def test_parallel_plan_cli():
    from cverl_b200._build import LIB_DIR
    out = subprocess.run([str(LIB_DIR / "cverl_parallel_plan"), "--dp", "2", "--pp", "2", "--tp", "2", "--rank", "5",
                          "--layers", "24", "--micro-batches", "4"], capture_output=True, text=True, check=True).stdout
    assert "rank=5 dp=1 pp=0 cp=0 tp=1 ep=0" in out
    assert "schedule=F0 F1 B0 F2 B1 F3 B2 B3" in out
    assert "layer_begin=0 layer_end=12" in out
    assert "world_size=8" in out and "parallel=dp2_pp2_cp1_tp2_ep1_sp1" in out and "micro_batches=4" in out
    # the reference's spellings: --num-layers, --all-ranks (every rank's block), --help
    every = subprocess.run([str(LIB_DIR / "cverl_parallel_plan"), "--dp", "2", "--pp", "2", "--all-ranks", "--num-layers",
                            "6", "--micro-batches", "4", "--local-rank", "1", "--local-world-size", "4", "--schedule"],
                           capture_output=True, text=True, check=True).stdout
    assert every.count("\nrank=") == 4 and "rank=3 dp=1 pp=1" in every and "layer_begin=3 layer_end=6" in every
    assert every.count("max_live_activations=2") == 2 and every.count("max_live_activations=1") == 2
    quiet = subprocess.run([str(LIB_DIR / "cverl_parallel_plan"), "--pp", "2", "--no-schedule"], capture_output=True,
                           text=True, check=True).stdout
    assert "schedule=" not in quiet and "max_live_activations=" in quiet
    usage = subprocess.run([str(LIB_DIR / "cverl_parallel_plan"), "--help"], capture_output=True, text=True, check=True)
    assert "--all-ranks" in usage.stdout and "--num-layers" in usage.stdout
    bad = subprocess.run([str(LIB_DIR / "cverl_parallel_plan"), "--pp", "4", "--micro-batches", "2"], capture_output=True,
                         text=True)
    assert bad.returncode == 1 and "cverl_parallel_plan:" in bad.stderr
