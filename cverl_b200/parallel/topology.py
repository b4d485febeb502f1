"""Rank <-> (dp, pp, cp, tp, ep) topology, groups, layer ranges and NCCL environment.

Same bijection and validation as the reference (src/distributed/topology.cc:
53-224): ``rank = ((((dp*PP + pp)*CP + cp)*TP + tp)*EP + ep`` (EP innermost,
then TP), world == dp*pp*cp*tp*ep, tp within one node, micro_batches >= pp,
contiguous layer ranges with the remainder on the early stages.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass
class ParallelDims:
    data: int = 1
    pipeline: int = 1
    context: int = 1
    tensor: int = 1
    expert: int = 1
    sequence: int = 1  # declared (must divide tensor); Megatron-SP proper is not a trainer mode
    micro_batches: int = 1

    @property
    def world(self) -> int:
        return self.data * self.pipeline * self.context * self.tensor * self.expert


@dataclass
class ClusterSpec:
    world_size: int = 1
    rank: int = 0
    local_rank: int = 0
    local_world_size: int = 1
    node_rank: int = 0
    gpus_per_node: int = 8


@dataclass
class MemoryPolicy:
    activation_checkpointing: bool = False
    shard_optimizer_state: bool = True
    shard_gradients: bool = False
    offload_optimizer_to_cpu: bool = False
    offload_parameters_to_cpu: bool = False


@dataclass
class NetworkPolicy:
    enable_p2p: bool = True
    enable_ib: bool = True
    enable_nvls: bool = True
    socket_ifname: str = ""
    ib_hca: str = ""
    topo_file: str = ""
    ib_gid_index: int = -1


@dataclass
class ParallelRankInfo:
    global_rank: int
    data_rank: int
    pipeline_rank: int
    context_rank: int
    tensor_rank: int
    expert_rank: int
    sequence_rank: int
    data_group: List[int]
    pipeline_group: List[int]
    context_group: List[int]
    tensor_group: List[int]
    expert_group: List[int]
    sequence_group: List[int]
    model_group: List[int]


class Topology:
    def __init__(self, dims: ParallelDims, cluster: Optional[ClusterSpec] = None,
                 memory: Optional[MemoryPolicy] = None, network: Optional[NetworkPolicy] = None):
        self.dims = dims
        self.cluster = cluster or ClusterSpec(world_size=dims.world)
        self.memory = memory or MemoryPolicy()
        self.network = network or NetworkPolicy()
        self.validate()

    def validate(self) -> None:
        d = self.dims
        for name in ("data", "pipeline", "context", "tensor", "expert", "sequence", "micro_batches"):
            if getattr(d, name) <= 0:
                raise ValueError(f"parallel dimension '{name}' must be positive")
        if d.world != self.cluster.world_size:
            raise ValueError(f"world size {self.cluster.world_size} != dp*pp*cp*tp*ep = {d.world}")
        if d.tensor > self.cluster.gpus_per_node:
            raise ValueError("tensor parallel size must fit inside one node")
        if d.tensor % d.sequence:
            raise ValueError("sequence parallel size must divide tensor parallel size")
        if d.micro_batches < d.pipeline:
            raise ValueError("micro_batches must be >= pipeline parallel size")
        if not (0 <= self.cluster.rank < self.cluster.world_size):
            raise ValueError("rank out of range")

    # ---- bijection -----------------------------------------------------------
    def rank_of(self, dp: int, pp: int, cp: int, tp: int, ep: int) -> int:
        d = self.dims
        return ((((dp * d.pipeline + pp) * d.context + cp) * d.tensor + tp) * d.expert + ep)

    def coords_of(self, rank: int) -> Tuple[int, int, int, int, int]:
        d = self.dims
        if not (0 <= rank < d.world):
            raise ValueError("rank out of range")
        ep = rank % d.expert
        rank //= d.expert
        tp = rank % d.tensor
        rank //= d.tensor
        cp = rank % d.context
        rank //= d.context
        pp = rank % d.pipeline
        dp = rank // d.pipeline
        return dp, pp, cp, tp, ep

    def rank_info(self, rank: Optional[int] = None) -> ParallelRankInfo:
        d = self.dims
        rank = self.cluster.rank if rank is None else rank
        dp, pp, cp, tp, ep = self.coords_of(rank)
        sp_span = d.tensor // d.sequence
        seq_base = (tp // d.sequence) * d.sequence
        return ParallelRankInfo(
            global_rank=rank, data_rank=dp, pipeline_rank=pp, context_rank=cp, tensor_rank=tp, expert_rank=ep,
            sequence_rank=tp % d.sequence,
            data_group=[self.rank_of(i, pp, cp, tp, ep) for i in range(d.data)],
            pipeline_group=[self.rank_of(dp, i, cp, tp, ep) for i in range(d.pipeline)],
            context_group=[self.rank_of(dp, pp, i, tp, ep) for i in range(d.context)],
            tensor_group=[self.rank_of(dp, pp, cp, i, ep) for i in range(d.tensor)],
            expert_group=[self.rank_of(dp, pp, cp, tp, i) for i in range(d.expert)],
            sequence_group=[self.rank_of(dp, pp, cp, seq_base + i, ep) for i in range(d.sequence)] if sp_span else [rank],
            model_group=[self.rank_of(dp, p, c, t, e) for p in range(d.pipeline) for c in range(d.context)
                         for t in range(d.tensor) for e in range(d.expert)],
        )

    def all_groups(self, axis: str) -> List[List[int]]:
        """Every distinct group of one axis (each rank appears in exactly one)."""
        seen, out = set(), []
        for r in range(self.dims.world):
            g = tuple(getattr(self.rank_info(r), axis + "_group"))
            if g not in seen:
                seen.add(g)
                out.append(list(g))
        return out

    # ---- pipeline layer ranges ------------------------------------------------
    def pipeline_layer_range(self, num_layers: int, pipeline_rank: Optional[int] = None) -> Tuple[int, int]:
        pp = self.dims.pipeline
        r = self.rank_info().pipeline_rank if pipeline_rank is None else pipeline_rank
        if num_layers < pp:
            raise ValueError("fewer layers than pipeline stages")
        base, rem = divmod(num_layers, pp)
        begin = r * base + min(r, rem)
        return begin, begin + base + (1 if r < rem else 0)

    # ---- NCCL environment -----------------------------------------------------
    def nccl_env(self) -> Dict[str, str]:
        n = self.network
        env = {
            "NCCL_P2P_DISABLE": "0" if n.enable_p2p else "1",
            "NCCL_IB_DISABLE": "0" if n.enable_ib else "1",
            "NCCL_NVLS_ENABLE": "1" if n.enable_nvls else "0",
            "NCCL_ASYNC_ERROR_HANDLING": "1",
            "TORCH_NCCL_BLOCKING_WAIT": "0",
        }
        if n.socket_ifname:
            env["NCCL_SOCKET_IFNAME"] = n.socket_ifname
        if n.ib_hca:
            env["NCCL_IB_HCA"] = n.ib_hca
        if n.topo_file:
            env["NCCL_TOPO_FILE"] = n.topo_file
        if n.ib_gid_index >= 0:
            env["NCCL_IB_GID_INDEX"] = str(n.ib_gid_index)
        return env

    def apply_nccl_env(self) -> None:
        """Export ``nccl_env()`` (the reference builds the map but never applies it)."""
        for k, v in self.nccl_env().items():
            os.environ.setdefault(k, v)


def cluster_spec_from_env(env=None) -> ClusterSpec:
    env = os.environ if env is None else env

    def geti(name, default):
        v = env.get(name)
        return int(v) if v not in (None, "") else default

    world = geti("WORLD_SIZE", 1)
    rank = geti("RANK", 0)
    gpn = geti("CVERL_GPUS_PER_NODE", geti("LOCAL_WORLD_SIZE", min(world, 8)))
    return ClusterSpec(world_size=world, rank=rank, local_rank=geti("LOCAL_RANK", rank % max(gpn, 1)),
                       local_world_size=geti("LOCAL_WORLD_SIZE", gpn), node_rank=geti("NODE_RANK", rank // max(gpn, 1)),
                       gpus_per_node=gpn)
