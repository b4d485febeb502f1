"""Process-group handles of one rank for every parallel axis the model code sees."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional


@dataclass
class ParallelContext:
    """Groups are ``torch.distributed`` process groups (``None`` = axis of size 1)."""

    tp_group: Optional[Any] = None
    tp_rank: int = 0
    tp_size: int = 1
    ep_group: Optional[Any] = None
    ep_rank: int = 0
    ep_size: int = 1
    cp_group: Optional[Any] = None
    cp_rank: int = 0
    cp_size: int = 1
    dp_group: Optional[Any] = None
    dp_rank: int = 0
    dp_size: int = 1
    pp_rank: int = 0
    pp_size: int = 1
    # the ranks of one model replica (pp x cp x tp x ep): the non-sharded optimizer modes sum their gradient norm here
    model_group: Optional[Any] = None
    # fused NVLink kernels (symmetric-memory paths) instead of NCCL for TP / ZeRO
    fused_comm: bool = False
    # ``parallel.tp_symm.TpSymm`` when tensor-parallel linears fuse their all-reduce into the GEMM
    tp_symm: Optional[Any] = None
    # ``parallel.tp_sp.TpSp`` when the tensor-parallel group shards the residual stream by token rows and fuses the
    # reduce-scatter / all-gather halves of every all-reduce into the GEMM epilogue and the norm kernels
    tp_sp: Optional[Any] = None
    # ``parallel.ep_symm.EpSymm`` when expert-parallel dispatch / combine run over peer-mapped memory
    ep_symm: Optional[Any] = None
    # ``parallel.cp_symm.CpSymm`` when context-parallel attention pulls K / V from peers instead of a ring
    cp_symm: Optional[Any] = None
    # context-parallel attention over a zig-zag resharding of q | k | v (``parallel.cp_zigzag``): every rank does
    # the same amount of causal attention work; off = contiguous shards, rank r attends r + 1/2 key blocks
    cp_zigzag: bool = False

    @property
    def single(self) -> bool:
        return self.tp_size == 1 and self.ep_size == 1 and self.cp_size == 1


SINGLE = ParallelContext()
