"""Rollout batches sent rank to rank as device tensors, and the trainer-side ingress queue.

Wire format (reference: src/rollout/nccl_gpu_batch_transport.cc:12-17,119-190,273-344): a
fixed 73-word int64 header ``{magic 'CVRLBATC', version 2, step, batch, prompt_len,
response_len, weight_version, payload_mode, n, 8 x {kind, dtype, ndim, shape[4], rsvd}}``
sent as a tensor of the transport's device, then either one message per tensor ("direct")
or one per dtype slab ("slab", ``CVERL_GPU_BATCH_NCCL_MODE=slab``).  The receiver reads the
header on the host to learn the shapes.  The eight tensor kinds are prompt_ids,
response_ids, response_mask, old_log_probs, rewards, advantages, group_ids, ref_log_probs.
"""
from __future__ import annotations

import os
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Optional

import torch

from ..parallel.collectives import Collectives
from .gpu_ipc import TENSOR_KINDS

MAGIC = int.from_bytes(b"CVRLBATC", "little")
VERSION = 2
HEADER_WORDS = 73
_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.int64, torch.int32, torch.uint8]


@dataclass
class GpuRolloutBatch:
    step: int = 0
    weight_version: int = 0
    prompt_len: int = 0
    response_len: int = 0
    tensors: Dict[str, torch.Tensor] = field(default_factory=dict)

    @property
    def batch(self) -> int:
        for t in self.tensors.values():
            return t.shape[0]
        return 0


def _mode() -> int:
    return 1 if os.environ.get("CVERL_GPU_BATCH_NCCL_MODE", "direct") == "slab" else 0


def _header(b: GpuRolloutBatch, mode: int) -> torch.Tensor:
    h = [0] * HEADER_WORDS
    h[0:9] = [MAGIC, VERSION, b.step, b.batch, b.prompt_len, b.response_len, b.weight_version, mode, len(b.tensors)]
    for i, (kind, t) in enumerate(b.tensors.items()):
        if kind not in TENSOR_KINDS:
            raise ValueError(f"unknown rollout tensor kind {kind}")
        if t.dim() > 4 or t.dtype not in _DTYPES:
            raise ValueError("rollout tensors have at most 4 dims and a supported dtype")
        base = 9 + 8 * i
        h[base] = TENSOR_KINDS.index(kind)
        h[base + 1] = _DTYPES.index(t.dtype)
        h[base + 2] = t.dim()
        for d, s in enumerate(t.shape):
            h[base + 3 + d] = s
    return torch.tensor(h, dtype=torch.int64)


class GpuBatchSender:
    def __init__(self, comm: Collectives, device):
        self.comm, self.device = comm, torch.device(device)

    def send(self, batch: GpuRolloutBatch, dst: int) -> None:
        if len(batch.tensors) > 8:
            raise ValueError("at most 8 tensors per rollout batch")
        mode = _mode()
        self.comm.send(_header(batch, mode).to(self.device), dst)
        tensors = [t.to(self.device).contiguous() for t in batch.tensors.values()]
        if mode == 0:
            for t in tensors:
                self.comm.send(t, dst)
        else:
            for dt in _DTYPES:
                group = [t.reshape(-1) for t in tensors if t.dtype == dt]
                if group:
                    self.comm.send(torch.cat(group), dst)


class GpuBatchReceiver:
    def __init__(self, comm: Collectives, device):
        self.comm, self.device = comm, torch.device(device)

    def recv(self, src: int) -> GpuRolloutBatch:
        like = torch.empty(HEADER_WORDS, dtype=torch.int64, device=self.device)
        h = self.comm.recv_like(like, src).cpu().tolist()          # the one device->host copy
        if h[0] != MAGIC or h[1] != VERSION:
            raise RuntimeError("rollout batch header: bad magic or version")
        step, bsz, p_len, r_len, wver, mode, n = h[2:9]
        if not (0 <= n <= 8):
            raise RuntimeError("rollout batch header: bad tensor count")
        specs = []
        for i in range(n):
            base = 9 + 8 * i
            kind, dt, nd = h[base], h[base + 1], h[base + 2]
            if not (0 <= kind < len(TENSOR_KINDS)) or not (0 <= dt < len(_DTYPES)) or not (0 <= nd <= 4):
                raise RuntimeError("rollout batch header: bad tensor descriptor")
            specs.append((TENSOR_KINDS[kind], _DTYPES[dt], tuple(h[base + 3:base + 3 + nd])))
        out = GpuRolloutBatch(step, wver, p_len, r_len)
        if mode == 0:
            for kind, dt, shape in specs:
                out.tensors[kind] = self.comm.recv_like(torch.empty(shape, dtype=dt, device=self.device), src)
        else:
            for dt in _DTYPES:
                group = [(k, s) for k, d, s in specs if d == dt]
                if not group:
                    continue
                total = sum(int(torch.Size(s).numel()) for _, s in group)
                slab = self.comm.recv_like(torch.empty(total, dtype=dt, device=self.device), src)
                off = 0
                for k, s in group:
                    n_el = int(torch.Size(s).numel())
                    out.tensors[k] = slab[off:off + n_el].view(s)
                    off += n_el
            out.tensors = {k: out.tensors[k] for k, _, _ in specs}
        if out.batch != bsz:
            raise RuntimeError("rollout batch header: batch size does not match the payload")
        return out


class TrainerIngressQueue:
    """Bounded FIFO of received batches (single consumer, not thread-safe, as in the reference)."""

    def __init__(self, capacity: int = 2):
        if capacity <= 0:
            raise ValueError("capacity must be positive")
        self.capacity = capacity
        self._q: Deque[GpuRolloutBatch] = deque()

    def __len__(self) -> int:
        return len(self._q)

    def full(self) -> bool:
        return len(self._q) >= self.capacity

    def push(self, batch: GpuRolloutBatch) -> bool:
        if self.full():
            return False
        self._q.append(batch)
        return True

    def pop(self) -> Optional[GpuRolloutBatch]:
        return self._q.popleft() if self._q else None
