"""1F1B pipeline schedule, peers, and the stage runner over NCCL p2p.

Schedule semantics follow the reference (src/distributed/pipeline.cc:41-121):
stage r of P runs ``P - r - 1`` warm-up forwards, then alternates one forward /
one backward while forwards remain, then drains the remaining backwards;
``micro_batches >= pipeline size`` is required.  ``max_live_activations``
replays a schedule, validates it (each micro-batch forwarded once before its
backward) and reports the peak number of stashed activations.

``PipelineStage`` executes the schedule for one rank: activations
``[tokens, H]`` go to the next stage and input gradients come back over
``torch.distributed`` p2p (tools/model/qwen3_5_pp_tp_ppo_trainer.cc:2272-2423),
issued on a side stream as non-blocking isend/irecv so that transfers overlap
the neighbouring micro-batch's compute.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

import torch


class PipelineActionType(enum.Enum):
    FORWARD = "forward"
    BACKWARD = "backward"


@dataclass(frozen=True)
class PipelineAction:
    type: PipelineActionType
    micro_batch: int


@dataclass(frozen=True)
class PipelinePeers:
    prev_rank: int  # global rank of the previous stage or -1
    next_rank: int  # global rank of the next stage or -1


def pipeline_1f1b_schedule(pipeline_rank: int, pipeline_size: int, micro_batches: int) -> List[PipelineAction]:
    if pipeline_size <= 0 or not (0 <= pipeline_rank < pipeline_size):
        raise ValueError("invalid pipeline rank/size")
    if micro_batches < pipeline_size:
        raise ValueError("1F1B requires micro_batches >= pipeline size")
    warmup = min(pipeline_size - pipeline_rank - 1, micro_batches)
    steady = micro_batches - warmup
    actions: List[PipelineAction] = []
    f = b = 0
    for _ in range(warmup):
        actions.append(PipelineAction(PipelineActionType.FORWARD, f))
        f += 1
    for _ in range(steady):
        actions.append(PipelineAction(PipelineActionType.FORWARD, f))
        f += 1
        actions.append(PipelineAction(PipelineActionType.BACKWARD, b))
        b += 1
    while b < micro_batches:
        actions.append(PipelineAction(PipelineActionType.BACKWARD, b))
        b += 1
    return actions


def pipeline_schedule_max_live_activations(actions: Sequence[PipelineAction], micro_batches: int) -> int:
    fwd_done, bwd_done = set(), set()
    live = peak = 0
    for a in actions:
        if not (0 <= a.micro_batch < micro_batches):
            raise ValueError("micro-batch index out of range in schedule")
        if a.type == PipelineActionType.FORWARD:
            if a.micro_batch in fwd_done:
                raise ValueError("micro-batch forwarded twice")
            fwd_done.add(a.micro_batch)
            live += 1
            peak = max(peak, live)
        else:
            if a.micro_batch not in fwd_done or a.micro_batch in bwd_done:
                raise ValueError("backward without a matching forward")
            bwd_done.add(a.micro_batch)
            live -= 1
    if len(fwd_done) != micro_batches or len(bwd_done) != micro_batches:
        raise ValueError("schedule does not cover every micro-batch")
    return peak


def pipeline_peers(pipeline_group: Sequence[int], pipeline_rank: int) -> PipelinePeers:
    n = len(pipeline_group)
    if not (0 <= pipeline_rank < n):
        raise ValueError("pipeline rank out of range")
    return PipelinePeers(pipeline_group[pipeline_rank - 1] if pipeline_rank > 0 else -1,
                         pipeline_group[pipeline_rank + 1] if pipeline_rank + 1 < n else -1)


class PipelineStage:
    """Runs one rank's 1F1B schedule.

    ``forward_fn(micro_batch, stage_input or None) -> stage_output`` runs this
    stage's layers (the first stage ignores the input and embeds tokens);
    ``loss_fn(micro_batch, stage_output) -> (tensor_to_backward, grad_seed)`` is
    called on the last stage only.  Activation shape and dtype are fixed by
    ``act_shape`` / ``act_dtype`` so receives can be posted ahead of time.
    """

    def __init__(self, peers: PipelinePeers, pipeline_rank: int, pipeline_size: int, micro_batches: int,
                 act_shape, act_dtype, device, group=None):
        self.peers = peers
        self.rank, self.size, self.micro_batches = pipeline_rank, pipeline_size, micro_batches
        self.act_shape, self.act_dtype, self.device = tuple(act_shape), act_dtype, device
        self.group = group
        self.schedule = pipeline_1f1b_schedule(pipeline_rank, pipeline_size, micro_batches)
        self.max_live = pipeline_schedule_max_live_activations(self.schedule, micro_batches)
        self._comm_stream = torch.cuda.Stream(device=device) if torch.device(device).type == "cuda" else None
        self._keep = []

    @property
    def first(self) -> bool:
        return self.rank == 0

    @property
    def last(self) -> bool:
        return self.rank == self.size - 1

    # -- p2p helpers: work on the side stream, hand over with events ------------
    def _send(self, t: torch.Tensor, dst: int):
        import torch.distributed as dist
        t = t.contiguous()
        if self._comm_stream is None:
            # never block on a send: in steady-state 1F1B both neighbours send at the same time
            req = dist.isend(t, dst=dst, group=self.group)
            self._keep.append(t)
            return req
        self._comm_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._comm_stream):
            t.record_stream(self._comm_stream)
            return dist.isend(t, dst=dst, group=self.group)

    def _recv(self, src: int) -> torch.Tensor:
        import torch.distributed as dist
        buf = torch.empty(self.act_shape, dtype=self.act_dtype, device=self.device)
        if self._comm_stream is None:
            dist.recv(buf, src=src, group=self.group)
            return buf
        self._comm_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._comm_stream):
            buf.record_stream(self._comm_stream)
            req = dist.irecv(buf, src=src, group=self.group)
            req.wait()
        torch.cuda.current_stream().wait_stream(self._comm_stream)
        return buf

    def run(self, forward_fn: Callable, loss_fn: Optional[Callable] = None) -> Dict[int, torch.Tensor]:
        """Executes the schedule; returns the last stage's per-micro-batch loss outputs."""
        self._keep = []
        stash: Dict[int, tuple] = {}
        results: Dict[int, torch.Tensor] = {}
        pending = []
        for act in self.schedule:
            m = act.micro_batch
            if act.type == PipelineActionType.FORWARD:
                x = None
                if not self.first:
                    x = self._recv(self.peers.prev_rank).requires_grad_(True)
                out = forward_fn(m, x)
                if self.last:
                    stash[m] = (x, out)
                else:
                    pending.append(self._send(out.detach(), self.peers.next_rank))
                    stash[m] = (x, out)
            else:
                x, out = stash.pop(m)
                if self.last:
                    target, seed = loss_fn(m, out)
                    results[m] = target.detach()
                    target.backward(seed)
                else:
                    g = self._recv(self.peers.next_rank)
                    out.backward(g)
                if not self.first:
                    pending.append(self._send(x.grad, self.peers.prev_rank))
        for req in pending:
            if req is not None:
                req.wait()
        if self._comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self._comm_stream)
        return results
