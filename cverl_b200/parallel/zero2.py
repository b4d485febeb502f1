"""ZeRO-2 with per-layer gradient buckets reduced while the backward pass runs.

``FlatZeroOptimizer`` keeps a full fp32 gradient twin of the flat parameter buffer and reduce-scatters
it once after the backward pass.  Here the gradient memory is one buffer per *bucket in flight*
(``FlatParams(grad_buckets=...)``: a bucket per layer on two or three rotating buffers, plus one pinned
buffer for the embedding / head), and a bucket is reduce-scattered into this rank's persistent fp32
shard gradient as soon as the backward pass has left its layer - on a side stream, overlapping the
next layer's backward kernels.  A 30 B-parameter model then needs 61 GB of bf16 parameters, 1/dp of
12 bytes per parameter for the shard (gradient, two moments) and a few bucket buffers, instead of
another 122 GB of fp32 gradients.

Shard layout: every bucket is split evenly over the data-parallel ranks (rank r owns elements
``[r * chunk_b, (r + 1) * chunk_b)`` of bucket b), so each reduce-scatter is balanced; a rank's
optimizer state is the concatenation of its pieces in bucket order.  This differs from the single
contiguous range of the flat ZeRO-1 shard on purpose: with one contiguous range a layer's bucket
would have a single owner and its reduction would be limited by that one GPU's inbound links.

Two transports: library collectives (NCCL ``reduce_scatter_tensor`` / ``all_gather_into_tensor``; gloo
for the CPU tests), or the peer-memory kernels (``FusedZero2Comm``): ``cvb_reduce_scatter_acc`` pulls
the piece from every peer's bucket buffer and accumulates it into the shard gradient, and ``cvb_flat_adamw_allgather`` stores the updated bf16 piece into every peer's parameter
buffer.

The reference reduce-scatters the whole flat gradient after the backward pass, optionally in
buckets but never overlapped with it (src/distributed/optimizer_sharding.cc:463-585), and keeps
full gradients; its ``--dp-grad-comm-dtype model`` halves them.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import _native as nv
from ..ops import optim as optim_ops
from ..ops.gemm import count_launch
from ..optim.adamw import AdamWOptions


class _Boundary(torch.autograd.Function):
    """Identity on the residual stream (``delta``, optional ``resid``) whose backward reports to the optimizer."""

    @staticmethod
    def forward(ctx, opt, bucket, delta, resid):
        ctx.opt, ctx.bucket = opt, bucket
        if resid is None:
            return delta.view_as(delta)
        return delta.view_as(delta), resid.view_as(resid)

    @staticmethod
    def backward(ctx, *grads):
        ctx.opt.on_boundary(ctx.bucket)
        if len(grads) == 1:
            return None, None, grads[0], None
        return None, None, grads[0], grads[1]


class FusedZero2Comm:
    """Peer-mapped placement of the parameter buffer and of every gradient bucket buffer, for the kernels.

    ``allocator`` is the hook ``FlatParams`` calls (collective over the group, same order on every rank): the
    bf16 parameter buffer first, then each fp32 gradient buffer.
    """

    def __init__(self, heap, max_blocks: int = 0, zero_by_reader: bool = False):
        from .symm import SymmBarrier
        self.heap = heap
        self.zero_by_reader = zero_by_reader
        self.params = None
        self.param_flat: Optional[torch.Tensor] = None
        self._grad_bufs: Dict[int, object] = {}          # local base pointer -> SymmBuffer
        self.barrier = SymmBarrier(heap)                 # used on the side stream only (one epoch sequence)
        self.barrier_main = SymmBarrier(heap)            # used on the main stream only
        self.max_blocks = max_blocks                     # CTAs of a reduce-scatter that overlaps the backward pass

    def allocator(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        if self.params is None:
            if dtype != torch.bfloat16:
                raise TypeError("the fused ZeRO path keeps model parameters in bf16")
            self.params = self.heap.alloc(numel * 2)
            self.param_flat = self.params.tensor(numel, torch.bfloat16)
            return self.param_flat
        if dtype != torch.float32:
            raise TypeError("gradient buffers are fp32")
        buf = self.heap.alloc(max(numel, 4) * 4)
        t = buf.tensor(numel, torch.float32)
        self._grad_bufs[t.data_ptr()] = buf
        return t

    def reduce_scatter_acc(self, bucket_grad: torch.Tensor, begin: int, n: int, scale: float,
                           out: torch.Tensor) -> None:
        """On the current stream: barrier, pull + accumulate, barrier, clear (the bucket buffer is free after it).
        ``zero_by_reader`` lets the pulling kernel clear what it read instead (no separate pass over the bucket,
        but the zeros then cross NVLink: worthwhile only while the links have room)."""
        buf = self._grad_bufs[bucket_grad.data_ptr()]
        self.barrier()
        nv.check(nv.cuda().cvb_reduce_scatter_acc(buf.ptr_array(), self.heap.world, self.heap.index, begin, n, scale,
                                                  out.data_ptr(), int(self.zero_by_reader), self.max_blocks,
                                                  nv.stream()), "cvb_reduce_scatter_acc")
        count_launch()
        self.barrier()
        if not self.zero_by_reader:
            bucket_grad.zero_()

    def adamw_allgather(self, o: AdamWOptions, step: int, grad, master, m, v, clip, begin: int) -> None:
        nv.check(nv.cuda().cvb_flat_adamw_allgather(grad.data_ptr(), nv.ptr(master), m.data_ptr(), v.data_ptr(),
                                                    nv.ptr(clip), self.params.ptr_array(), self.heap.world,
                                                    self.heap.index, begin, grad.numel(), o.lr, o.beta1, o.beta2,
                                                    o.eps, o.weight_decay, step, nv.stream()),
                 "cvb_flat_adamw_allgather")
        count_launch()


class _AdamFacade:
    """What the checkpoint writer asks of ``FlatZeroOptimizer.adam``."""

    def __init__(self, opt):
        self._opt = opt

    @property
    def master(self):
        return self._opt.master

    @property
    def parameter_shard(self):
        return self._opt.master if self._opt.master is not None else self._opt.fp.flat[:0]

    @property
    def step_count(self):
        return self._opt.step_count


class BucketedZero2Optimizer:
    """AdamW over bucket-sharded state; gradients are reduced bucket by bucket during the backward pass.

    Usage: build the model with ``grad_buckets=True, bucket_align=dp * 8``, construct this with the model, run
    forward / backward as usual (any number of micro-batches), call ``step()``.  ``last_metrics`` is the
    3-float device tensor ``[local_sq, global_sq, clip_scale]`` of ``FlatZeroOptimizer``.
    """

    def __init__(self, model, options: AdamWOptions, *, dp_group=None, dp_rank: int = 0, dp_size: int = 1,
                 norm_group=None, norm_world: int = 1, max_grad_norm: float = 1.0, fused_comm=None,
                 overlap: bool = True, comm_dtype: Optional[torch.dtype] = None):
        """``comm_dtype`` (library transports only): reduce the buckets in this dtype instead of fp32 - bf16 halves the
        gradient traffic, the sum still lands in the fp32 shard gradient (the reference's ``--dp-grad-comm-dtype``,
        src/distributed/optimizer_sharding.cc:463-585)."""
        options.validate("BucketedZero2Optimizer")
        self.comm_dtype = comm_dtype if comm_dtype not in (None, torch.float32) else None
        if self.comm_dtype is not None and fused_comm is not None:
            raise ValueError("the peer-memory kernels reduce in fp32; use comm_dtype with the library transports")
        fp = model.flat
        if not fp.bucketed:
            raise ValueError("BucketedZero2Optimizer needs a model built with grad_buckets=True")
        self.model, self.fp, self.options = model, fp, options
        self.dp_group, self.dp_rank, self.dp_size = dp_group, dp_rank, dp_size
        self.norm_group, self.norm_world = norm_group, norm_world
        self.max_grad_norm = max_grad_norm
        self.fused = fused_comm
        if fused_comm is not None and fused_comm.param_flat is not fp.flat:
            raise RuntimeError("the fused path needs FlatParams allocated by FusedZero2Comm.allocator")
        dev = fp.flat.device
        self.device = dev
        self.chunk: Dict[int, int] = {}
        self.piece_off: Dict[int, int] = {}
        off = 0
        for b in fp.bucket_ids:
            lo, hi = fp.bucket_ranges[b]
            if (hi - lo) % (dp_size * 4):
                raise ValueError("bucket lengths must be multiples of 4 * dp (build the model with "
                                 "bucket_align = dp * 8 and pad_multiple = dp * 8)")
            self.chunk[b] = (hi - lo) // dp_size
            self.piece_off[b] = off
            off += self.chunk[b]
        self.shard_numel = off
        # nominal position of this rank's shard in the rank-major concatenation of all shards (checkpoint metadata;
        # the pieces themselves are spread over the buckets)
        self.begin, self.end = dp_rank * off, (dp_rank + 1) * off
        self.adam = _AdamFacade(self)
        self._bucket_params: Dict[int, list] = {b: [] for b in fp.bucket_ids}
        for p in list(fp.params.values()) + list(getattr(model, "fused", {}).values()):
            at = (p.data_ptr() - fp.flat.data_ptr()) // fp.flat.element_size()
            self._bucket_params[fp.bucket_of_offset(at)].append(p)
        self.grad_shard = torch.zeros(off, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros(off, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(off, dtype=torch.float32, device=dev)
        self.master = None
        if options.use_master_weights:
            self.master = torch.cat([self._param_piece(b).float() for b in fp.bucket_ids])
        self.step_count = 0
        self.last_metrics = torch.zeros(3, dtype=torch.float32, device=dev)
        self._cuda = dev.type == "cuda"
        self.overlap = overlap and self._cuda and dp_size > 1
        self.side = torch.cuda.Stream(device=dev) if self.overlap else None
        self._slot_free: Dict[int, torch.cuda.Event] = {}     # slot -> event after which the buffer is zero and idle
        self._active: List[int] = []                          # layer buckets written in this pass, not yet reduced
        self._tmp: Optional[torch.Tensor] = None
        self.reduced_buckets = 0                              # reductions launched from inside the backward pass
        # ``pre_reduce(bucket)``: runs on the main stream once a bucket's gradients are complete and before they are
        # reduced over the data-parallel group - the place for the model-parallel sums of that bucket (tensor-parallel
        # shares of replicated parameters, the context-parallel sum)
        self.pre_reduce = getattr(model, "sync_bucket_grads", None)
        model.backward_boundary = self._boundary

    # ---- layout ---------------------------------------------------------------------------------------------
    def _param_piece(self, b: int) -> torch.Tensor:
        lo, _ = self.fp.bucket_ranges[b]
        c = self.chunk[b]
        return self.fp.flat[lo + self.dp_rank * c: lo + (self.dp_rank + 1) * c]

    def _piece(self, t: torch.Tensor, b: int) -> torch.Tensor:
        return t[self.piece_off[b]: self.piece_off[b] + self.chunk[b]]

    # ---- backward-pass hooks ----------------------------------------------------------------------------------
    def _boundary(self, delta, resid, bucket: int):
        if not (delta.requires_grad or (resid is not None and resid.requires_grad)):
            return delta, resid
        out = _Boundary.apply(self, bucket, delta, resid)
        return (out, None) if resid is None else out

    def on_boundary(self, k: int) -> None:
        """Backward reached the boundary in front of layer bucket ``k``: that bucket is complete, and bucket
        ``k - 1`` is about to be written."""
        last = self.fp.bucket_ids[-1]
        if 1 <= k <= last:
            self._reduce(k)
            self.reduced_buckets += 1
        if k - 1 >= 1:
            self._acquire(k - 1)

    def _acquire(self, b: int) -> None:
        slot = self.fp.grad_slot_of.get(b)
        if self.overlap and slot is not None and slot in self._slot_free:
            torch.cuda.current_stream(self.device).wait_event(self._slot_free[slot])
        if b not in self._active:
            self._active.append(b)

    def _fold_autograd(self, b: int) -> None:
        """Parameters whose gradient came through autograd (ops without a native kernel) instead of ``main_grad``."""
        for p in self._bucket_params[b]:
            if p.grad is not None:
                p.main_grad.add_(p.grad.float())
                p.grad = None

    def _reduce(self, b: int) -> None:
        if b in self._active:
            self._active.remove(b)
        self._fold_autograd(b)
        if self.pre_reduce is not None:
            self.pre_reduce(b)
        g = self.fp.bucket_grad(b)
        c = self.chunk[b]
        out = self._piece(self.grad_shard, b)
        if self.dp_size == 1:
            out.add_(g)
            g.zero_()
            return
        import torch.distributed as dist
        slot = self.fp.grad_slot_of.get(b)
        main = torch.cuda.current_stream(self.device) if self._cuda else None
        if self.overlap:
            ready = torch.cuda.Event()
            ready.record(main)
            self.side.wait_event(ready)
            ctx = torch.cuda.stream(self.side)
        else:
            import contextlib
            ctx = contextlib.nullcontext()
        with ctx:
            if self.fused is not None:
                self.fused.reduce_scatter_acc(g, self.dp_rank * c, c, 1.0 / self.dp_size, out)
            elif self._cuda:
                cd = self.comm_dtype or torch.float32
                if self._tmp is None or self._tmp.numel() < c or self._tmp.dtype != cd:
                    self._tmp = torch.empty(max(self.chunk.values()), dtype=cd, device=self.device)
                tmp = self._tmp[:c]
                src = g if self.comm_dtype is None else g.to(cd)
                if self.comm_dtype is None:
                    dist.reduce_scatter_tensor(tmp, src, op=dist.ReduceOp.AVG, group=self.dp_group)
                    out.add_(tmp)
                else:       # low-precision sum, mean taken in fp32
                    dist.reduce_scatter_tensor(tmp, src, op=dist.ReduceOp.SUM, group=self.dp_group)
                    out.add_(tmp.float(), alpha=1.0 / self.dp_size)
                g.zero_()
            else:   # gloo has no reduce-scatter: all-reduce the bucket and keep this rank's piece
                full = g.clone() if self.comm_dtype is None else g.to(self.comm_dtype)
                dist.all_reduce(full, group=self.dp_group)
                out.add_(full[self.dp_rank * c:(self.dp_rank + 1) * c].float() / self.dp_size)
                g.zero_()
            if self.overlap:
                done = torch.cuda.Event()
                done.record(self.side)
                if slot is not None:
                    self._slot_free[slot] = done

    def finish_backward(self) -> None:
        """Reduce whatever the boundaries have not (the first layer when its input needs no gradient, the pinned
        bucket), then make the current stream wait for the side stream."""
        for b in sorted(self._active, reverse=True):
            self._reduce(b)
        for b in self.fp.bucket_ids:
            if b not in self.fp.grad_slot_of:
                self._reduce(b)
        if self.overlap:
            torch.cuda.current_stream(self.device).wait_stream(self.side)

    # ---- the step ---------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self) -> None:
        import torch.distributed as dist
        self.finish_backward()
        o = self.options
        local_sq = optim_ops.sumsq(self.grad_shard)
        global_sq = local_sq
        if self.norm_world > 1:
            global_sq = local_sq.clone()
            dist.all_reduce(global_sq, group=self.norm_group)
        clip = optim_ops.clip_scale(global_sq, self.max_grad_norm)
        use_clip = clip if self.max_grad_norm > 0 else None
        self.step_count += 1
        fp = self.fp
        for b in fp.bucket_ids:
            lo, hi = fp.bucket_ranges[b]
            c = self.chunk[b]
            g, m, v = (self._piece(t, b) for t in (self.grad_shard, self.exp_avg, self.exp_avg_sq))
            master = self._piece(self.master, b) if self.master is not None else None
            if self.fused is not None and self.dp_size > 1:
                self.fused.adamw_allgather(o, self.step_count, g, master, m, v, use_clip, lo + self.dp_rank * c)
                continue
            optim_ops.flat_adamw_step(g, master, self._param_piece(b), m, v, clip=use_clip, lr=o.lr, beta1=o.beta1,
                                      beta2=o.beta2, eps=o.eps, weight_decay=o.weight_decay, step=self.step_count)
            if self.dp_size > 1:
                piece = self._param_piece(b)
                if self._cuda:
                    dist.all_gather_into_tensor(fp.flat[lo:hi], piece, group=self.dp_group)
                else:
                    parts = [torch.empty_like(piece) for _ in range(self.dp_size)]
                    dist.all_gather(parts, piece.clone(), group=self.dp_group)
                    fp.flat[lo:hi].copy_(torch.cat(parts))
        if self.fused is not None and self.dp_size > 1:
            self.fused.barrier_main()        # every rank's stores have landed before the next forward reads them
        self.grad_shard.zero_()
        self.last_metrics = torch.cat([local_sq.reshape(1), global_sq.reshape(1), clip[:1]])

    @torch.no_grad()
    def all_gather_params(self) -> None:
        """Rebuild the full parameter buffer from every rank's pieces (after loading a checkpoint)."""
        import torch.distributed as dist
        if self.dp_size == 1:
            return
        for b in self.fp.bucket_ids:
            lo, hi = self.fp.bucket_ranges[b]
            piece = self._param_piece(b).clone()
            if self._cuda:
                dist.all_gather_into_tensor(self.fp.flat[lo:hi], piece, group=self.dp_group)
            else:
                parts = [torch.empty_like(piece) for _ in range(self.dp_size)]
                dist.all_gather(parts, piece, group=self.dp_group)
                self.fp.flat[lo:hi].copy_(torch.cat(parts))

    # ---- checkpoint state -------------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        shard = self.master if self.master is not None else torch.cat([self._param_piece(b)
                                                                      for b in self.fp.bucket_ids])
        return {"flat_param_shard": shard.detach().clone(), "flat_exp_avg": self.exp_avg.detach().clone(),
                "flat_exp_avg_sq": self.exp_avg_sq.detach().clone(),
                "optim_step": torch.tensor(self.step_count, dtype=torch.int64),
                "bucket_chunks": torch.tensor([self.chunk[b] for b in self.fp.bucket_ids], dtype=torch.int64)}

    def load_state_dict(self, sd: dict) -> None:
        chunks = [int(x) for x in sd["bucket_chunks"]]
        if chunks != [self.chunk[b] for b in self.fp.bucket_ids]:
            raise ValueError("checkpoint was written with another bucket layout or data-parallel size")
        shard = sd["flat_param_shard"].to(self.device)
        for b in self.fp.bucket_ids:
            self._param_piece(b).copy_(self._piece(shard, b).to(self.fp.flat.dtype))
        if self.master is not None:
            self.master.copy_(shard.float())
        self.exp_avg.copy_(sd["flat_exp_avg"].to(self.device))
        self.exp_avg_sq.copy_(sd["flat_exp_avg_sq"].to(self.device))
        self.step_count = int(sd["optim_step"])
