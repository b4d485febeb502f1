"""Micro-benchmarks of the fused compute + collective kernels against their NCCL counterparts.

``torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m cverl_b200.bench_collectives [--numel E]``

One process per GPU.  Every case is timed with CUDA events on the launching stream after a barrier, 3 warm-ups,
``--iters`` timed runs, and reported as the MAX over ranks (rank 0 prints one JSON line per case):

* ``zero_rs``   reduce-scatter (mean) of the fp32 gradient buffer + squared norm of the shard:
                one pull kernel over peer memory (``cvb_reduce_scatter_sumsq``, between two flag barriers)
                vs ``reduce_scatter_tensor`` + a norm kernel.
* ``zero_ag``   AdamW on the shard + all-gather of the bf16 parameters: one kernel whose stores go to every
                peer (``cvb_flat_adamw_allgather``) vs the local AdamW kernel + ``all_gather_into_tensor``.
* ``tp_gemm``   row-parallel linear, GEMM + all-reduce: the tcgen05 GEMM whose epilogue stores each tile into
                every peer's slot, a flag barrier and a local sum, vs the same GEMM + NCCL all-reduce.
* ``tp_sp``     one tensor-parallel layer half with the token-sharded residual stream: row-parallel GEMM whose
                epilogue reduce-scatters its tiles to their owners, residual add + RMSNorm on this rank's rows,
                all-gather of the normalised rows overlapped with the column-parallel GEMM on the local rows
                (``parallel/tp_sp.py``), vs GEMM + NCCL all-reduce + add-RMSNorm on all rows + GEMM.
* ``push``      weight push of the bf16 parameter buffer from rank i to rank i + N/2 by peer stores
                (``cvb_broadcast_store``) vs NCCL send / recv.

``link_frac`` is the bytes that must cross NVLink per GPU and direction divided by the time and by 770 GB/s (the
measured peer-copy bandwidth of this pool); for ``tp_gemm`` the roofline time is the slower of FLOPs / measured
GEMM peak and bytes / 770 GB/s, and ``roofline_frac`` = that time / measured time.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

LINK_GBS = 770.0


def _time(fn, iters, group):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ms = []
    for _ in range(iters):
        dist.barrier(group)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    t = torch.tensor([sum(ms) / len(ms)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--numel", type=int, default=752 * 1024 * 1024, help="parameters (0.8B model: 7.5e8)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=40960)
    ap.add_argument("--what", default="zero_rs,zero_ag,tp_gemm,tp_sp,push")
    a = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    from . import _native as nv
    from .ops import optim as optim_ops
    from .optim import AdamWOptions
    from .optim.adamw import FlatAdamW
    from .parallel.symm import FusedZeroComm, P2pBroadcaster, SymmetricHeap

    def report(**kw):
        if rank == 0:
            print(json.dumps(kw), flush=True)

    n = a.numel // (world * 8) * (world * 8)
    shard = n // world
    begin = rank * shard
    what = set(a.what.split(","))
    heap = SymmetricHeap(group, dev)

    if what & {"zero_rs", "zero_ag"} and world > 1:
        fc = FusedZeroComm(heap)
        params = fc.allocator(n, torch.bfloat16)
        grads = fc.allocator(n, torch.float32)
        params.normal_(0, 0.02)
        gshard = torch.empty(shard, dtype=torch.float32, device=dev)
        out = torch.empty(shard, dtype=torch.float32, device=dev)
        adam = FlatAdamW(params[begin:begin + shard], AdamWOptions(lr=1e-6, beta2=0.95, use_master_weights=False))
        if "zero_rs" in what:
            def fused_rs():
                grads.fill_(1e-3)   # (the fused call zeroes the buffer afterwards, as the optimizer needs)
                fc.reduce_scatter_mean_sumsq(gshard, begin)

            def nccl_rs():
                grads.fill_(1e-3)
                dist.reduce_scatter_tensor(out, grads, op=dist.ReduceOp.AVG, group=group)
                optim_ops.sumsq(out)
                grads.zero_()

            def fill_only():
                grads.fill_(1e-3)
            t_fill = _time(fill_only, a.iters, group)
            tf, tn = _time(fused_rs, a.iters, group) - t_fill, _time(nccl_rs, a.iters, group) - t_fill
            link_bytes = (world - 1) * shard * 4          # pulled from every peer
            report(case="zero_rs", n_gpus=world, numel=n, fused_ms=tf, nccl_ms=tn,
                   link_gbs=link_bytes / tf / 1e6, link_frac=link_bytes / tf / 1e6 / LINK_GBS,
                   note="reduce-scatter(mean) + sumsq + zeroing of the 4-byte gradient buffer")
        if "zero_ag" in what:
            clip = torch.ones(1, device=dev)

            def fused_ag():
                fc.adamw_allgather(adam, gshard, clip, begin)

            def nccl_ag():
                adam.step(gshard, clip=clip)
                dist.all_gather_into_tensor(params, params[begin:begin + shard], group=group)
            gshard.fill_(1e-3)
            tf, tn = _time(fused_ag, a.iters, group), _time(nccl_ag, a.iters, group)
            link_bytes = (world - 1) * shard * 2          # stored to every peer
            report(case="zero_ag", n_gpus=world, numel=n, fused_ms=tf, nccl_ms=tn,
                   link_gbs=link_bytes / tf / 1e6, link_frac=link_bytes / tf / 1e6 / LINK_GBS,
                   note="AdamW on the shard (24 B / element local traffic) + all-gather of bf16 parameters")
        nv.check_status(dev)

    if "tp_gemm" in what and world > 1:
        from .ops import gemm_nt
        from .parallel.tp_symm import TpSymm
        M, N, K = a.tokens, 1024, max(64, 2048 // world)  # out_proj of the 0.8B model: K = 2048 split over TP
        tp = TpSymm(group, dev, M, N)
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02

        def fused():
            tp.reduce_gemm_nt(x, w)

        def nccl():
            y = gemm_nt(x, w)
            dist.all_reduce(y, group=group)
        tf, tn = _time(fused, a.iters, group), _time(nccl, a.iters, group)
        flops = 2.0 * M * N * K
        link_bytes = (world - 1) * M * N * 2
        peak = 1627e12
        try:
            from .bench_kernels import _peaks
            peak = _peaks()["bf16_tflops"] * 1e12
        except Exception:
            pass
        roof_ms = max(flops / peak, link_bytes / (LINK_GBS * 1e9)) * 1e3
        report(case="tp_gemm", n_gpus=world, M=M, N=N, K=K, fused_ms=tf, nccl_ms=tn, roofline_ms=roof_ms,
               roofline_frac=roof_ms / tf, link_gbs=link_bytes / tf / 1e6)
        nv.check_status(dev)

    if "tp_sp" in what and world > 1 and a.tokens % (128 * world) == 0:
        from . import ops
        from .ops import gemm_nt
        from .parallel import tp_sp
        M, H, K, N2 = a.tokens, 1024, max(64, 2048 // world), 7168 // world   # out_proj -> norm -> gate|up
        sp = tp_sp.TpSp(group, dev, M, H, arena_slots=1)
        rl = M // world
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w1 = torch.randn(H, K, device=dev, dtype=torch.bfloat16) * 0.02
        w2 = torch.randn(N2, H, device=dev, dtype=torch.bfloat16) * 0.02
        wn = torch.zeros(H, device=dev, dtype=torch.bfloat16)
        resid_l = torch.randn(rl, H, device=dev, dtype=torch.bfloat16)
        resid_f = torch.randn(M, H, device=dev, dtype=torch.bfloat16)

        def fused():
            with torch.no_grad():
                sp.slot = 0
                parts = tp_sp.row_linear(x, w1, sp)
                full, _ = tp_sp.norm_gather(parts, resid_l, wn, 1e-6, 1.0, sp, True)
                tp_sp.col_linear(full, w2, sp)

        def nccl():
            with torch.no_grad():
                y = gemm_nt(x, w1)
                dist.all_reduce(y, group=group)
                n1, _ = ops.add_rmsnorm(y, resid_f, wn, 1e-6, 1.0)
                gemm_nt(n1, w2)
        tf, tn = _time(fused, a.iters, group), _time(nccl, a.iters, group)
        flops = 2.0 * M * H * K + 2.0 * M * N2 * H
        link_bytes = 2 * (world - 1) * rl * H * 2         # reduce-scatter out + all-gather out, per GPU
        peak = 1627e12
        try:
            from .bench_kernels import _peaks
            peak = _peaks()["bf16_tflops"] * 1e12
        except Exception:
            pass
        roof_ms = max(flops / peak, link_bytes / (LINK_GBS * 1e9)) * 1e3
        report(case="tp_sp", n_gpus=world, M=M, H=H, K=K, N2=N2, fused_ms=tf, nccl_ms=tn, roofline_ms=roof_ms,
               roofline_frac=roof_ms / tf, compute_ms=flops / peak * 1e3, link_ms=link_bytes / (LINK_GBS * 1e6),
               note="row GEMM -> RS (epilogue) -> add+RMSNorm on T/n rows -> AG (copy engines) || column GEMM")
        nv.check_status(dev)

    if "push" in what and world > 1 and world % 2 == 0:
        nbytes = n * 2
        pb = P2pBroadcaster(heap, nbytes)
        src = torch.empty(n, dtype=torch.bfloat16, device=dev).normal_()
        dst = pb.tensor(n, torch.bfloat16)
        half = world // 2

        def fused():
            if rank < half:
                pb.push(src, [rank + half])
            pb.sync()

        def nccl():
            if rank < half:
                dist.send(src, rank + half, group=group)
            else:
                dist.recv(dst, rank - half, group=group)
        tf, tn = _time(fused, a.iters, group), _time(nccl, a.iters, group)
        report(case="push", n_gpus=world, bytes=nbytes, fused_ms=tf, nccl_ms=tn, link_gbs=nbytes / tf / 1e6,
               link_frac=nbytes / tf / 1e6 / LINK_GBS, note=f"{half} trainers -> {half} rollout ranks, one copy each")
        nv.check_status(dev)
    if "nvls" in what and world > 1:
        # the same collectives through the NVSwitch multicast address (multimem.st / multimem.ld_reduce)
        from .parallel import nvls
        try:
            rs = nvls.NvlsReduceScatter(group, dev, n)
        except RuntimeError as exc:
            report(case="nvls", n_gpus=world, unavailable=str(exc))
            rs = None
        if rs is not None:
            gshard = torch.empty(shard, dtype=torch.float32, device=dev)
            out = torch.empty(shard, dtype=torch.float32, device=dev)

            def mm_rs():
                rs.reduce(gshard, begin)

            def nccl_rs():
                dist.reduce_scatter_tensor(out, rs.grad, op=dist.ReduceOp.AVG, group=group)
                optim_ops.sumsq(out)
            rs.grad.fill_(1e-3 * (rank + 1))
            tf, tn = _time(mm_rs, a.iters, group), _time(nccl_rs, a.iters, group)
            dist.reduce_scatter_tensor(out, rs.grad, op=dist.ReduceOp.AVG, group=group)
            err = float((out - gshard).abs().max())
            report(case="nvls_zero_rs", n_gpus=world, numel=n, fused_ms=tf, nccl_ms=tn, max_abs_diff=err,
                   egress_gbs=(world - 1) * shard * 4 / tf / 1e6,
                   note="reduce-scatter(mean) + sumsq; the sum is formed in the switch, each GPU receives its shard "
                        "once and still ships (n-1)/n of its buffer")
            del rs, gshard, out
            torch.cuda.empty_cache()
            nbytes = n * 2
            bc = nvls.NvlsBroadcaster(group, dev, nbytes)
            src = torch.empty(n, dtype=torch.bfloat16, device=dev).normal_()
            dst = bc.tensor(n, torch.bfloat16)
            part = n // world // 8 * 8

            def mm_push():          # every rank multicasts its 1/n of the weights: the parameter all-gather
                bc.push(src[rank * part:(rank + 1) * part], rank * part * 2)
                bc.sync()

            def mm_push_one():      # one sender, everyone receives: the 1 -> n weight broadcast
                if rank == 0:
                    bc.push(src, 0)
                bc.sync()

            def nccl_bcast():
                dist.broadcast(src if rank == 0 else dst, 0, group=group)

            def nccl_ag():
                dist.all_gather_into_tensor(dst[:part * world], src[rank * part:(rank + 1) * part], group=group)
            t1, t2 = _time(mm_push_one, a.iters, group), _time(nccl_bcast, a.iters, group)
            report(case="nvls_push_1_to_n", n_gpus=world, bytes=nbytes, fused_ms=t1, nccl_ms=t2,
                   egress_gbs=nbytes / t1 / 1e6, link_frac=nbytes / t1 / 1e6 / LINK_GBS,
                   note="one multimem.st per 16 bytes on rank 0; the switch delivers to every rank")
            t3, t4 = _time(mm_push, a.iters, group), _time(nccl_ag, a.iters, group)
            report(case="nvls_allgather", n_gpus=world, bytes=nbytes, fused_ms=t3, nccl_ms=t4,
                   ingress_gbs=(world - 1) * part * 2 / t3 / 1e6,
                   link_frac=(world - 1) * part * 2 / t3 / 1e6 / LINK_GBS,
                   note="every rank multicasts its shard: egress 1/n of the buffer, ingress (n-1)/n")
            del bc, src, dst
            torch.cuda.empty_cache()
            m = a.tokens * 1024
            ar = nvls.NvlsAllReduce(group, dev, m)
            x = torch.empty(m, dtype=torch.bfloat16, device=dev).normal_()

            def mm_ar():
                ar.all_reduce()

            def nccl_ar():
                dist.all_reduce(x, group=group)
            t5, t6 = _time(mm_ar, a.iters, group), _time(nccl_ar, a.iters, group)
            report(case="nvls_allreduce_bf16", n_gpus=world, numel=m, fused_ms=t5, nccl_ms=t6,
                   note="[tokens, 1024] bf16 partial sums: ld_reduce + multimem.st of each rank's slice")
        nv.check_status(dev)
    dist.barrier(group)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
