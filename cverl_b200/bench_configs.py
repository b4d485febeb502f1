"""The benchmark configurations beside the headline one, behind ``bench.py --config NAME``.

* ``cpu_loss``        CPU fp32 GRPO / PPO loss step on [64, 512] through the public C ABI (no GPU), this library
                      against the reference's ``libcverl`` when ``baseline/_ref/lib/libcverl_ref.so`` exists.
* ``moe30b_ep8_sft``  Qwen3-30B-A3B-shaped MoE (48 layers, hidden 2048, 32 q / 4 kv heads, head dim 128, 128 experts
                      top-8, expert FFN 768, vocab 151,936), supervised step, expert parallel over all ranks,
                      sequence length 4096, 8 sequences per GPU, expert dispatch / combine over peer memory.
* ``cp8_attention``   context-parallel ring attention of the Qwen3.5-0.8B attention shape (8 q / 2 kv heads, head
                      dim 256) at 131,072 tokens, batch 1, forward + backward, standalone; then one actor step of
                      the first four layers of that model on the same sequence.
* ``zero2_dp8_push``  the same 30 B model, data parallel over all ranks, ZeRO stage 2 with per-layer gradient
                      buckets reduced during the backward pass (``parallel/zero2.py``), sequence length 2048; then
                      the trainer -> rollout push of the full bf16 weights from the first half of the ranks to the
                      second half with the ``broadcast_store`` kernel (each trainer rank stores 1 / n of the buffer
                      into every rollout rank's parameter buffer: one read, n remote stores).

Weights are initialised on the device (``Qwen35Model.init_weights_on_device``), token ids are uniform over the
vocabulary.  Every number is CUDA-event time between barrier + synchronize pairs, max over ranks, after the warm-up
steps; each run prints one JSON line in the layout of the headline benchmark.  ``--layers`` (fewer layers) marks
the line ``invalid``: it exists to try a configuration on fewer GPUs than it is sized for.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import torch

CONFIGS = ("cpu_loss", "moe30b_ep8_sft", "cp8_attention", "zero2_dp8_push")
ROOT = Path(__file__).resolve().parents[1]


def _dist_setup():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    return world, rank, local_rank, dev


def _barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def _timed(fn, steps, world, dev):
    """Milliseconds for ``steps`` calls: CUDA events between barrier + synchronize pairs, max over ranks."""
    _barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    _barrier(world)
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item()


def _finish(out, rank, world, sampler, args, launches):
    from . import _native as nv
    from .utils import fallbacks
    sampler.stop()
    nv.check_status()
    if rank == 0:
        out.update({"n_gpus": world, "steps": args.steps, "warmup": args.warmup, "dtype": "bf16",
                    "clocks": sampler.summary(), "gpu_launches": launches,
                    "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
                    "library_fallbacks": fallbacks.total(), "vs_baseline": None})
        if args.layers:
            out["invalid"] = "debug run with fewer layers"
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return 0


# ---------------------------------------------------------------------------------------------------------------
def cpu_loss(args) -> int:
    cmd = [sys.executable, "-m", "cverl_b200.bench_cpu_loss", "--iters", str(max(args.steps, 50))]
    ref = ROOT / "baseline" / "_ref" / "lib" / "libcverl_ref.so"
    if ref.exists():
        cmd += ["--other", str(ref)]
    p = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True)
    line = [ln for ln in p.stdout.splitlines() if ln.startswith("{")]
    if p.returncode != 0 or not line:
        print(json.dumps({"config": "cpu_loss", "error": (p.stderr or p.stdout)[-400:]}))
        return 1
    r = json.loads(line[-1])
    out = {"metric": "CPU fp32 GRPO/PPO loss step [64,512], microseconds per step", "value": r.get("ours_us_per_step"),
           "unit": "us/step", "reference_us_per_step": r.get("other_us_per_step"),
           "speedup_vs_reference": r.get("speedup_vs_other"), "higher_is_better": False, "n_gpus": 0, "dtype": "fp32", "data": "synthetic",
           "config": {"name": "cpu_loss", "batch": 64, "seq": 512}, "detail": r, "gpu_launches": 0}
    print(json.dumps(out))
    return 0


# ---------------------------------------------------------------------------------------------------------------
def _sft_step_fn(model, opt, ids_dev, micro_batch, extra=None):
    """One supervised step on ``ids_dev`` [B, S]: mean next-token NLL over all positions, micro-batched."""
    B, S = ids_dev.shape
    n_mb = B // micro_batch
    denom = float(B * (S - 1))

    def step():
        nll = torch.zeros((), dtype=torch.float32, device=ids_dev.device)
        for m in range(n_mb):
            ids = ids_dev[m * micro_batch:(m + 1) * micro_batch]
            lp = model.response_logprobs(ids, 1)
            seed = torch.full_like(lp, -1.0 / denom)
            lp.backward(seed)
            nll -= lp.detach().float().sum() / denom
        if extra is not None:
            extra()
        opt.step()
        return nll
    return step


def moe30b_ep8_sft(args, ClockSampler) -> int:
    from . import ops
    from .models.config import Qwen35TextConfig
    from .models.qwen3_5 import Qwen35Model
    from .optim import AdamWOptions
    from .parallel.mesh import build_context
    from .parallel.zero import FlatZeroOptimizer
    from .trainer.ppo_trainer import _average_non_expert_grads
    world, rank, local_rank, dev = _dist_setup()
    cfg = Qwen35TextConfig.qwen3_30b_a3b()
    if args.layers:
        cfg = Qwen35TextConfig(**{**{k: getattr(cfg, k) for k in cfg.__dataclass_fields__},
                                  "num_hidden_layers": args.layers, "layer_types": cfg.layer_types[:args.layers]})
    S, seqs = args.seq_len or 4096, args.seqs_per_gpu or 8
    mb = args.micro_batch or 1
    ctx = build_context(world, rank, ep=world)
    if world > 1 and args.ep_comm == "symm":
        from .parallel.ep_symm import EpSymm
        # A randomly initialised router may send many tokens of a deep layer to the same few experts; an entry that
        # does not fit its receive buffer is dropped (its rows read as zeros) and the run reports it.  Every buffer
        # and every saved activation of the expert path has the capacity's static size, so the factor is a trade
        # against memory: 3 x the balanced load keeps the 48-layer model inside 180 GB.
        cap = int(mb * S * cfg.num_experts_per_tok * args.ep_capacity_factor) + 128
        ctx.ep_symm = EpSymm(ctx.ep_group, dev, cap, cfg.hidden_size)
    model = Qwen35Model(cfg, dtype=torch.bfloat16, device=dev, ctx=ctx, pad_multiple=8)
    model.init_weights_on_device(seed=1234)
    opt = FlatZeroOptimizer(model.flat, AdamWOptions(lr=1e-6, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01,
                                                     use_master_weights=False),
                            dp_size=1, norm_group=None, norm_world=world, max_grad_norm=1.0)
    g = torch.Generator().manual_seed(1000 + rank)
    host_ids = torch.randint(0, cfg.vocab_size, (seqs, S), generator=g).pin_memory()
    ids_dev = host_ids.to(dev)
    extra = (lambda: _average_non_expert_grads(model, ctx)) if world > 1 else None
    step = _sft_step_fn(model, opt, ids_dev, mb, extra)
    _barrier(world)      # ranks finish building and initialising the model at different times; the flag barriers
    #                      inside the step are bounded waits of about a second, so line the ranks up first
    for _ in range(max(args.warmup, 0)):
        step()
    sampler = ClockSampler(local_rank)
    sampler.start()
    l0 = ops.launch_counter["n"]
    ms = _timed(step, args.steps, world, dev)
    launches = ops.launch_counter["n"] - l0
    last = {}

    def e2e():
        ids_dev.copy_(host_ids, non_blocking=True)
        last["nll"] = step().cpu()
    e2e()
    ms_e2e = _timed(e2e, args.steps, world, dev)
    tokens = seqs * S * world
    overflow = int(ctx.ep_symm.overflow.item()) if getattr(ctx, "ep_symm", None) is not None else 0
    out = {"metric": "supervised-step tokens/s (device, max over ranks)", "value": tokens / (ms / args.steps / 1e3),
           "unit": "tokens/s", "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
           "data": "synthetic uniform token ids, random-init weights (device-side initialisation)",
           "config": {"name": "moe30b_ep8_sft", "model": f"Qwen3-30B-A3B shape, {cfg.num_hidden_layers} layers",
                      "seq_len": S, "seqs_per_gpu": seqs, "micro_batch_seqs": mb, "parallelism": f"ep{world}",
                      "ep_comm": args.ep_comm if world > 1 else "none",
                      "local_params": int(model.flat.numel), "ep_receive_overflow": overflow,
                      "l2": "working set far above the 126 MB L2"},
           "e2e": {"value": tokens / (ms_e2e / args.steps / 1e3), "unit": "tokens/s",
                   "h2d_bytes_per_step": host_ids.numel() * 8, "d2h_bytes_per_step": 4,
                   "ms_per_step": ms_e2e / args.steps},
           "loss": float(last["nll"])}
    return _finish(out, rank, world, sampler, args, launches)


# ---------------------------------------------------------------------------------------------------------------
def cp8_attention(args, ClockSampler) -> int:
    from . import ops
    from .models.config import Qwen35TextConfig
    from .models.qwen3_5 import Qwen35Model
    from .optim import AdamWOptions
    from .parallel.context_parallel import ring_attention
    from .parallel.mesh import build_context
    from .parallel.zero import FlatZeroOptimizer
    world, rank, local_rank, dev = _dist_setup()
    full = Qwen35TextConfig.qwen3_5_0_8b()
    S = args.seq_len or 131072
    Hq, Hkv, D = full.num_attention_heads, full.num_key_value_heads, full.head_dim
    T = S // world
    ctx = build_context(world, rank, cp=world)
    ctx.cp_zigzag = world > 1 and args.cp_comm != "symm"
    symm = None
    if world > 1 and args.cp_comm == "symm":
        from .parallel.cp_symm import CpSymm
        symm = ctx.cp_symm = CpSymm(ctx.cp_group, dev)
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    q = torch.randn(1, Hq, T, D, device=dev, dtype=torch.bfloat16, generator=g).requires_grad_()
    k = torch.randn(1, Hkv, T, D, device=dev, dtype=torch.bfloat16, generator=g).requires_grad_()
    v = torch.randn(1, Hkv, T, D, device=dev, dtype=torch.bfloat16, generator=g).requires_grad_()
    do = torch.randn(1, Hq, T, D, device=dev, dtype=torch.bfloat16, generator=g)

    from .parallel.cp_zigzag import zigzag_ring_attention
    q4, k4, v4, do4 = (t.detach().transpose(1, 2).contiguous() for t in (q, k, v, do))
    for t in (q4, k4, v4):
        t.requires_grad_()

    def ring_fwd():
        return ring_attention(q, k, v, ctx.cp_group, rank, world, S, symm=symm, key="bench")

    def ring_fwd_bwd():
        q.grad = k.grad = v.grad = None
        ring_fwd().backward(do)

    def fwd():          # the shard IS the zig-zag layout here: random rows need no resharding
        return zigzag_ring_attention(q4, k4, v4, ctx.cp_group, rank, world)

    def fwd_bwd():
        q4.grad = k4.grad = v4.grad = None
        fwd().backward(do4)
    _barrier(world)
    for _ in range(max(args.warmup, 1)):
        fwd_bwd()
        ring_fwd_bwd()
    sampler = ClockSampler(local_rank)
    sampler.start()
    l0 = ops.launch_counter["n"]
    with torch.no_grad():
        ms_f = _timed(fwd, args.steps, world, dev) / args.steps
        ms_ring_f = _timed(ring_fwd, args.steps, world, dev) / args.steps
    ms_fb = _timed(fwd_bwd, args.steps, world, dev) / args.steps
    launches = ops.launch_counter["n"] - l0
    ms_ring_fb = _timed(ring_fwd_bwd, args.steps, world, dev) / args.steps
    flops_f = 4.0 * S * S * Hq * D / 2            # causal: half of the score matrix
    # one actor step of the first four layers (3 Gated-DeltaNet + 1 full attention) on the same sequence
    n_layers = 4
    cfg = Qwen35TextConfig(**{**{kk: getattr(full, kk) for kk in full.__dataclass_fields__},
                              "num_hidden_layers": n_layers, "layer_types": full.layer_types[:n_layers]})
    model = Qwen35Model(cfg, dtype=torch.bfloat16, device=dev, ctx=ctx, pad_multiple=8)
    model.init_weights_on_device(seed=1234)
    opt = FlatZeroOptimizer(model.flat, AdamWOptions(lr=1e-6, beta2=0.95, use_master_weights=False), dp_size=1,
                            norm_group=None, norm_world=world, max_grad_norm=1.0)
    ids = torch.randint(0, cfg.vocab_size, (1, S), generator=torch.Generator().manual_seed(5)).to(dev)
    P = 256

    def model_step():
        import torch.distributed as dist
        lp = model.response_logprobs(ids, P)
        lp.backward(torch.full_like(lp, -1.0 / lp.numel() / world))
        model.sync_replicated_grads()
        if world > 1:
            dist.all_reduce(model.flat.main_grad, group=ctx.cp_group)
        opt.step()
    for _ in range(max(args.warmup, 1)):
        model_step()
    ms_model = _timed(model_step, args.steps, world, dev) / args.steps
    out = {"metric": "context-parallel causal attention forward+backward, ms (device, max over ranks)",
           "value": ms_fb, "unit": "ms", "ms_per_step": ms_fb, "higher_is_better": False, "scaling": "strong",
           "data": "bf16 Q/K/V ~ N(0,1), batch 1",
           "config": {"name": "cp8_attention", "seq_len": S, "heads_q": Hq, "heads_kv": Hkv, "head_dim": D,
                      "parallelism": f"cp{world}", "cp_comm": args.cp_comm if world > 1 else "none",
                      "sharding": "zig-zag (value, forward_ms); the contiguous ring is reported beside it",
                      "l2": "K/V of 131,072 tokens (268 MB) exceed the L2"},
           "contiguous_ring_fwd_bwd_ms": ms_ring_fb, "contiguous_ring_forward_ms": ms_ring_f,
           "model_step_attention": "zig-zag" if ctx.cp_zigzag else "contiguous ring",
           "forward_ms": ms_f, "forward_tflops_total": flops_f / ms_f / 1e9,
           "fwd_bwd_tflops_total": 3.5 * flops_f / ms_fb / 1e9,
           "model_step_4_layers_ms": ms_model, "model_step_tokens_per_s": S / (ms_model / 1e3)}
    return _finish(out, rank, world, sampler, args, launches)


# ---------------------------------------------------------------------------------------------------------------
def zero2_dp8_push(args, ClockSampler) -> int:
    from . import ops
    from .models.config import Qwen35TextConfig
    from .models.qwen3_5 import Qwen35Model
    from .optim import AdamWOptions
    from .parallel.mesh import build_context
    from .parallel.symm import SymmetricHeap
    from .parallel.zero2 import BucketedZero2Optimizer, FusedZero2Comm
    import torch.distributed as dist
    world, rank, local_rank, dev = _dist_setup()
    cfg = Qwen35TextConfig.qwen3_30b_a3b()
    if args.layers:
        cfg = Qwen35TextConfig(**{**{k: getattr(cfg, k) for k in cfg.__dataclass_fields__},
                                  "num_hidden_layers": args.layers, "layer_types": cfg.layer_types[:args.layers]})
    S, seqs = args.seq_len or 2048, args.seqs_per_gpu or 2
    mb = args.micro_batch or 1
    ctx = build_context(world, rank, dp=world)
    comm = None
    if world > 1 and args.zero_comm == "symm":
        comm = FusedZero2Comm(SymmetricHeap(ctx.dp_group, dev), max_blocks=args.rs_blocks)
    model = Qwen35Model(cfg, dtype=torch.bfloat16, device=dev, ctx=ctx, pad_multiple=world * 8, grad_buckets=True,
                        bucket_align=world * 8, grad_slots=args.grad_slots,
                        flat_allocator=comm.allocator if comm else None)
    model.init_weights_on_device(seed=1234)
    opt = BucketedZero2Optimizer(model, AdamWOptions(lr=1e-6, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01,
                                                     use_master_weights=False),
                                 dp_group=ctx.dp_group, dp_rank=rank, dp_size=world, norm_group=None,
                                 norm_world=world, max_grad_norm=1.0, fused_comm=comm, overlap=not args.no_overlap,
                                 comm_dtype=torch.bfloat16 if (comm is None and args.grad_comm_dtype == "bfloat16")
                                 else None)
    g = torch.Generator().manual_seed(1000 + rank)
    host_ids = torch.randint(0, cfg.vocab_size, (seqs, S), generator=g).pin_memory()
    ids_dev = host_ids.to(dev)
    step = _sft_step_fn(model, opt, ids_dev, mb)
    _barrier(world)      # line the ranks up before the first bounded flag barrier (see moe30b_ep8_sft)
    for _ in range(max(args.warmup, 0)):
        step()
    sampler = ClockSampler(local_rank)
    sampler.start()
    l0, r0 = ops.launch_counter["n"], opt.reduced_buckets
    ms = _timed(step, args.steps, world, dev) / args.steps
    launches = ops.launch_counter["n"] - l0
    in_backward = (opt.reduced_buckets - r0) / max(args.steps * (seqs // mb), 1)
    last = {}

    def e2e():
        ids_dev.copy_(host_ids, non_blocking=True)
        last["nll"] = step().cpu()
    e2e()
    ms_e2e = _timed(e2e, args.steps, world, dev) / args.steps
    # exposed optimizer tail: everything from the end of the backward pass (the last buckets, norm, AdamW, gather)
    def tail_only():
        opt.step()
    ms_tail = _timed(tail_only, args.steps, world, dev) / args.steps
    # trainer -> rollout push: the first half of the ranks are trainers, the second half rollout workers; trainer t
    # stores its 1 / n of the bf16 parameter buffer into the same offsets of every rollout rank's buffer
    push = {}
    if world >= 2 and world % 2 == 0:
        import ctypes as C
        from . import _native as nv
        from .parallel.symm import SymmBarrier
        half = world // 2
        nbytes = model.flat.flat.numel() * 2
        part = (nbytes // half + 255) // 256 * 256
        opt.grad_shard = opt.exp_avg = opt.exp_avg_sq = None       # the training measurement is over: make room
        torch.cuda.empty_cache()
        src = model.flat.flat.view(torch.uint8)
        if comm is not None:
            dst_ptrs, barrier, own = comm.params.peer_ptrs, comm.barrier_main, src      # straight into the parameters
        else:
            heap = SymmetricHeap(ctx.dp_group, dev)
            recv = heap.alloc(nbytes)
            dst_ptrs, barrier, own = recv.peer_ptrs, SymmBarrier(heap), recv.tensor(nbytes, torch.uint8)
        want = torch.stack([src[:1 << 24].float().sum(), src[-(1 << 24):].float().sum()])
        if rank >= half:
            own.zero_()
        # every trainer holds the full weights: trainer t pushes the whole buffer to rollout rank half + t (one
        # stream per link pair).  --push-pattern slices: trainer t stores slice t into EVERY rollout rank instead
        # (each sender then feeds every rollout rank at once: measured 14x slower on 8 GPUs with 61 GB)
        if args.push_pattern == "pairs":
            lo, hi = 0, nbytes // 16 * 16
            dsts = [dst_ptrs[half + rank]] if rank < half else []
        else:
            lo = rank * part
            hi = min(lo + part, nbytes) // 16 * 16
            dsts = [dst_ptrs[d] + lo for d in range(half, world)]
        arr = (C.c_void_p * max(len(dsts), 1))(*dsts)

        def push_fn():
            barrier()                                  # receivers are ready (nobody still reads the old weights)
            if rank < half and hi > lo:
                nv.check(nv.cuda().cvb_broadcast_store(src[lo:hi].data_ptr(), arr, len(dsts), hi - lo, nv.stream()),
                         "cvb_broadcast_store")
                ops.launch_counter["n"] += 1
            barrier()                                  # every piece has landed
        for _ in range(2):
            push_fn()
        ms_push = _timed(push_fn, args.steps, world, dev) / args.steps
        got = torch.stack([own[:1 << 24].float().sum(), own[-(1 << 24):].float().sum()])
        sums = [torch.empty_like(got) for _ in range(world)]
        wants = [torch.empty_like(want) for _ in range(world)]
        dist.all_gather(sums, got)
        dist.all_gather(wants, want)
        ok = all(torch.equal(sums[r], wants[0]) for r in range(half, world))
        push = {"weight_push_ms": ms_push, "weight_bytes": nbytes, "trainers": half, "rollout_ranks": half,
                "per_receiver_gbs": nbytes / (ms_push / 1e3) / 1e9,
                "per_sender_gbs": (hi - lo) * len(dsts) / (ms_push / 1e3) / 1e9 if rank < half else None,
                "push_pattern": args.push_pattern, "push_verified": ok,
                "push_target": "parameter buffers" if comm is not None else "receive buffers"}
    tokens = seqs * S * world
    out = {"metric": "ZeRO-2 supervised-step tokens/s (device, max over ranks); weight-sync seconds",
           "value": tokens / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms, "higher_is_better": True,
           "scaling": "weak", "data": "synthetic uniform token ids, random-init weights (device-side initialisation)",
           "config": {"name": "zero2_dp8_push", "model": f"Qwen3-30B-A3B shape, {cfg.num_hidden_layers} layers",
                      "seq_len": S, "seqs_per_gpu": seqs, "micro_batch_seqs": mb, "parallelism": f"dp{world}",
                      "zero": "stage 2, per-layer buckets reduced during backward on a side stream",
                      "zero_comm": args.zero_comm if world > 1 else "none", "overlap": not args.no_overlap,
                      "grad_comm_dtype": args.grad_comm_dtype if comm is None else "float32", "grad_slots": args.grad_slots, "rs_blocks": args.rs_blocks if comm else None, "params": int(model.flat.numel),
                      "buckets_reduced_inside_each_backward_pass": in_backward,
                      "l2": "working set far above the 126 MB L2"},
           "optimizer_tail_ms": ms_tail,
           "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": host_ids.numel() * 8,
                   "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e},
           "loss": float(last["nll"])}
    out.update(push)
    return _finish(out, rank, world, sampler, args, launches)


def run(args, ClockSampler) -> int:
    if args.config == "cpu_loss":
        return cpu_loss(args)
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device", "config": args.config}))
        return 1
    return {"moe30b_ep8_sft": moe30b_ep8_sft, "cp8_attention": cp8_attention,
            "zero2_dp8_push": zero2_dp8_push}[args.config](args, ClockSampler)
