#!/usr/bin/env python
"""Headline benchmark: Qwen3.5-0.8B-shaped GRPO actor update, tokens/s.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

One step = the full actor update of the reference trainer: forward to response
log-probs, clipped PPO loss, backward, gradient reduce-scatter, global-norm
clip, FlatAdamW, parameter all-gather.  Weak scaling: 128 sequences of
256 + 1024 tokens per GPU (1024 sequences per step on 8 GPUs, the configuration
BASELINE.json names).  Synthetic uniform token ids, random-init bf16 weights.

Two measurements, both device-timed with CUDA events between barrier +
synchronize pairs, max over ranks:
  value : inputs resident on the device, no host read inside the timed region;
  e2e   : ActorEngine.update_from_host - every step copies its inputs from
          pinned host memory and reads the step metrics back to the host.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

SEQS_PER_GPU = 128
PROMPT_LEN, RESPONSE_LEN = 256, 1024


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--micro-batch", type=int, default=int(os.environ.get("CVERL_BENCH_MICRO_BATCH", "0")),
                    help="sequences per micro-batch; 0 = 32 per tensor-parallel rank (about 100 GB of the 180 GB HBM)")
    ap.add_argument("--tp", type=int, default=int(os.environ.get("CVERL_BENCH_TP", "0")))
    ap.add_argument("--seqs-per-gpu", type=int, default=0, help="0 = the configuration's own (128 for the headline)")
    ap.add_argument("--config", default="grpo_0_8b",
                    choices=["grpo_0_8b", "cpu_loss", "moe30b_ep8_sft", "cp8_attention", "zero2_dp8_push"],
                    help="grpo_0_8b is the headline benchmark; the others are described in cverl_b200/bench_configs.py")
    ap.add_argument("--seq-len", type=int, default=0, help="other configurations: 0 = the named sequence length")
    ap.add_argument("--ep-comm", default="symm", choices=["symm", "nccl"])
    ap.add_argument("--cp-comm", default="nccl", choices=["symm", "nccl"])
    ap.add_argument("--ep-capacity-factor", type=float, default=3.0,
                    help="moe30b_ep8_sft: receive-buffer rows per rank as a multiple of the balanced load")
    ap.add_argument("--grad-slots", type=int, default=2, help="zero2_dp8_push: gradient bucket buffers in flight")
    ap.add_argument("--rs-blocks", type=int, default=0,
                    help="zero2_dp8_push: CTAs of a bucket's reduce-scatter kernel while it overlaps the backward pass")
    ap.add_argument("--grad-comm-dtype", default="float32", choices=["float32", "bfloat16"],
                    help="zero2_dp8_push with --zero-comm nccl: dtype in which the gradient buckets are reduced")
    ap.add_argument("--push-pattern", default="pairs", choices=["pairs", "slices"],
                    help="zero2_dp8_push: trainer t -> rollout t (whole buffer), or slice t -> every rollout rank")
    ap.add_argument("--no-overlap", action="store_true", help="zero2_dp8_push: reduce buckets on the main stream")
    ap.add_argument("--tp-comm", default=os.environ.get("CVERL_BENCH_TP_COMM", "sp"), choices=["sp", "symm", "nccl"],
                    help="tensor-parallel communication: sp = token-sharded residual stream, reduce-scatter in the "
                         "GEMM epilogue and all-gather in the norm kernels over peer-mapped memory; symm = all-reduce "
                         "by mirror stores from the GEMM epilogue; nccl = library collectives")
    ap.add_argument("--zero-comm", default=os.environ.get("CVERL_BENCH_ZERO", "symm"), choices=["symm", "nccl"],
                    help="ZeRO communication: symm = own kernels over peer-mapped memory, nccl = library collectives")
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (result marked invalid)")
    ap.add_argument("--no-check", action="store_true",
                    help="skip the untimed comparison of the fused communication kernels with the NCCL path")
    return ap.parse_args()


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.2):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:  # NVML missing: report no clocks rather than fail the run
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop.set()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def reference_arm(args):
    """Runs the unmodified reference trainer (built out of tree by ``baseline/build_ref.py``) on this
    benchmark's configuration; nothing of this framework is imported on that path."""
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
    import ref_arm
    return ref_arm.run(args)


def consistency_check(model, ctx, opt, fused_comm, dev_batch, micro_batch, world, dev):
    """One forward / backward of the first micro-batch through this package's fused communication kernels and
    once more through NCCL, on the same weights and tokens: returns the differences in the loss-side quantity
    (mean response log-prob) and in the global gradient norm, and (with data parallelism) of the fused ZeRO
    reduce-scatter against ``reduce_scatter_tensor``.  Runs before warm-up; leaves the gradients zeroed."""
    import torch.distributed as dist
    ids = dev_batch["input_ids"][:micro_batch]
    g = torch.Generator(device=dev).manual_seed(99)
    seed = torch.randn(ids.shape[0], RESPONSE_LEN, device=dev, generator=g) / ids.shape[0]

    def one_pass():
        model.flat.main_grad.zero_()
        lp = model.response_logprobs(ids, PROMPT_LEN)
        lp.backward(seed)
        model.sync_replicated_grads()
        sq = model.flat.main_grad.double().pow(2).sum()
        dist.all_reduce(sq)
        return float(lp.detach().double().mean()), float(sq.sqrt())

    fused = one_pass()
    saved = (ctx.tp_sp, ctx.tp_symm)
    ctx.tp_sp = ctx.tp_symm = None
    try:
        plain = one_pass()
    finally:
        ctx.tp_sp, ctx.tp_symm = saved
    out = {"loss_abs_diff": abs(fused[0] - plain[0]),
           "grad_norm_rel_diff": abs(fused[1] - plain[1]) / max(plain[1], 1e-30)}
    if fused_comm is not None:
        # the gradients of the NCCL pass are still in the buffer: reduce-scatter them both ways
        want = torch.empty(opt.shard_numel, dtype=torch.float32, device=dev)
        dist.reduce_scatter_tensor(want, model.flat.main_grad.clone(), op=dist.ReduceOp.AVG, group=ctx.dp_group)
        got = torch.empty_like(want)
        sq = fused_comm.reduce_scatter_mean_sumsq(got, opt.begin).clone()      # zeroes the gradient buffer
        out["zero_rs_rel_diff"] = float((got - want).norm() / want.norm().clamp_min(1e-30))
        out["zero_sumsq_rel_diff"] = float((sq[0] - want.pow(2).sum()).abs() / want.pow(2).sum().clamp_min(1e-30))
    model.flat.main_grad.zero_()
    worst = torch.tensor([out["loss_abs_diff"], out["grad_norm_rel_diff"], out.get("zero_rs_rel_diff", 0.0)],
                         device=dev)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    out["loss_abs_diff"], out["grad_norm_rel_diff"] = float(worst[0]), float(worst[1])
    # bf16 activations summed in another order: a few 1e-3 is rounding, more is a wrong kernel
    out["ok"] = bool(worst[0] < 2e-2 and worst[1] < 5e-2 and worst[2] < 1e-4)
    return out


def main():
    args = parse_args()
    if args.config != "grpo_0_8b" and args.impl != "reference":
        from cverl_b200 import bench_configs
        return bench_configs.run(args, ClockSampler)
    if args.seqs_per_gpu <= 0:
        args.seqs_per_gpu = SEQS_PER_GPU
    if args.impl == "reference":
        return reference_arm(args)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from cverl_b200 import ops
    from cverl_b200.models.config import Qwen35TextConfig
    from cverl_b200.models.qwen3_5 import Qwen35Model
    from cverl_b200.optim import AdamWOptions
    from cverl_b200.parallel.mesh import build_context
    from cverl_b200.parallel.zero import FlatZeroOptimizer
    from cverl_b200.trainer.actor import ActorConfig, ActorEngine, synthetic_rl_batch
    from cverl_b200 import _native as nv

    tp = args.tp if args.tp > 0 else (2 if world >= 2 else 1)
    dp = world // tp
    if args.micro_batch <= 0:
        args.micro_batch = 32 * tp
    ctx = build_context(world, rank, tp=tp, dp=dp)
    cfg = Qwen35TextConfig.qwen3_5_0_8b()
    if args.layers:
        cfg = Qwen35TextConfig(num_hidden_layers=args.layers)
    if tp > 2 and args.tp_comm == "symm":
        # measured (cverl_b200.bench_collectives): the mirror-store all-reduce beats NCCL at TP=2 (0.25 vs 0.32 ms
        # on the out_proj shape) and loses from TP=4 on, where every rank would store its full partial N-1 times
        args.tp_comm = "nccl"
    if tp > 1 and args.tp_comm == "sp":
        from cverl_b200.parallel.tp_sp import TpSp
        ctx.tp_sp = TpSp(ctx.tp_group, dev, args.micro_batch * (PROMPT_LEN + RESPONSE_LEN), cfg.hidden_size,
                         arena_slots=2 * cfg.num_hidden_layers + 1)
    if tp > 1 and args.tp_comm == "symm":
        from cverl_b200.parallel.tp_symm import TpSymm
        ctx.tp_symm = TpSymm(ctx.tp_group, dev, args.micro_batch * (PROMPT_LEN + RESPONSE_LEN), cfg.hidden_size)
    fused_comm = None
    if dp > 1 and args.zero_comm == "symm":
        from cverl_b200.parallel.symm import FusedZeroComm, SymmetricHeap
        fused_comm = FusedZeroComm(SymmetricHeap(ctx.dp_group, dev))
    model = Qwen35Model(cfg, dtype=torch.bfloat16, device=dev, ctx=ctx, pad_multiple=dp * 8,
                        flat_allocator=fused_comm.allocator if fused_comm else None)
    model.init_weights(seed=1234)
    opt = FlatZeroOptimizer(model.flat, AdamWOptions(lr=1e-6, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01,
                                                     use_master_weights=False),
                            dp_group=ctx.dp_group, dp_rank=ctx.dp_rank, dp_size=dp,
                            norm_group=None, norm_world=world, max_grad_norm=1.0, fused_comm=fused_comm)
    engine = ActorEngine(model, opt, ActorConfig(mode="ppo", micro_batch_size=args.micro_batch))

    # each DP rank sees its own sequences; TP peers of one DP rank see the same ones
    seqs_local = args.seqs_per_gpu * tp
    host_batch = engine.pin_batch(synthetic_rl_batch(seqs_local, PROMPT_LEN, RESPONSE_LEN, cfg.vocab_size,
                                                     seed=1000 + ctx.dp_rank))
    dev_batch = {k: v.to(dev) for k, v in host_batch.items()}
    tokens_per_step = args.seqs_per_gpu * world * (PROMPT_LEN + RESPONSE_LEN)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    barrier()        # model construction takes different times per rank; the kernels' flag barriers are bounded waits
    check = None
    if world > 1 and not args.no_check:
        check = consistency_check(model, ctx, opt, fused_comm, dev_batch, args.micro_batch, world, dev)
        nv.check_status(dev)
        if not check["ok"]:
            if rank == 0:
                print(json.dumps({"error": "fused communication kernels disagree with the NCCL path", "check": check}))
            return 1
    for _ in range(max(args.warmup, 0)):
        engine.update(dev_batch, PROMPT_LEN)
    nv.check_status(dev)

    sampler = ClockSampler(local_rank)
    sampler.start()
    l0 = ops.launch_counter["n"]
    ms_dev = timed(lambda: engine.update(dev_batch, PROMPT_LEN), args.steps)
    launches = ops.launch_counter["n"] - l0
    last = {}

    def e2e_step():
        last["m"] = engine.update_from_host(host_batch, PROMPT_LEN)

    e2e_step()  # one untimed pass of the host path
    ms_e2e = timed(e2e_step, args.steps)
    sampler.stop()
    nv.check_status(dev)

    if rank == 0:
        ms_per_step = ms_dev / args.steps
        value = tokens_per_step / (ms_per_step / 1e3)
        e2e_value = tokens_per_step / (ms_e2e / args.steps / 1e3)
        h2d = ActorEngine.host_batch_bytes(host_batch)
        d2h = int(last["m"].numel() * last["m"].element_size())
        out = {
            "metric": "actor-update tokens/s (device, max over ranks)",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights",
            "config": {"model": "Qwen3.5-0.8B-shaped hybrid (18 Gated-DeltaNet + 6 full-attention layers, tied head)",
                       "global_batch": args.seqs_per_gpu * world, "seq_len": PROMPT_LEN + RESPONSE_LEN,
                       "prompt_len": PROMPT_LEN, "response_len": RESPONSE_LEN,
                       "parallelism": f"dp{dp}xtp{tp}", "micro_batch_seqs": args.micro_batch,
                       "optimizer": "FlatAdamW ZeRO-1 reduce-scatter, clip 1.0",
                       "zero_comm": args.zero_comm if dp > 1 else "none",
                       "tp_comm": args.tp_comm if tp > 1 else "none",
                       "l2": "per-step working set (activations + 1.5 GB weights + 3 GB fp32 grads) exceeds the "
                             "126 MB L2, no explicit flush"},
            "clocks": sampler.summary(),
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": launches,
            "loss": float(last["m"][0]),
            "peak_mem_gb": round(torch.cuda.max_memory_allocated(dev) / 2 ** 30, 1),
        }
        if check is not None:
            out["check"] = check
        from cverl_b200.utils import fallbacks
        out["library_fallbacks"] = fallbacks.total()     # hot ops that left their native kernel (0 expected)
        if args.layers:
            out["invalid"] = "debug run with fewer layers"
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
