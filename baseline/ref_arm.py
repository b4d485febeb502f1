"""Reference arm of ``bench.py``: the unmodified reference trainer on the benchmark's configuration.

``run(args)`` is called once per rank (``bench.py --impl reference`` runs alone for one GPU and
under ``torch.distributed.run`` for several).  Every rank starts ONE process of the reference's
own executable ``qwen3_5_pp_tp_ppo_trainer`` (built from the untouched sources by
``baseline/build_ref.py``) with the flags its launcher passes
(tools/distributed/run_qwen_pp_tp_ppo_trainer.sh:66-121): bf16, tensor-parallel 2 from two GPUs
on, data-parallel over the rest, prompt 256 + response 1024 tokens, 128 sequences per GPU and
step as micro-batches of one sequence (the reference's only batching), the flat sharded
optimizer.  The reference rendezvouses through NCCL-id files, not through torchrun's store.

The number reported is the reference's own ``step_time_s`` (host clock between two device
synchronisations, maximum over ranks, tools/model/qwen3_5_pp_tp_ppo_trainer.cc:2200-2202,
2538-2540,2654), averaged over the timed steps.  Nothing of ``cverl_b200`` is imported here.
"""
from __future__ import annotations

import json
import os
import re
import subprocess
import sys
import threading
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
TRAINER = HERE / "_ref" / "bin" / "qwen3_5_pp_tp_ppo_trainer"

SEQS_PER_GPU = 128
PROMPT_LEN, RESPONSE_LEN = 256, 1024
# Measured on this pool's B200s (2 timed steps of 4 micro-batches each, step_time_s 28.50 s at one GPU and
# 28.48 s at two GPUs with tensor-parallel 2): one micro-batch of the reference = one 1280-token sequence costs
# about 7.1 s whatever the tensor-parallel width (per-token sequential scan kernels, one launch per chunk in the
# backward), so one full-size step of 128 sequences per GPU takes about 15 minutes at one GPU and 30 minutes
# from two GPUs on (256 sequences per tensor-parallel pair).  The arm therefore times as many steps as fit its
# time limit (at least one, without warm-up) and reports itself unavailable, with these figures, when not even
# one step fits.  The limit is CVERL_BENCH_REF_BUDGET_S seconds; unset, it is 1700 s on a box with one visible
# GPU (a single-GPU benchmark run) and 820 s on a multi-GPU box, where the same command is repeated at several
# GPU counts.
S_PER_MICROBATCH = {1: 7.13, 2: 7.12}
STARTUP_S = 30.0


def time_limit_s() -> float:
    env = os.environ.get("CVERL_BENCH_REF_BUDGET_S")
    if env:
        return float(env)
    try:
        import torch
        visible = torch.cuda.device_count()
    except Exception:
        visible = 1
    return 1700.0 if visible <= 1 else 820.0


def unavailable(why: str) -> int:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class SmiSampler(threading.Thread):
    """SM clock and throttle reasons from ``nvidia-smi`` while the reference steps."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, period_s: float = 1.0):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._halt = threading.Event()

    def run(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._halt.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=10)
                f = [x.strip() for x in out.stdout.strip().split(",")]
                self.samples.append(int(f[0]))
                self.max_mhz = int(f[1])
                for name, val in zip(names, f[2:]):
                    if val.lower().startswith("active"):
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(self.period)

    def stop(self):
        self._halt.set()

    def summary(self):
        busy = sorted(s for s in self.samples)
        return {"sm_mhz": busy[len(busy) // 2] if busy else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons)}


def ensure_model_dir(local_rank: int, layers: int | None) -> Path:
    """Random-init Qwen3.5-0.8B-shaped model directory, written once per box by local rank 0."""
    tag = "full" if layers is None else f"l{layers}"
    out = Path(os.environ.get("CVERL_BENCH_REF_MODEL_DIR", f"/tmp/cverl_ref_model_qwen3_5_0_8b_{tag}"))
    done = out / ".complete"
    if local_rank == 0 and not done.exists():
        sys.path.insert(0, str(HERE))
        import synth_model
        synth_model.write_model_dir(synth_model.QWEN3_5_0_8B, out, layers)
        done.write_text("ok")
    deadline = time.time() + 600
    while not done.exists():
        if time.time() > deadline:
            raise RuntimeError("model directory was not written in time")
        time.sleep(0.5)
    return out


def trainer_command(model_dir: Path, rank: int, local_rank: int, world: int, tp: int, micro_batches: int, steps: int,
                    layers: int, id_prefix: str):
    dp = world // tp
    return [str(TRAINER), str(model_dir),
            "--global-rank", str(rank), "--device", str(local_rank),
            "--dp-size", str(dp), "--pp-size", "1", "--cp-size", "1", "--tp-size", str(tp), "--ep-size", "1",
            "--sp-size", "1", "--layers", str(layers), "--prompt-len", str(PROMPT_LEN),
            "--response-len", str(RESPONSE_LEN), "--micro-batches", str(micro_batches), "--grad-accum-steps", "1",
            "--steps", str(steps), "--train-mode", "ppo", "--lr", "1e-6", "--clip-ratio", "0.2",
            "--max-grad-norm", "1.0", "--dp-grad-bucket-mb", "25", "--dp-grad-comm-dtype", "model",
            "--master-weights", "false", "--dp-shard-optimizer", "true", "--dp-flat-shard-optimizer", "true",
            "--vary-tokens-by-step", "true", "--dtype", "bfloat16", "--id-prefix", id_prefix]


def run(args) -> int:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not TRAINER.exists():
        return unavailable("reference trainer binary is not built (run python baseline/build_ref.py)")
    tp = 2 if world >= 2 else 1
    seqs = getattr(args, "seqs_per_gpu", SEQS_PER_GPU)
    micro_batches = seqs * tp                  # sequences per data-parallel replica and step
    layers = args.layers if getattr(args, "layers", 0) else 24
    model_dir = ensure_model_dir(local_rank, None if layers == 24 else layers)

    # The measured cost of one reference micro-batch fixes how many steps fit the time budget.
    per_mb_s = float(os.environ.get("CVERL_BENCH_REF_S_PER_MICROBATCH", "0") or 0) or S_PER_MICROBATCH[tp]
    per_mb_s *= layers / 24.0
    warmup, steps = max(args.warmup, 0), max(args.steps, 1)
    shortened = None
    est_step = per_mb_s * micro_batches
    limit_s = time_limit_s()
    if STARTUP_S + est_step * (warmup + steps) > limit_s:
        fit = int((limit_s - STARTUP_S) // est_step)
        if fit < 1:
            return unavailable(
                f"one full-size step of the unmodified reference trainer takes about {est_step:.0f} s at "
                f"{world} GPU(s) ({micro_batches} one-sequence micro-batches x {per_mb_s:.2f} s, measured on this "
                f"pool: step_time_s 28.5 s for 4 micro-batches at tp{tp}), i.e. about "
                f"{seqs * world * (PROMPT_LEN + RESPONSE_LEN) / est_step:.0f} tokens/s; that does not fit this "
                f"arm's {limit_s:.0f} s time limit (set CVERL_BENCH_REF_BUDGET_S to run it)")
        new_warmup = 1 if fit >= 3 else 0
        new_steps = max(1, min(steps, fit - new_warmup))
        shortened = {"requested_steps": steps, "requested_warmup": warmup,
                     "reason": f"one reference step takes about {est_step:.0f} s; its per-step time does not depend "
                               f"on warm-up (first step 29.3 s, second 28.5 s at 4 micro-batches)"}
        warmup, steps = new_warmup, new_steps

    # every rank must derive the same prefix for the NCCL-id files: the rendezvous port and run id are shared
    port = os.environ.get("MASTER_PORT", "0")
    run_id = os.environ.get("TORCHELASTIC_RUN_ID", "single") if world > 1 else str(os.getpid())
    id_prefix = f"/tmp/cverl_ref_arm_{port}_{run_id}"
    if rank == 0:
        for stale in Path("/tmp").glob(Path(id_prefix).name + "_*.bin"):
            stale.unlink()
    cmd = trainer_command(model_dir, rank, local_rank, world, tp, micro_batches, warmup + steps, layers, id_prefix)
    env = dict(os.environ)
    sampler = SmiSampler(local_rank)
    sampler.start()
    t0 = time.time()
    proc = subprocess.run(cmd, capture_output=True, text=True, env=env)
    wall = time.time() - t0
    sampler.stop()
    log_dir = Path(os.environ.get("CVERL_BENCH_REF_LOG_DIR", "/tmp"))
    (log_dir / f"cverl_ref_arm_rank{rank}.log").write_text(proc.stdout + "\n--- stderr ---\n" + proc.stderr)
    if rank != 0:
        return 0 if proc.returncode == 0 else 1
    times = [float(m) for m in re.findall(r"step_time_s=([0-9.eE+-]+)", proc.stdout)]
    if proc.returncode not in (0,) or len(times) < warmup + steps:
        tail = (proc.stderr.strip() or proc.stdout.strip())[-300:].replace("\n", " | ")
        return unavailable(f"reference trainer exited {proc.returncode} after {len(times)} steps: {tail}")
    timed = times[warmup:warmup + steps]
    s_per_step = sum(timed) / len(timed)
    tokens = seqs * world * (PROMPT_LEN + RESPONSE_LEN)
    value = tokens / s_per_step
    m = re.findall(r" loss_sum=([0-9.eE+-]+|-?nan|-?inf)", proc.stdout)
    out = {
        "impl": "reference",
        "metric": "actor-update tokens/s (device, max over ranks)",
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": s_per_step * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "reference's stock synthetic token ids, random-init weights",
        "config": {"model": "Qwen3.5-0.8B-shaped hybrid (18 Gated-DeltaNet + 6 full-attention layers, tied head)",
                   "global_batch": seqs * world, "seq_len": PROMPT_LEN + RESPONSE_LEN, "prompt_len": PROMPT_LEN,
                   "response_len": RESPONSE_LEN, "parallelism": f"dp{world // tp}xtp{tp}", "micro_batch_seqs": 1,
                   "optimizer": "reference FlatAdamW, flat sharded optimizer, clip 1.0",
                   "timing": "reference's own step_time_s: host clock between device synchronisations, max over "
                             "ranks", "l2": "per-step working set exceeds the 126 MB L2, no explicit flush"},
        "clocks": sampler.summary(),
        # the stock path builds its token ids on the device and reads its metrics back every step, so the step
        # time already is the reference's end-to-end time; there is no separate host-fed entry point to time
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 36 * world, "ms_per_step": s_per_step * 1e3,
                "note": "same run: the reference creates its synthetic ids on the device"},
        "gpu_launches": None,
        "loss": m[-1] if m else None,
        "wall_s": round(wall, 1),
        "step_times_s": [round(t, 3) for t in times],
    }
    if shortened:
        out["shortened"] = shortened
    if layers != 24:
        out["invalid"] = "debug run with fewer layers"
    if seqs != SEQS_PER_GPU:
        out["invalid"] = "debug run with fewer sequences per GPU"
    print(json.dumps(out))
    return 0
