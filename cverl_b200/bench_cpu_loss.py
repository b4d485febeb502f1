"""CPU fp32 GRPO / PPO loss step through the public C ABI, this library against any ABI-compatible one.

``python -m cverl_b200.bench_cpu_loss [--other baseline/_ref/lib/libcverl_ref.so] [--iters 200]``

The step on ``[batch 64, seq 512]`` tensors (log_prob ~ N(-2, 0.5^2); old = log_prob + N(0, 0.05^2); ref =
log_prob + N(0, 0.1^2); response mask = first L tokens, L ~ U[32, 512]; Bernoulli(0.5) outcome rewards in groups
of 8; values ~ N(0, 1)):

1. ``cverl_grpo_outcome_advantage_f32_cpu`` (eps 1e-6, std normalisation),
2. ``cverl_gae_advantage_return_f32_cpu`` (gamma 1.0, lambda 0.95; whitened advantages),
3. ``cverl_masked_whiten_f32_cpu`` of the GRPO advantages,
4. ``cverl_ppo_clipped_loss_f32_cpu`` (clip 0.2, dual clip 3.0, token-mean) and its backward,
5. ``cverl_kl_penalty_f32_cpu`` (k3) and its backward.

Both libraries get the same buffers through the same ``ctypes`` prototypes (the ABI is shared: ten
``cverl_*_f32_cpu`` symbols, ``cverl_tensor2d_t`` views).  Prints one JSON line: microseconds per step for each,
their ratio, and the largest difference between the two libraries' outputs.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import sys
import time
from pathlib import Path

import numpy as np


class T2(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int), ("device", C.c_int), ("rows", C.c_int64),
                ("cols", C.c_int64)]


class PpoOut(C.Structure):
    _fields_ = [("pg_loss", C.c_float), ("pg_clipfrac", C.c_float), ("ppo_kl", C.c_float),
                ("pg_clipfrac_lower", C.c_float)]


def view(a: np.ndarray) -> T2:
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"] and a.ndim == 2
    return T2(a.ctypes.data, 0, 0, a.shape[0], a.shape[1])


def bind(path: str):
    lib = C.CDLL(path)
    f = C.c_float
    lib.cverl_grpo_outcome_advantage_f32_cpu.argtypes = [T2, T2, C.c_void_p, f, C.c_int, T2, T2]
    lib.cverl_gae_advantage_return_f32_cpu.argtypes = [T2, T2, T2, f, f, T2, T2]
    lib.cverl_masked_whiten_f32_cpu.argtypes = [T2, T2, C.c_int, T2]
    lib.cverl_ppo_clipped_loss_f32_cpu.argtypes = [T2, T2, T2, T2, f, f, f, f, C.c_int, C.POINTER(PpoOut)]
    lib.cverl_ppo_clipped_loss_backward_f32_cpu.argtypes = [T2, T2, T2, T2, f, f, f, f, C.c_int, T2]
    lib.cverl_kl_penalty_f32_cpu.argtypes = [T2, T2, C.c_int, T2]
    lib.cverl_kl_penalty_backward_f32_cpu.argtypes = [T2, T2, C.c_int, T2]
    return lib


def make_inputs(batch: int, seq: int, seed: int):
    rng = np.random.default_rng(seed)
    lp = rng.normal(-2.0, 0.5, (batch, seq)).astype(np.float32)
    old = (lp + rng.normal(0, 0.05, (batch, seq))).astype(np.float32)
    ref = (lp + rng.normal(0, 0.1, (batch, seq))).astype(np.float32)
    lengths = rng.integers(32, seq + 1, batch)
    mask = (np.arange(seq)[None, :] < lengths[:, None]).astype(np.float32)
    rewards = np.zeros((batch, seq), np.float32)
    rewards[np.arange(batch), lengths - 1] = rng.integers(0, 2, batch).astype(np.float32)
    values = rng.normal(0, 1, (batch, seq)).astype(np.float32)
    groups = (np.arange(batch) // 8).astype(np.int64)
    return dict(lp=lp, old=old, ref=ref, mask=mask, rewards=rewards, values=values, groups=groups)


def step(lib, d, out):
    ok = 0
    ok |= lib.cverl_grpo_outcome_advantage_f32_cpu(view(d["rewards"]), view(d["mask"]), d["groups"].ctypes.data, 1e-6, 1,
                                                   view(out["adv"]), view(out["ret"]))
    ok |= lib.cverl_gae_advantage_return_f32_cpu(view(d["rewards"]), view(d["values"]), view(d["mask"]), 1.0, 0.95,
                                                 view(out["gae_adv"]), view(out["gae_ret"]))
    ok |= lib.cverl_masked_whiten_f32_cpu(view(out["adv"]), view(d["mask"]), 1, view(out["white"]))
    res = PpoOut()
    ok |= lib.cverl_ppo_clipped_loss_f32_cpu(view(d["old"]), view(d["lp"]), view(out["white"]), view(d["mask"]), 0.2,
                                             -1.0, -1.0, 3.0, 0, C.byref(res))
    ok |= lib.cverl_ppo_clipped_loss_backward_f32_cpu(view(d["old"]), view(d["lp"]), view(out["white"]),
                                                      view(d["mask"]), 0.2, -1.0, -1.0, 3.0, 0, view(out["dlp"]))
    ok |= lib.cverl_kl_penalty_f32_cpu(view(d["lp"]), view(d["ref"]), 3, view(out["kl"]))
    ok |= lib.cverl_kl_penalty_backward_f32_cpu(view(d["lp"]), view(d["ref"]), 3, view(out["dkl"]))
    if ok != 0:
        raise RuntimeError("a C ABI call returned an error status")
    out["pg_loss"] = res.pg_loss
    return out


def timed(lib, d, iters: int):
    out = {k: np.zeros_like(d["lp"]) for k in ("adv", "ret", "gae_adv", "gae_ret", "white", "dlp", "kl", "dkl")}
    for _ in range(5):
        step(lib, d, out)
    t0 = time.perf_counter()
    for _ in range(iters):
        step(lib, d, out)
    return (time.perf_counter() - t0) / iters * 1e6, out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--other", default="", help="an ABI-compatible library to time on the same buffers")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    from . import _build
    if not _build.HOST_LIB.exists():
        _build.build_host()
    d = make_inputs(a.batch, a.seq, a.seed)
    us, out = timed(bind(str(_build.HOST_LIB)), d, a.iters)
    report = {"config": {"batch": a.batch, "seq": a.seq, "iters": a.iters, "dtype": "fp32", "device": "cpu"},
              "ours_us_per_step": us, "ours_pg_loss": out["pg_loss"]}
    if a.other:
        if not Path(a.other).exists():
            report["other"] = f"{a.other} not found"
        else:
            us2, out2 = timed(bind(a.other), d, a.iters)
            diffs = {k: float(np.abs(out[k] - out2[k]).max()) for k in out if k != "pg_loss"}
            report.update({"other": a.other, "other_us_per_step": us2, "other_pg_loss": out2["pg_loss"],
                           "speedup_vs_other": us2 / us, "max_abs_diff": max(diffs.values()),
                           "max_abs_diff_by_output": diffs})
    print(json.dumps(report))
    return 0


if __name__ == "__main__":
    sys.exit(main())
