"""Trainer CLI on one B200: a few bf16 steps of a Qwen3.5-shaped model through the native kernels (tcgen05 GEMMs,
attention, Gated DeltaNet, fused LM head) with checkpoint and resume; pass = finite metrics, gradients on every
rank, parameters moved, and a resumed run that continues from the saved step."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _run(*flags, timeout=400):
    cmd = [sys.executable, "-m", "cverl_b200.trainer.ppo_trainer", "--dtype", "bfloat16", "--config", "qwen3_5_0_8b",
           "--max-layers", "4", "--prompt-len", "128", "--response-len", "384", "--micro-batches", "2",
           "--micro-batch-seqs", "2", "--lr", "1e-5", *flags]
    env = dict(os.environ, PYTHONPATH=str(ROOT), MASTER_ADDR="127.0.0.1", MASTER_PORT="29577", RANK="0",
               WORLD_SIZE="1", LOCAL_RANK="0")
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-3000:]
    rows = [dict(kv.split("=", 1) for kv in ln.split()) for ln in p.stdout.splitlines() if ln.startswith("step=")]
    return rows


def test_trainer_cli_bf16_steps_checkpoint_resume(tmp_path):
    ck = tmp_path / "ck"
    rows = _run("--steps", "3", "--checkpoint-dir", str(ck), "--checkpoint-every", "2")
    assert [r["step"] for r in rows] == ["0", "1", "2"]
    for r in rows:
        assert r["all_ranks_have_grad"] == "true" and r["all_ranks_updated"] == "true"
        for key in ("loss_sum", "global_grad_norm", "step_time_s"):
            v = float(r[key])
            assert v == v and abs(v) < 1e9
    assert (ck / "latest_checkpoint.txt").read_text().strip() == "step_000002"
    resumed = _run("--steps", "4", "--resume-checkpoint", str(ck))
    assert [r["step"] for r in resumed] == ["2", "3"]
    assert float(resumed[0]["loss_sum"]) == pytest.approx(float(rows[2]["loss_sum"]), rel=2e-2, abs=1e-3)
