"""``bench.py --config``: the CPU configuration end to end, and the GPU configurations on reduced depth (the
line is then marked invalid; the point is that every configuration's code path runs)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def _bench(*flags, nproc=1, port=29820, timeout=600):
    if nproc == 1:
        cmd = [sys.executable, "bench.py", *flags]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), "bench.py", "--gpus", str(nproc), *flags]
    p = subprocess.run(cmd, cwd=ROOT, env=dict(os.environ, PYTHONPATH=str(ROOT)), capture_output=True, text=True,
                       timeout=timeout)
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-3000:]
    lines = [ln for ln in p.stdout.splitlines() if ln.startswith("{")]
    assert lines, p.stdout[-1500:]
    return json.loads(lines[-1])


def test_cpu_loss_config():
    out = _bench("--config", "cpu_loss", "--steps", "20")
    assert out["value"] > 0 and out["unit"] == "us/step" and out["higher_is_better"] is False
    assert out["detail"]["config"] == {"batch": 64, "seq": 512, "iters": 50, "dtype": "fp32", "device": "cpu"}


@pytest.mark.gpu
@pytest.mark.parametrize("config,flags", [
    ("moe30b_ep8_sft", ["--layers", "2", "--seq-len", "512", "--seqs-per-gpu", "2"]),
    ("zero2_dp8_push", ["--layers", "2", "--seq-len", "512", "--seqs-per-gpu", "2"]),
    ("cp8_attention", ["--seq-len", "4096"]),
])
def test_gpu_configs_reduced(config, flags):
    n = 2 if torch.cuda.device_count() >= 2 else 1
    out = _bench("--config", config, "--steps", "2", "--warmup", "1", *flags, nproc=n)
    assert out["value"] > 0 and out["n_gpus"] == n and out["gpu_launches"] > 0 and out["library_fallbacks"] == 0
    assert out["config"]["name"] == config
    if config == "zero2_dp8_push":
        assert out["config"]["buckets_reduced_inside_each_backward_pass"] == 2
        if n == 2:
            assert out["push_verified"] is True
    if config != "cp8_attention":
        assert out["invalid"] and 0 < out["loss"] < 20


def test_reference_arm_gets_the_headline_batch_by_default(monkeypatch):
    """`bench.py --impl reference` hands the reference arm the headline configuration (128 sequences per GPU) when
    no size is given, and the caller's value when one is."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    seen = []
    monkeypatch.setattr(bench, "reference_arm", lambda args: seen.append(args.seqs_per_gpu) or 0)
    monkeypatch.setattr(sys, "argv", ["bench.py", "--impl", "reference", "--gpus", "1"])
    assert bench.main() == 0
    monkeypatch.setattr(sys, "argv", ["bench.py", "--impl", "reference", "--seqs-per-gpu", "4"])
    assert bench.main() == 0
    assert seen == [bench.SEQS_PER_GPU, 4] and bench.SEQS_PER_GPU == 128
