"""Optimizer parity with the reference itself: five AdamW steps of its two optimizer classes against this package's.

    python baseline/ref_optimizer_check.py [--keep DIR]

``baseline/ref_optimizer_check.cc`` runs the reference's ``FlatAdamW`` and ``Fp32MasterAdamW`` (from the reference
library built by ``baseline/build_ref.py``) for five steps on data both sides can state exactly (parameter
``sin(0.37 i)``, gradient of step k ``cos(0.11 i + k) / 3``), with and without fp32 master weights, and writes the
final parameters and moments.  The same five steps run through ``cverl_b200.optim`` (CPU statements of the fused
kernel) and every tensor is compared.  One JSON line; exit code 0 when all agree within 2e-6, 3 when the reference
library is not built.
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--keep", default="")
    a = ap.parse_args(argv)
    import torch

    from cverl_b200.models.hf_io import HfModelLoader
    from cverl_b200.optim import AdamWOptions
    from cverl_b200.optim.adamw import FlatAdamW, Fp32MasterAdamW
    import ref_common
    try:
        exe = ref_common.link_driver(HERE / "ref_optimizer_check.cc", "ref_optimizer_check")
    except ref_common.Unavailable as exc:
        print(json.dumps({"unavailable": str(exc)}))
        return 3
    with tempfile.TemporaryDirectory(prefix="cverl_ref_") as tmp:
        work = Path(a.keep) if a.keep else Path(tmp)
        work.mkdir(parents=True, exist_ok=True)
        r = subprocess.run([str(exe), str(work / "reference.safetensors")], capture_output=True, text=True)
        if r.returncode != 0:
            print(json.dumps({"agree": False, "error": r.stderr[-300:]}))
            return 1
        ref = HfModelLoader(work / "reference.safetensors").load_metadata()
        n = 1000
        idx = torch.arange(n, dtype=torch.float32)
        diffs = {}
        for master in (False, True):
            tag = "master" if master else "bf16"
            o = AdamWOptions(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01, use_master_weights=master)
            p0 = torch.sin(idx * 0.37)
            flat = FlatAdamW(p0.clone() if master else p0.bfloat16(), o)
            ta = p0[:600].clone().bfloat16().requires_grad_(True)
            tb = p0[600:].clone().bfloat16().view(20, 20).requires_grad_(True)
            per = Fp32MasterAdamW([ta, tb], o)
            for k in range(5):
                g = torch.cos(idx * 0.11 + k) / 3.0
                flat.step(g)
                ta.grad, tb.grad = g[:600].bfloat16(), g[600:].view(20, 20).bfloat16()
                per.accumulate_model_grads()
                per.step()
                per.zero_grad()
            mine = {f"flat.{tag}.param": flat.parameter_shard.float(), f"flat.{tag}.exp_avg": flat.exp_avg,
                    f"flat.{tag}.exp_avg_sq": flat.exp_avg_sq, f"tensorwise.{tag}.a": ta.detach().float(),
                    f"tensorwise.{tag}.b": tb.detach().float(), f"tensorwise.{tag}.exp_avg_sq_b": per.exp_avg_sq[1]}
            for name, t in mine.items():
                diffs[name] = float((t - ref.load_tensor(name).reshape(t.shape)).abs().max())
        ok = len(diffs) == 12 and max(diffs.values()) <= 2e-6
        print(json.dumps({"tensors_compared": len(diffs), "largest_difference": max(diffs.values()),
                          "bit_identical": sum(1 for v in diffs.values() if v == 0.0), "agree": ok}))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
