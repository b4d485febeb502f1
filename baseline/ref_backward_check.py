"""Backward parity with the reference itself: parameter gradients of its policy class against this package's model.

    python baseline/ref_backward_check.py [--keep DIR]

``baseline/ref_backward_check.cc`` builds the reference's ``Qwen3_5CausalLmPolicy`` (through its factory) on a model
directory written by this package, back-propagates a weighted negative log-likelihood of a fixed response and
writes every parameter's gradient with the reference's own safetensors writer; it is linked against the reference
library that ``baseline/build_ref.py`` built.  This package's model back-propagates the same loss on the same
directory (fp32, CPU) and every gradient is compared - the per-expert tensors of the mixture-of-experts model
against the slices of the packed expert weights; an expert no token was routed to has no gradient there and a zero
gradient here.  One JSON line per model (Qwen3.5 hybrid, Qwen3-MoE); exit code 0 when all agree, 3 when the
reference library is not built.
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
PROMPT = [5, 6, 7, 8, 9, 42]
RESPONSE = [100, 3, 17, 250, 11, 2, 77, 1]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--keep", default="")
    a = ap.parse_args(argv)
    import torch

    from cverl_b200.models.config import Qwen35TextConfig
    from cverl_b200.models.hf_io import HfModelLoader, load_model_weights, synthesize_model_dir
    from cverl_b200.models.qwen3_5 import Qwen35Model, _packed_moe_names
    import ref_common
    try:
        exe = ref_common.link_driver(HERE / "ref_backward_check.cc", "ref_backward_check")
    except ref_common.Unavailable as exc:
        print(json.dumps({"unavailable": str(exc)}))
        return 3
    with tempfile.TemporaryDirectory(prefix="cverl_ref_") as tmp:
        work = Path(a.keep) if a.keep else Path(tmp)
        work.mkdir(parents=True, exist_ok=True)
        ok = True
        for moe in (False, True):
            d = synthesize_model_dir(Qwen35TextConfig.tiny(moe=moe), work / f"model_{int(moe)}", seed=11, dtype=torch.float32)
            grads_file = work / f"grads_{int(moe)}.safetensors"
            r = subprocess.run([str(exe), str(d), ",".join(map(str, PROMPT)), ",".join(map(str, RESPONSE)), str(grads_file)],
                               capture_output=True, text=True)
            row = {"model": "qwen3_moe" if moe else "qwen3_5"}
            if r.returncode != 0:
                row.update(agree=False, error=r.stderr[-300:])
                print(json.dumps(row))
                ok = False
                continue
            ref_loss = float(r.stdout.split("loss=")[1].split()[0])
            loader = HfModelLoader(d).load_metadata()
            cfg = loader.config()
            model = Qwen35Model(cfg, dtype=torch.float32)
            load_model_weights(model, loader)
            lp = model.response_logprobs(torch.tensor([PROMPT + RESPONSE]), len(PROMPT))
            w = (torch.arange(len(RESPONSE)).float() * 0.1 + 0.5).view(1, -1)
            loss = -(lp * w).sum()
            loss.backward()
            for prm in list(model.flat.params.values()) + list(model.fused.values()):
                if prm.grad is not None:
                    prm.main_grad.add_(prm.grad.float())
                    prm.grad = None

            def grad_of(name):
                spec = model.spec_by_name[name]
                if spec.expert < 0:
                    return model.flat.params[name].main_grad
                layer = int(name[len(cfg.layer_root):].split(".")[0])
                gu, dn = _packed_moe_names(layer)
                inter = cfg.moe_intermediate_size
                if name.endswith("gate_proj.weight"):
                    return model.flat.params[gu].main_grad[spec.expert, :inter]
                if name.endswith("up_proj.weight"):
                    return model.flat.params[gu].main_grad[spec.expert, inter:]
                return model.flat.params[dn].main_grad[spec.expert]
            ref = HfModelLoader(grads_file).load_metadata()
            worst, bad = 0.0, []
            for name in ref.names():
                g_ref = ref.load_tensor(name)
                diff = float((grad_of(name).reshape(g_ref.shape) - g_ref).abs().max())
                scale = float(g_ref.abs().max())
                worst = max(worst, diff / max(scale, 1e-3))
                if diff > 2e-6 + 1e-4 * scale:
                    bad.append(name)
            absent_nonzero = [s.name for s in model.specs
                              if s.name not in ref.names() and float(grad_of(s.name).abs().max()) != 0.0]
            same = (not bad and not absent_nonzero and abs(float(loss) - ref_loss) <= 1e-5 * abs(ref_loss))
            ok = ok and same
            row.update(loss=float(loss), reference_loss=ref_loss, gradients_compared=len(ref.names()),
                       worst_relative_difference=worst, differing=bad[:5], nonzero_where_reference_has_none=absent_nonzero[:5],
                       agree=same)
            print(json.dumps(row))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
