"""Model directories written by this package, read by the reference's own loader.

    python baseline/ref_loader_check.py [--keep DIR]

Writes a small random Qwen3.5 and a small Qwen3-MoE model directory (config.json + model.safetensors) with
``cverl_b200.models.hf_io.synthesize_model_dir``, links ``baseline/ref_loader_check.cc`` against the reference's
compiled ``hf_model_loader`` object (``python baseline/build_ref.py`` must have run) and LibTorch, and compares what
the reference's ``HfModelLoader`` reads - model type, layer count, tensor count, element count, sum of absolute
values - with what this package's reader gives.  Prints one JSON line per model; exit code 0 when all agree,
3 when the reference objects are not built.
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
    ap.add_argument("--keep", default="", help="work directory to keep (default: a temporary one)")
    a = ap.parse_args(argv)
    import torch
    from cverl_b200.models.config import Qwen35TextConfig
    from cverl_b200.models.hf_io import HfModelLoader, synthesize_model_dir
    import ref_common
    obj = HERE / "_ref" / "obj" / "src__model__hf_model_loader.cc.o"
    try:
        exe = ref_common.link_driver(HERE / "ref_loader_check.cc", "ref_loader_check", link_library=False,
                                     extra_objects=[obj])
    except ref_common.Unavailable as exc:
        print(json.dumps({"unavailable": str(exc)}))
        return 3
    with tempfile.TemporaryDirectory(prefix="cverl_ref_") as tmp:
        work = Path(a.keep) if a.keep else Path(tmp)
        work.mkdir(parents=True, exist_ok=True)
        ok = True
        for moe in (False, True):
            d = synthesize_model_dir(Qwen35TextConfig.tiny(moe=moe), work / f"model_{int(moe)}", dtype=torch.bfloat16)
            r = subprocess.run([str(exe), str(d)], capture_output=True, text=True)
            ours = HfModelLoader(d).load_metadata()
            names = ours.names()
            mine = {"tensors": len(names), "numel": sum(ours.info(n).nbytes // 2 for n in names),
                    "abs_sum": sum(float(ours.load_tensor(n).double().abs().sum()) for n in names)}
            theirs = {}
            for tok in r.stdout.split():
                k, _, v = tok.partition("=")
                theirs[k] = v
            same = (r.returncode == 0 and int(theirs.get("tensors", -1)) == mine["tensors"]
                    and int(theirs.get("numel", -1)) == mine["numel"]
                    and abs(float(theirs.get("abs_sum", "nan")) - mine["abs_sum"]) <= 1e-9 * mine["abs_sum"]
                    and theirs.get("model_type") == ("qwen3_moe" if moe else "qwen3_5"))
            ok = ok and same
            print(json.dumps({"model": "qwen3_moe" if moe else "qwen3_5", "reference": theirs, "ours": mine, "agree": same,
                              "stderr": r.stderr[-200:]}))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
