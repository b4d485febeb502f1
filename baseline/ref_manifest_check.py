"""The vLLM weight manifest against the reference's own tool.

    python baseline/ref_manifest_check.py [--keep DIR]

Compiles the reference's ``tools/rollout/vllm_weight_manifest.cc`` as it is, links it against the reference library
built by ``baseline/build_ref.py``, and runs it on model directories written by this package (Qwen3.5 hybrid,
Qwen3-MoE) with packed and unpacked settings; ``python -m cverl_b200.cli.vllm_weight_manifest`` must print the same JSON
document (parameter names in the same order, dtype names, shapes, packing fields).  One JSON line per case; exit
code 0 when all agree, 3 when the reference library is not built.
"""
from __future__ import annotations

import argparse
import contextlib
import io
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

    from cverl_b200.cli import vllm_weight_manifest
    from cverl_b200.models.config import Qwen35TextConfig
    from cverl_b200.models.hf_io import synthesize_model_dir
    import ref_common
    src = ref_common.reference_source_dir()
    try:
        exe = ref_common.link_driver(src / "tools" / "rollout" / "vllm_weight_manifest.cc", "vllm_weight_manifest")
    except ref_common.Unavailable as exc:
        print(json.dumps({"unavailable": str(exc)}))
        return 3
    with tempfile.TemporaryDirectory(prefix="cverl_ref_") as tmp:
        work = Path(a.keep) if a.keep else Path(tmp)
        work.mkdir(parents=True, exist_ok=True)
        ok = True
        for moe in (False, True):
            d = synthesize_model_dir(Qwen35TextConfig.tiny(moe=moe), work / f"model_{int(moe)}", seed=3, dtype=torch.float32)
            for flags in (["--send-dtype", "bfloat16", "--no-packed"],
                          ["--send-dtype", "float32", "--packed", "--packed-buffer-size-bytes", "4096",
                           "--packed-num-buffers", "3"]):
                r = subprocess.run([str(exe), "--model-dir", str(d), *flags], capture_output=True, text=True)
                buf = io.StringIO()
                with contextlib.redirect_stdout(buf):
                    vllm_weight_manifest.main(["--model-dir", str(d), *flags])
                same = r.returncode == 0 and json.loads(r.stdout) == json.loads(buf.getvalue())
                ok = ok and same
                print(json.dumps({"model": "qwen3_moe" if moe else "qwen3_5", "flags": flags[:3], "agree": same,
                                  "names": len(json.loads(buf.getvalue())["update_info"]["names"])}))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
