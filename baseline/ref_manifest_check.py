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

    import build_ref
    from cverl_b200.cli import vllm_weight_manifest
    from cverl_b200.models.config import Qwen35TextConfig
    from cverl_b200.models.hf_io import synthesize_model_dir
    ref_lib = HERE / "_ref" / "lib"
    if not (ref_lib / "libcverl_ref.so").exists():
        print(json.dumps({"unavailable": "reference library not built (python baseline/build_ref.py)"}))
        return 3
    paths, src = build_ref.find_paths(), build_ref.default_source_dir()
    with tempfile.TemporaryDirectory(prefix="cverl_refman_") as tmp:
        work = Path(a.keep) if a.keep else Path(tmp)
        work.mkdir(parents=True, exist_ok=True)
        lib = Path(torch.__file__).parent / "lib"
        exe = work / "vllm_weight_manifest"
        incs = [src / "include", HERE / "shim", paths["json_inc"], *paths["torch_inc"]]
        cmd = ["g++", "-std=c++17", "-O1", f"-D_GLIBCXX_USE_CXX11_ABI={paths['cxx11_abi']}",
               str(src / "tools" / "rollout" / "vllm_weight_manifest.cc"), *[f for i in incs for f in ("-I", str(i))],
               "-L", str(ref_lib), "-lcverl_ref", "-L", str(lib), "-ltorch", "-ltorch_cpu", "-lc10",
               f"-Wl,-rpath,{ref_lib}", f"-Wl,-rpath,{lib}", "-o", str(exe)]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            print(json.dumps({"unavailable": "compiling the reference tool failed: " + p.stderr[-300:]}))
            return 3
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
