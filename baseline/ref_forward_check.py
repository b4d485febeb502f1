"""Forward parity with the reference itself: its own, unmodified forward tool against this package's model.

    python baseline/ref_forward_check.py [--keep DIR] [--tokens 5,6,7,...]

Compiles the reference's ``tools/model/qwen3_5_forward.cc`` as it is, links it against the reference library that
``baseline/build_ref.py`` built (``baseline/_ref/lib/libcverl_ref.so``), and runs it on CPU in fp32 on two small
random model directories written by this package (Qwen3.5 hybrid: Gated-DeltaNet + full attention layers; Qwen3-MoE)
- once for the final hidden states, once for the logits (``--save-output``: its raw ``CVTENSR1`` tensor file).  This
package's forward of the same directory and tokens is compared element by element.  One JSON line per case; exit
code 0 when every case agrees within ``--atol`` (default 2e-5), 3 when the reference library is not built.
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
    ap.add_argument("--tokens", default="5,6,7,8,9,42,100,3,17,250,11,2,77,1,300,64,8")
    ap.add_argument("--atol", type=float, default=2e-5)
    a = ap.parse_args(argv)
    import torch

    from cverl_b200.cli import qwen3_5_forward as fwd
    from cverl_b200.models.config import Qwen35TextConfig
    from cverl_b200.models.hf_io import HfModelLoader, load_model_weights, synthesize_model_dir
    from cverl_b200.models.qwen3_5 import Qwen35Model
    import ref_common
    src = ref_common.reference_source_dir()
    try:
        exe = ref_common.link_driver(src / "tools" / "model" / "qwen3_5_forward.cc", "qwen3_5_forward")
    except ref_common.Unavailable as exc:
        print(json.dumps({"unavailable": str(exc)}))
        return 3
    with tempfile.TemporaryDirectory(prefix="cverl_ref_") as tmp:
        work = Path(a.keep) if a.keep else Path(tmp)
        work.mkdir(parents=True, exist_ok=True)
        ids = torch.tensor([[int(t) for t in a.tokens.split(",") if t]], dtype=torch.long)
        ok = True
        for moe in (False, True):
            cfg = Qwen35TextConfig.tiny(moe=moe)
            d = synthesize_model_dir(cfg, work / f"model_{int(moe)}", seed=11, dtype=torch.float32)
            loader = HfModelLoader(d).load_metadata()
            model = Qwen35Model(loader.config(), dtype=torch.float32)
            load_model_weights(model, loader)
            for logits in (False, True):
                raw = work / f"ref_{int(moe)}_{int(logits)}.bin"
                r = subprocess.run([str(exe), str(d), "--tokens", a.tokens, *(["--logits"] if logits else []),
                                    "--save-output", str(raw), "--device", "cpu"], capture_output=True, text=True)
                row = {"model": "qwen3_moe" if moe else "qwen3_5", "output": "logits" if logits else "hidden"}
                if r.returncode != 0:
                    row.update(agree=False, error=r.stderr[-300:])
                else:
                    ref = fwd.load_tensor_binary(raw)
                    with torch.no_grad():
                        mine = (fwd.forward_logits(model, ids) if logits else model.forward_hidden(ids)).float()
                    diff = (mine - ref).abs()
                    row.update(shape=list(ref.shape), max_abs=float(diff.max()), ref_abs_max=float(ref.abs().max()),
                               argmax_equal=bool((mine.argmax(-1) == ref.argmax(-1)).all()),
                               agree=bool(list(mine.shape) == list(ref.shape) and float(diff.max()) <= a.atol))
                ok = ok and row["agree"]
                print(json.dumps(row))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
