"""Prints the parsed text config and the tensor index of a Hugging Face model directory.

``python -m cverl_b200.cli.inspect_hf_model DIR [--tensors] [--check] [--find TEXT] [--load-tensor NAME] [--load-all]``

``--check`` verifies that every tensor the text model requires is present with the expected shape
(reference: tools/model/inspect_hf_model.cc).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import sys

from ..models.hf_io import HfModelLoader
from ..models.params import model_param_specs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("model_dir_positional", nargs="?", default="", help="model directory (the reference's argv[1])")
    ap.add_argument("--model-dir", default="")
    ap.add_argument("--tensors", action="store_true", help="list every tensor with dtype and shape")
    ap.add_argument("--check", action="store_true", help="verify required tensors and shapes")
    ap.add_argument("--find", default="", help="list the tensors whose name contains this text")
    ap.add_argument("--load-tensor", default="", help="read one tensor and report dtype, shape and bytes")
    ap.add_argument("--load-all", action="store_true", help="read every tensor and report count, bytes and seconds")
    a = ap.parse_args(argv)
    a.model_dir = a.model_dir or a.model_dir_positional
    if not a.model_dir:
        ap.error("a model directory is required")
    loader = HfModelLoader(a.model_dir).load_metadata()
    cfg = loader.config()
    names = loader.names()
    total = sum(loader.info(n).nbytes for n in names)
    out = {"model_dir": a.model_dir, "config": dataclasses.asdict(cfg), "num_tensors": len(names),
           "total_bytes": total}
    if a.tensors:
        out["tensors"] = [{"name": n, "dtype": str(loader.info(n).dtype).replace("torch.", ""),
                           "shape": list(loader.info(n).shape)} for n in names]
    if a.find:
        hits = [n for n in names if a.find in n]
        out["matches"] = [{"name": n, "dtype": str(loader.info(n).dtype).replace("torch.", ""),
                           "shape": list(loader.info(n).shape)} for n in hits]
        out["match_count"] = len(hits)
    if a.load_tensor:
        t = loader.load_tensor(a.load_tensor)
        out["loaded_tensor"] = {"name": a.load_tensor, "dtype": str(t.dtype).replace("torch.", ""),
                                "shape": list(t.shape), "nbytes": t.numel() * t.element_size()}
    if a.load_all:
        import time
        t0 = time.perf_counter()
        nbytes = 0
        for n in names:
            t = loader.load_tensor(n)
            nbytes += t.numel() * t.element_size()
        out["loaded_all"] = {"tensor_count": len(names), "nbytes": nbytes,
                             "seconds": round(time.perf_counter() - t0, 4)}
    rc = 0
    if a.check:
        problems = []
        for spec in model_param_specs(cfg):
            if not loader.has(spec.name):
                problems.append(f"missing {spec.name}")
            elif tuple(loader.info(spec.name).shape) != tuple(spec.full_shape):
                problems.append(f"shape of {spec.name}: {tuple(loader.info(spec.name).shape)} != {tuple(spec.full_shape)}")
        out["check"] = {"ok": not problems, "problems": problems}
        rc = 0 if not problems else 2
    print(json.dumps(out, indent=2, default=str))
    return rc


if __name__ == "__main__":
    sys.exit(main())
