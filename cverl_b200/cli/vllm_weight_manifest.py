"""Prints the weight-update manifest a vLLM weight-transfer engine expects for a model directory.

``python -m cverl_b200.cli.vllm_weight_manifest --model-dir DIR [--send-dtype bfloat16] [--no-packed]``

JSON: ``backend``, ``model_dir`` and ``update_info`` with parallel ``names`` / ``dtype_names`` / ``shapes``
lists (every tensor the text model requires, in model order), the packing options and
``is_checkpoint_format: false``.  Same content as the reference tool
(tools/rollout/vllm_weight_manifest.cc:24-81).
"""
from __future__ import annotations

import argparse
import json
import sys

from ..models.hf_io import HfModelLoader
from ..models.params import required_weight_names


def build_update_info(model_dir: str, send_dtype: str = "float32", packed: bool = True,
                      packed_buffer_size_bytes: int = 1 << 30, packed_num_buffers: int = 2) -> dict:
    if send_dtype not in ("float32", "bfloat16", "float16"):
        raise ValueError("--send-dtype must be float32|bfloat16|float16")
    loader = HfModelLoader(model_dir).load_metadata()
    cfg = loader.config()
    names = required_weight_names(cfg)
    return {"names": names, "dtype_names": [send_dtype] * len(names),
            "shapes": [list(loader.info(n).shape) for n in names], "packed": packed,
            "packed_buffer_size_bytes": packed_buffer_size_bytes, "packed_num_buffers": packed_num_buffers,
            "is_checkpoint_format": False}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model-dir", required=True)
    ap.add_argument("--send-dtype", default="float32")
    ap.add_argument("--packed", dest="packed", action="store_true", default=True)
    ap.add_argument("--no-packed", dest="packed", action="store_false")
    ap.add_argument("--packed-buffer-size-bytes", type=int, default=1 << 30)
    ap.add_argument("--packed-num-buffers", type=int, default=2)
    a = ap.parse_args(argv)
    info = build_update_info(a.model_dir, a.send_dtype, a.packed, a.packed_buffer_size_bytes, a.packed_num_buffers)
    print(json.dumps({"backend": "vllm_native_rl_nccl", "model_dir": a.model_dir, "update_info": info}, indent=2))
    return 0


if __name__ == "__main__":
    sys.exit(main())
