"""Runs the text model forward on given token ids and dumps logits / hidden-state statistics.

``python -m cverl_b200.cli.qwen3_5_forward --model-dir DIR --ids 1,2,3 [--max-layers N] [--dump out.pt]``

Prints a JSON summary (shape, mean, std, first values, arg-max tokens) and optionally saves the fp32
logits; ``--compare other.pt`` reports max abs / relative differences against a previous dump, which
is how a forward is checked against another implementation (reference: tools/model/qwen3_5_forward.cc,
tools/model/compare_qwen3_5_forward.py).
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from ..models.config import Qwen35TextConfig
from ..models.hf_io import HfModelLoader, load_model_weights
from ..models.qwen3_5 import Qwen35Model


def forward_logits(model: Qwen35Model, ids: torch.Tensor) -> torch.Tensor:
    """[B, S] ids -> fp32 logits [B, S, V] (full vocabulary; for inspection, not for training)."""
    with torch.no_grad():
        h = model.forward_hidden(ids)
        w = model.lm_head_weight()
        return h.float() @ w.float().t()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model-dir", required=True)
    ap.add_argument("--ids", default="1,2,3,4")
    ap.add_argument("--max-layers", type=int, default=-1)
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--dump", default="")
    ap.add_argument("--compare", default="")
    a = ap.parse_args(argv)
    loader = HfModelLoader(a.model_dir).load_metadata()
    cfg = loader.config()
    if a.max_layers > 0:
        fields = {k: getattr(cfg, k) for k in cfg.__dataclass_fields__}
        fields.update(num_hidden_layers=a.max_layers, layer_types=cfg.layer_types[:a.max_layers])
        cfg = Qwen35TextConfig(**fields)
    model = Qwen35Model(cfg, dtype=getattr(torch, a.dtype), device=a.device)
    load_model_weights(model, loader)
    ids = torch.tensor([[int(t) for t in a.ids.split(",") if t]], dtype=torch.long, device=a.device)
    logits = forward_logits(model, ids).cpu()
    out = {"shape": list(logits.shape), "mean": float(logits.mean()), "std": float(logits.std()),
           "first": [float(v) for v in logits[0, -1, :8]], "argmax": logits[0].argmax(-1).tolist()}
    if a.dump:
        torch.save({"ids": ids.cpu(), "logits": logits}, a.dump)
    if a.compare:
        other = torch.load(a.compare)["logits"]
        diff = (logits - other).abs()
        out["compare"] = {"max_abs": float(diff.max()), "max_rel": float((diff / (other.abs() + 1e-6)).max()),
                          "argmax_equal": bool((logits.argmax(-1) == other.argmax(-1)).all())}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
