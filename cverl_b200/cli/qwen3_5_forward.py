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


TENSOR_MAGIC = b"CVTENSR1"


def save_tensor_binary(t: torch.Tensor, path) -> None:
    """The reference's raw tensor file (tools/model/qwen3_5_forward.cc:77-96): 8-byte magic ``CVTENSR1``, int64
    rank, int64 extents, fp32 values in row-major order - what its comparison script reads."""
    import struct
    out = t.detach().cpu().contiguous().float()
    with open(path, "wb") as f:
        f.write(TENSOR_MAGIC)
        f.write(struct.pack("<q", out.dim()))
        f.write(struct.pack(f"<{out.dim()}q", *out.shape))
        f.write(out.numpy().tobytes())


def load_tensor_binary(path) -> torch.Tensor:
    import struct

    import numpy as np
    raw = open(path, "rb").read()
    if raw[:8] != TENSOR_MAGIC:
        raise ValueError(f"{path}: not a CVTENSR1 tensor file")
    (rank,) = struct.unpack_from("<q", raw, 8)
    if not 0 <= rank <= 8:
        raise ValueError(f"{path}: bad rank {rank}")
    shape = struct.unpack_from(f"<{rank}q", raw, 16)
    n = 1
    for d in shape:
        n *= d
    data = np.frombuffer(raw, dtype="<f4", count=n, offset=16 + 8 * rank)
    return torch.from_numpy(data.copy()).reshape(shape)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("model_dir_positional", nargs="?", default="", help="model directory (the reference's argv[1])")
    ap.add_argument("--model-dir", default="")
    ap.add_argument("--ids", "--tokens", dest="ids", default="1,2,3,4")
    ap.add_argument("--max-layers", "--layers", dest="max_layers", type=int, default=-1)
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--logits", action="store_true", help="the default output; accepted for the reference's command lines")
    ap.add_argument("--hidden", action="store_true", help="output the final-normed hidden states instead of logits")
    ap.add_argument("--dump", default="")
    ap.add_argument("--save-output", default="", help="write the output tensor as a CVTENSR1 raw file")
    ap.add_argument("--compare", default="")
    a = ap.parse_args(argv)
    a.model_dir = a.model_dir or a.model_dir_positional
    if not a.model_dir:
        ap.error("a model directory is required")
    loader = HfModelLoader(a.model_dir).load_metadata()
    cfg = loader.config()
    if a.max_layers > 0:
        fields = {k: getattr(cfg, k) for k in cfg.__dataclass_fields__}
        fields.update(num_hidden_layers=a.max_layers, layer_types=cfg.layer_types[:a.max_layers])
        cfg = Qwen35TextConfig(**fields)
    model = Qwen35Model(cfg, dtype=getattr(torch, a.dtype), device=a.device)
    load_model_weights(model, loader)
    ids = torch.tensor([[int(t) for t in a.ids.split(",") if t]], dtype=torch.long, device=a.device)
    if a.hidden:
        with torch.no_grad():
            logits = model.forward_hidden(ids).float().cpu()        # [1, S, H]; named for the code below
    else:
        logits = forward_logits(model, ids).cpu()
    out = {"shape": list(logits.shape), "mean": float(logits.mean()), "std": float(logits.std()),
           "first": [float(v) for v in logits[0, -1, :8]], "argmax": logits[0].argmax(-1).tolist(),
           "output": "hidden" if a.hidden else "logits", "tokens": int(ids.shape[1]), "layers": cfg.num_hidden_layers}
    if not a.hidden:
        out["top5_token_ids"] = logits[0, -1].topk(min(5, logits.shape[-1])).indices.tolist()
    if a.save_output:
        save_tensor_binary(logits, a.save_output)
        out["saved_output"] = a.save_output
    if a.dump:
        torch.save({"ids": ids.cpu(), "logits": logits}, a.dump)
    if a.compare:
        other = load_tensor_binary(a.compare) if open(a.compare, "rb").read(8) == TENSOR_MAGIC else \
            torch.load(a.compare)["logits"]
        diff = (logits - other).abs()
        out["compare"] = {"max_abs": float(diff.max()), "max_rel": float((diff / (other.abs() + 1e-6)).max()),
                          "argmax_equal": bool((logits.argmax(-1) == other.argmax(-1)).all())}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
