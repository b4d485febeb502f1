"""CIFAR-10 parquet (the Hugging Face ``uoft-cs/cifar10`` layout: an image column ``img`` / ``image`` and ``label``)
to flat tensors a C++ or Python benchmark can map directly:

``<split>_images.f32`` (float32 [N, 3, 32, 32], normalised with the usual per-channel mean / std),
``<split>_labels.i64`` (int64 [N]) and ``<split>_meta.json`` (shape, dtypes, mean, std).

``python -m cverl_b200.cli.export_cifar10_tensors --parquet train-00000-of-00001.parquet --out-dir data/cifar10``
The reference's exporter: tools/bench/export_hf_cifar10_tensors.py.
"""
from __future__ import annotations

import argparse
import io
import json
import sys
from pathlib import Path

import numpy as np

MEAN = (0.4914, 0.4822, 0.4465)
STD = (0.2470, 0.2435, 0.2616)


def decode(record) -> np.ndarray:
    """One image record (dict with bytes / path, raw bytes, or a PIL image) -> float32 [3, H, W] in [0, 1]."""
    from PIL import Image
    if isinstance(record, dict):
        if record.get("bytes") is not None:
            img = Image.open(io.BytesIO(record["bytes"]))
        elif record.get("path"):
            img = Image.open(record["path"])
        else:
            raise ValueError("image record has neither bytes nor a path")
    elif isinstance(record, (bytes, bytearray)):
        img = Image.open(io.BytesIO(record))
    else:
        img = record
    return np.asarray(img.convert("RGB"), dtype=np.float32).transpose(2, 0, 1) / 255.0


def export(parquet: str, out_dir: str, split: str = "train") -> dict:
    import pyarrow.parquet as pq
    table = pq.read_table(parquet)
    cols = set(table.column_names)
    image_col = "img" if "img" in cols else "image"
    if image_col not in cols or "label" not in cols:
        raise ValueError(f"expected image and label columns, got {table.column_names}")
    images = np.stack([decode(r) for r in table[image_col].to_pylist()])
    labels = np.asarray(table["label"].to_pylist(), dtype=np.int64)
    mean = np.asarray(MEAN, np.float32).reshape(1, 3, 1, 1)
    std = np.asarray(STD, np.float32).reshape(1, 3, 1, 1)
    images = np.ascontiguousarray((images - mean) / std, dtype=np.float32)
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    images.tofile(out / f"{split}_images.f32")
    labels.tofile(out / f"{split}_labels.i64")
    meta = {"source": "huggingface:uoft-cs/cifar10", "parquet": str(parquet), "split": split,
            "examples": int(images.shape[0]), "shape": list(images.shape), "dtype": "float32", "label_dtype": "int64",
            "normalized": True, "mean": list(MEAN), "std": list(STD)}
    (out / f"{split}_meta.json").write_text(json.dumps(meta, indent=2) + "\n")
    return meta


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--parquet", required=True)
    ap.add_argument("--out-dir", required=True)
    ap.add_argument("--split", default="train")
    a = ap.parse_args(argv)
    meta = export(a.parquet, a.out_dir, a.split)
    print(f"exported {meta['examples']} examples to {a.out_dir}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
