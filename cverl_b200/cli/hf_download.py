"""Downloads a model snapshot or one dataset file from the Hugging Face hub into a local directory.

``python -m cverl_b200.cli.hf_download model Qwen/Qwen3.5-0.8B --local-dir models/Qwen3.5-0.8B``
``python -m cverl_b200.cli.hf_download dataset openai/gsm8k main/train-00000-of-00001.parquet --local-dir data``

Prints ``CVERL_HF_LOCAL_DIR=<dir>`` or ``CVERL_HF_DATASET_FILE=<path>`` on success, the lines the reference's
helpers parse (src/hf_downloader.cc:69-108, src/data/hf_dataset.cc).  Needs ``huggingface_hub`` and network
access; a file that is already cached under ``--local-dir`` is returned without contacting the hub.
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path


def download_hf_snapshot(repo_id: str, local_dir, allow_patterns=None) -> Path:
    local = Path(local_dir)
    if (local / "config.json").exists() and any(local.glob("*.safetensors")):
        return local
    try:
        from huggingface_hub import snapshot_download
    except ImportError as exc:
        raise RuntimeError("download_hf_snapshot needs the huggingface_hub package") from exc
    return Path(snapshot_download(repo_id=repo_id, local_dir=str(local), allow_patterns=allow_patterns))


def download_hf_dataset_file(repo_id: str, filename: str, local_dir) -> Path:
    path = Path(local_dir) / filename
    if path.exists():
        return path
    try:
        from huggingface_hub import hf_hub_download
    except ImportError as exc:
        raise RuntimeError("download_hf_dataset_file needs the huggingface_hub package") from exc
    return Path(hf_hub_download(repo_id=repo_id, filename=filename, repo_type="dataset", local_dir=str(local_dir)))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="kind", required=True)
    m = sub.add_parser("model")
    m.add_argument("repo_id")
    m.add_argument("--local-dir", required=True)
    d = sub.add_parser("dataset")
    d.add_argument("repo_id")
    d.add_argument("filename")
    d.add_argument("--local-dir", required=True)
    a = ap.parse_args(argv)
    try:
        if a.kind == "model":
            print(f"CVERL_HF_LOCAL_DIR={download_hf_snapshot(a.repo_id, a.local_dir)}")
        else:
            print(f"CVERL_HF_DATASET_FILE={download_hf_dataset_file(a.repo_id, a.filename, a.local_dir)}")
    except Exception as exc:  # no network, missing package, unknown repository
        print(f"hf_download failed: {exc}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
