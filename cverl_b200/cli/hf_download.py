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


def download_hf_snapshot(repo_id: str, local_dir, allow_patterns=None, *, revision=None, cache_dir=None, token=None,
                         ignore_patterns=None, local_files_only: bool = False) -> Path:
    """Model snapshot into ``local_dir`` (returned as it is when it already holds a config and safetensors files).
    The keyword options are those of the reference's wrapper (tools/hf_snapshot_download.py)."""
    local = Path(local_dir) if local_dir else None
    if local is not None and (local / "config.json").exists() and any(local.glob("*.safetensors")):
        return local
    try:
        from huggingface_hub import snapshot_download
    except ImportError as exc:
        raise RuntimeError("download_hf_snapshot needs the huggingface_hub package") from exc
    return Path(snapshot_download(repo_id=repo_id, revision=revision, local_dir=str(local) if local else None,
                                  cache_dir=cache_dir or None, token=token or None,
                                  allow_patterns=allow_patterns or None, ignore_patterns=ignore_patterns or None,
                                  local_files_only=local_files_only))


def snapshot_info(repo_id: str, revision=None, token=None) -> dict:
    """What a dry run prints: the commit and the number of files of a model repository."""
    try:
        from huggingface_hub import model_info
    except ImportError as exc:
        raise RuntimeError("snapshot_info needs the huggingface_hub package") from exc
    info = model_info(repo_id, revision=revision, token=token)
    return {"repo_id": repo_id, "sha": info.sha, "file_count": len(info.siblings or [])}


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
    m.add_argument("--local-dir", default="")
    m.add_argument("--revision")
    m.add_argument("--cache-dir")
    m.add_argument("--token")
    m.add_argument("--allow-pattern", action="append", default=[])
    m.add_argument("--ignore-pattern", action="append", default=[])
    m.add_argument("--local-files-only", action="store_true")
    m.add_argument("--dry-run", action="store_true", help="print the repository's commit and file count, download nothing")
    d = sub.add_parser("dataset")
    d.add_argument("repo_id")
    d.add_argument("filename")
    d.add_argument("--local-dir", required=True)
    argv = list(sys.argv[1:] if argv is None else argv)
    if "--repo-id" in argv and (not argv or argv[0] not in ("model", "dataset")):
        # the reference's form (tools/hf_snapshot_download.py): --repo-id ID [options], no sub-command
        i = argv.index("--repo-id")
        if i + 1 >= len(argv):
            ap.error("--repo-id needs a value")
        argv = ["model", argv[i + 1]] + argv[:i] + argv[i + 2:]
    a = ap.parse_args(argv)
    try:
        if a.kind == "model" and a.dry_run:
            info = snapshot_info(a.repo_id, a.revision, a.token)
            print(f"CVERL_HF_REPO_ID={info['repo_id']}\nCVERL_HF_SHA={info['sha']}\n"
                  f"CVERL_HF_FILE_COUNT={info['file_count']}\nCVERL_HF_LOCAL_DIR={a.local_dir}")
        elif a.kind == "model":
            path = download_hf_snapshot(a.repo_id, a.local_dir, a.allow_pattern, revision=a.revision,
                                        cache_dir=a.cache_dir, token=a.token, ignore_patterns=a.ignore_pattern,
                                        local_files_only=a.local_files_only)
            print(f"CVERL_HF_LOCAL_DIR={path}")
        else:
            print(f"CVERL_HF_DATASET_FILE={download_hf_dataset_file(a.repo_id, a.filename, a.local_dir)}")
    except Exception as exc:  # no network, missing package, unknown repository
        print(f"hf_download failed: {exc}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
