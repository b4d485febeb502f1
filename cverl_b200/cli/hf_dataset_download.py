"""Writes one split of a Hugging Face dataset (Hub id or local directory) as prompt / answer JSONL.

``python -m cverl_b200.cli.hf_dataset_download --dataset gsm8k --name main --split train --output-file gsm8k.jsonl``

Prints ``CVERL_HF_DATASET_FILE=<path>`` and ``CVERL_HF_DATASET_ROWS=<n>``, the two markers the reference's helper
prints (tools/hf_dataset_download.py, tools/data/hf_dataset_download.cc).
"""
from __future__ import annotations

import argparse
import sys

from ..data import download_hf_dataset


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--dataset", required=True)
    ap.add_argument("--name")
    ap.add_argument("--split", default="train")
    ap.add_argument("--prompt-field", default="question")
    ap.add_argument("--answer-field", default="answer")
    ap.add_argument("--output-file", required=True)
    ap.add_argument("--cache-dir")
    ap.add_argument("--token")
    ap.add_argument("--max-examples", type=int, default=-1)
    ap.add_argument("--local-files-only", action="store_true")
    ap.add_argument("--trust-remote-code", action="store_true",
                    help="let the datasets library run the loading script a dataset repository ships")
    a = ap.parse_args(argv)
    res = download_hf_dataset(a.dataset, a.output_file, name=a.name, split=a.split, prompt_field=a.prompt_field,
                              answer_field=a.answer_field, cache_dir=a.cache_dir, token=a.token,
                              max_examples=a.max_examples, local_files_only=a.local_files_only,
                              trust_remote_code=a.trust_remote_code)
    print(f"CVERL_HF_DATASET_FILE={res.output_file}")
    print(f"CVERL_HF_DATASET_ROWS={res.rows}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
