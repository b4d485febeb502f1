"""Prompt/answer JSONL reader, and the conversion of a Hugging Face dataset split into such a file
(reference: src/data/hf_dataset.cc:145-265)."""
from __future__ import annotations

import ctypes as C
import json
from dataclasses import dataclass
from pathlib import Path
from typing import List, Optional

from .. import _native as nv


@dataclass
class PromptAnswerExample:
    prompt: str
    answer: str


def _lib():
    lib = nv.host()
    if not getattr(lib, "_jsonl_bound", False):
        lib.cverl_jsonl_open.restype = C.c_void_p
        lib.cverl_jsonl_open.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, C.c_int64]
        lib.cverl_jsonl_error.restype = C.c_char_p
        lib.cverl_jsonl_error.argtypes = [C.c_void_p]
        lib.cverl_jsonl_rows.restype = C.c_int64
        lib.cverl_jsonl_rows.argtypes = [C.c_void_p]
        lib.cverl_jsonl_get.restype = C.c_char_p
        lib.cverl_jsonl_get.argtypes = [C.c_void_p, C.c_int64, C.c_int]
        lib.cverl_jsonl_close.argtypes = [C.c_void_p]
        lib._jsonl_bound = True
    return lib


def load_prompt_answer_jsonl(path, prompt_field: str = "prompt", answer_field: str = "answer",
                             max_examples: int = -1) -> List[PromptAnswerExample]:
    """Rows of a JSONL file as (prompt, answer) pairs.  ``max_examples``: negative = every row, 0 = none (the
    reference's rule); numbers and booleans are kept as their JSON text, ``null`` reads as the empty string."""
    lib = _lib()
    h = lib.cverl_jsonl_open(str(path).encode(), prompt_field.encode(), answer_field.encode(), max_examples)
    try:
        err = lib.cverl_jsonl_error(h)
        if err:
            raise ValueError(f"load_prompt_answer_jsonl: {err.decode()}")
        return [PromptAnswerExample(lib.cverl_jsonl_get(h, i, 0).decode(), lib.cverl_jsonl_get(h, i, 1).decode())
                for i in range(lib.cverl_jsonl_rows(h))]
    finally:
        lib.cverl_jsonl_close(h)


DATASET_ALIASES = {"gsm8k": "openai/gsm8k"}


@dataclass
class HfDatasetDownloadResult:
    output_file: Path
    rows: int
    source: str


def _split_files(root: Path, name: Optional[str], split: str) -> List[Path]:
    """Data files of one split inside a dataset snapshot: parquet shards (``<name>/<split>-00000-of-0000N.parquet``,
    the layout of the Hub's converted datasets), or ``<split>.jsonl|json|csv``."""
    bases = [root / name] if name and (root / name).is_dir() else []
    bases.append(root)
    for base in bases:
        for pattern in (f"{split}-*.parquet", f"**/{split}-*.parquet", f"{split}.parquet", f"{split}.jsonl",
                        f"{split}.json", f"{split}.csv", f"**/{split}.jsonl"):
            hits = sorted(base.glob(pattern))
            if hits:
                return hits
    return []


def _rows_of(path: Path):
    if path.suffix == ".parquet":
        import pyarrow.parquet as pq
        for batch in pq.ParquetFile(str(path)).iter_batches():
            yield from batch.to_pylist()
    elif path.suffix == ".jsonl":
        with path.open(encoding="utf-8") as f:
            for line in f:
                if line.strip():
                    yield json.loads(line)
    elif path.suffix == ".json":
        doc = json.loads(path.read_text(encoding="utf-8"))
        yield from (doc if isinstance(doc, list) else doc.get("data", doc.get("rows", [])))
    else:
        import csv
        with path.open(newline="", encoding="utf-8") as f:
            yield from csv.DictReader(f)


def download_hf_dataset(dataset: str, output_file, *, name: Optional[str] = None, split: str = "train",
                        prompt_field: str = "question", answer_field: str = "answer", cache_dir=None,
                        token: Optional[str] = None, max_examples: int = -1,
                        local_files_only: bool = False, trust_remote_code: bool = False) -> HfDatasetDownloadResult:
    """One split of a Hugging Face dataset as a prompt / answer JSONL file.

    ``dataset`` is a Hub id (``gsm8k`` is an alias of ``openai/gsm8k``) or a local directory holding the split's
    parquet / JSONL / JSON / CSV files.  A Hub id is resolved with the ``datasets`` library when it is installed,
    else with ``huggingface_hub.snapshot_download(repo_type="dataset")`` and the snapshot's parquet shards are
    read with ``pyarrow``; ``local_files_only`` keeps both to the local cache.  Every row becomes
    ``{"prompt": str(row[prompt_field]), "answer": str(row[answer_field])}`` (``None`` becomes the empty string);
    a row without the two fields is an error that lists the keys it has.  The reference shells out to a Python
    helper for this (src/data/hf_dataset.cc:214-265, tools/hf_dataset_download.py).
    """
    dataset_id = DATASET_ALIASES.get(dataset, dataset)
    out = Path(output_file)
    out.parent.mkdir(parents=True, exist_ok=True)
    rows_iter, source = None, ""
    root = Path(dataset)
    if root.is_dir():
        files = _split_files(root, name, split)
        if not files:
            raise FileNotFoundError(f"no data files of split '{split}' under {root}")
        rows_iter, source = (r for f in files for r in _rows_of(f)), str(root)
    else:
        try:
            import datasets  # noqa: F401
        except ImportError:
            datasets = None
        if datasets is not None:
            if local_files_only:
                import os
                os.environ["HF_DATASETS_OFFLINE"] = "1"
            extra = {"trust_remote_code": True} if trust_remote_code else {}    # only sent when asked for
            ds = datasets.load_dataset(path=dataset_id, name=name, split=split, cache_dir=cache_dir, token=token,
                                       download_mode="reuse_dataset_if_exists", **extra)
            rows_iter, source = iter(ds), f"datasets:{dataset_id}"
        else:
            from huggingface_hub import snapshot_download
            snap = Path(snapshot_download(repo_id=dataset_id, repo_type="dataset", cache_dir=cache_dir, token=token,
                                          local_files_only=local_files_only,
                                          allow_patterns=["*.parquet", "*.jsonl", "*.json", "*.csv"]))
            files = _split_files(snap, name, split)
            if not files:
                raise FileNotFoundError(f"no data files of split '{split}' in the snapshot of {dataset_id}")
            rows_iter, source = (r for f in files for r in _rows_of(f)), f"hub:{dataset_id}"
    n = 0
    tmp = out.with_suffix(out.suffix + ".tmp")
    with tmp.open("w", encoding="utf-8") as f:
        for row in rows_iter:
            if max_examples >= 0 and n >= max_examples:
                break
            if prompt_field not in row or answer_field not in row:
                raise KeyError(f"dataset row missing {prompt_field!r} or {answer_field!r}; available keys: "
                               f"{sorted(row.keys())}")
            item = {"prompt": "" if row[prompt_field] is None else str(row[prompt_field]),
                    "answer": "" if row[answer_field] is None else str(row[answer_field])}
            f.write(json.dumps(item, ensure_ascii=False) + "\n")
            n += 1
    tmp.replace(out)
    return HfDatasetDownloadResult(out, n, source)
