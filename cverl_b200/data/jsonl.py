"""Prompt/answer JSONL reader (reference: src/data/hf_dataset.cc:145-265).

``download_hf_dataset`` mirrors the reference's helper that shells out to a Hugging Face
download script; this build runs without network access, so it only resolves files that are
already on disk and raises otherwise.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from pathlib import Path
from typing import List

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
                             max_examples: int = 0) -> List[PromptAnswerExample]:
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


def download_hf_dataset(repo_id: str, filename: str, local_dir) -> Path:
    path = Path(local_dir) / filename
    if path.exists():
        return path
    raise RuntimeError(f"download_hf_dataset: {repo_id}/{filename} is not cached under {local_dir} and this build has "
                       "no network access")
