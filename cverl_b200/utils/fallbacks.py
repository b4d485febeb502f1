"""Counting and announcing every time a hot op leaves its native kernel for a library or PyTorch path.

A CUDA tensor whose shape or dtype a kernel does not accept is served by a slower path (``torch`` SDPA, the
PyTorch statement of the chunked scan, cuBLAS).  That must never happen silently on a GPU run: ``note`` counts
the event under ``(op, reason)``, warns the first time each pair is seen, and raises instead when
``CVERL_B200_STRICT=1``.  ``counts()`` / ``reset()`` let trainers and tests read the tally.
"""
from __future__ import annotations

import os
import warnings
from collections import Counter
from typing import Dict, Tuple

_counts: Counter = Counter()


class NativeKernelFallback(UserWarning):
    pass


def note(op: str, reason: str) -> None:
    key = (op, reason)
    _counts[key] += 1
    if os.environ.get("CVERL_B200_STRICT") == "1":
        raise RuntimeError(f"{op}: native kernel not used ({reason}) and CVERL_B200_STRICT=1")
    if _counts[key] == 1:
        warnings.warn(f"{op}: native sm_100a kernel not used ({reason}); running the library / PyTorch path. "
                      f"Further occurrences are counted, not printed.", NativeKernelFallback, stacklevel=3)


def counts() -> Dict[Tuple[str, str], int]:
    return dict(_counts)


def total() -> int:
    return sum(_counts.values())


def reset() -> None:
    _counts.clear()
