"""GSM8K rule reward: strict ``#### <number>`` or flexible last-number extraction
(reference: src/reward/gsm8k.cc:14-156); implemented in csrc/text_reward.cc."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence

from .. import _native as nv


@dataclass
class Gsm8kRewardOptions:
    method: str = "strict"          # "strict" or "flexible"
    correct_score: float = 1.0
    format_score: float = 0.0
    no_answer_score: float = 0.0
    solution_clip_chars: int = 300


def _lib():
    lib = nv.host()
    if not getattr(lib, "_gsm_bound", False):
        lib.cverl_gsm8k_extract.argtypes = [C.c_char_p, C.c_int, C.c_int64, C.c_char_p, C.c_int64]
        lib.cverl_gsm8k_reward.restype = C.c_double
        lib.cverl_gsm8k_reward.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.c_int64, C.c_double, C.c_double,
                                           C.c_double]
        lib.cverl_gsm8k_normalize_gold.argtypes = [C.c_char_p, C.c_char_p, C.c_int64]
        lib._gsm_bound = True
    return lib


def extract_gsm8k_answer(solution: str, options: Gsm8kRewardOptions = Gsm8kRewardOptions()) -> Optional[str]:
    buf = C.create_string_buffer(512)
    ok = _lib().cverl_gsm8k_extract(solution.encode(), int(options.method == "flexible"),
                                    options.solution_clip_chars, buf, 512)
    return buf.value.decode() if ok else None


def normalize_gsm8k_ground_truth(gold: str) -> str:
    buf = C.create_string_buffer(len(gold.encode()) + 16)
    _lib().cverl_gsm8k_normalize_gold(gold.encode(), buf, len(buf))
    return buf.value.decode()


def compute_gsm8k_reward(solution: str, ground_truth: str,
                         options: Gsm8kRewardOptions = Gsm8kRewardOptions()) -> float:
    return _lib().cverl_gsm8k_reward(solution.encode(), ground_truth.encode(), int(options.method == "flexible"),
                                     options.solution_clip_chars, options.correct_score, options.format_score,
                                     options.no_answer_score)


def compute_gsm8k_rewards(solutions: Sequence[str], ground_truths: Sequence[str],
                          options: Gsm8kRewardOptions = Gsm8kRewardOptions()) -> List[float]:
    if len(solutions) != len(ground_truths):
        raise ValueError("compute_gsm8k_rewards: size mismatch")
    return [compute_gsm8k_reward(s, g, options) for s, g in zip(solutions, ground_truths)]
