"""Builds the tensor batch of a GRPO step from prompts, sampled responses and gold answers.

Prompts are tokenised once per prompt index with the limit ``max_prompt_len`` (an over-long prompt keeps its
FIRST ``max_prompt_len`` tokens) and LEFT-padded; a response that comes as text is tokenised with the limit
``max_response_len`` and gets an EOS where the limit leaves room (``add_eos``, on by default as in the reference),
a response that comes with token ids keeps its first ``max_response_len`` ids (an empty id list counts as "no
ids": the text is tokenised); responses are RIGHT-padded; ``response_mask`` marks real response tokens;
``group_ids`` is the prompt index; the scalar GSM8K rule reward sits on the last real response token.
Reference: src/rollout/rollout_batch.cc:42-136 (checked against the reference's own function by
``baseline/ref_rollout_batch_check.py``).

With one of the two native tokenizers the whole batch is built by ``cverl_build_gsm8k_rollout_batch``
(csrc/rollout_batch.cc): distinct prompts and then samples are tokenised and scored on several threads, each
writing its own rows of the output tensors.  Any other ``Tokenizer`` takes the Python loop below, which states
the same rules.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..reward import Gsm8kRewardOptions, compute_gsm8k_reward
from ..text import ByteTokenizer, EncodeOptions, HfBpeTokenizer, Tokenizer


@dataclass
class RolloutSample:
    prompt_index: int
    response_text: str
    response_token_ids: Optional[List[int]] = None


@dataclass
class RolloutBatch:
    prompt_ids: torch.Tensor       # [B, P] int64, left padded
    response_ids: torch.Tensor     # [B, R] int64, right padded
    response_mask: torch.Tensor    # [B, R] float32
    token_rewards: torch.Tensor    # [B, R] float32
    rewards: torch.Tensor          # [B] float32
    group_ids: torch.Tensor        # [B] int64

    def to(self, device) -> "RolloutBatch":
        return RolloutBatch(*(getattr(self, f).to(device) for f in self.__dataclass_fields__))


def _build_native(tokenizer, prompts, answers, samples, P: int, R: int, opts: Gsm8kRewardOptions, pad: int,
                  threads: int, add_bos: bool, add_eos: bool) -> RolloutBatch:
    import ctypes as C
    import os

    import numpy as np

    from .. import _native as nv
    lib = nv.host()
    fn = lib.cverl_build_gsm8k_rollout_batch
    i64, i64p, cpp = C.c_int64, C.POINTER(C.c_int64), C.POINTER(C.c_char_p)
    fn.restype = C.c_int
    fn.argtypes = [C.c_int, C.c_void_p, i64, cpp, i64p, cpp, i64, i64p, cpp, i64p, i64p, i64p, C.POINTER(C.c_uint8),
                   i64, i64, i64, C.c_int, C.c_int, i64, i64, C.c_int, i64, C.c_double, C.c_double, C.c_double, C.c_int,
                   i64p, i64p,
                   C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float), i64p]
    B, NP = len(samples), len(prompts)
    praw = [p.encode("utf-8") for p in prompts]
    araw = [a.encode("utf-8") for a in answers]
    rraw = [s.response_text.encode("utf-8") for s in samples]
    idx = np.asarray([s.prompt_index for s in samples], dtype=np.int64)
    has = np.asarray([bool(s.response_token_ids) for s in samples], dtype=np.uint8)
    offs = np.zeros(B + 1, dtype=np.int64)
    np.cumsum([len(s.response_token_ids) if s.response_token_ids else 0 for s in samples], out=offs[1:])
    given = np.asarray([t for s in samples if s.response_token_ids for t in s.response_token_ids] or [0],
                       dtype=np.int64)
    out = RolloutBatch(torch.empty((B, P), dtype=torch.int64), torch.empty((B, R), dtype=torch.int64),
                       torch.empty((B, R), dtype=torch.float32), torch.empty((B, R), dtype=torch.float32),
                       torch.empty(B, dtype=torch.float32), torch.empty(B, dtype=torch.int64))

    def ptr(t, ty):
        return C.cast(t.data_ptr(), C.POINTER(ty))

    def nptr(a, ty):
        return a.ctypes.data_as(C.POINTER(ty))
    is_bpe = isinstance(tokenizer, HfBpeTokenizer)
    if threads <= 0:
        threads = min(os.cpu_count() or 1, 16)
    rc = fn(int(is_bpe), tokenizer._h if is_bpe else None, pad,
            (C.c_char_p * max(NP, 1))(*praw), (i64 * max(NP, 1))(*[len(b) for b in praw]),
            (C.c_char_p * max(NP, 1))(*araw), NP, nptr(idx, i64), (C.c_char_p * B)(*rraw),
            (i64 * B)(*[len(b) for b in rraw]), nptr(given, i64), nptr(offs, i64), nptr(has, C.c_uint8), B, P, R,
            int(add_bos), int(add_eos), tokenizer.bos_id, tokenizer.eos_id, int(opts.method == "flexible"), opts.solution_clip_chars, opts.correct_score, opts.format_score,
            opts.no_answer_score, threads, ptr(out.prompt_ids, i64), ptr(out.response_ids, i64),
            ptr(out.response_mask, C.c_float), ptr(out.token_rewards, C.c_float), ptr(out.rewards, C.c_float),
            ptr(out.group_ids, i64))
    if rc != 0:
        raise ValueError("sample prompt_index out of range")
    return out


def build_gsm8k_rollout_batch(tokenizer: Tokenizer, prompts: Sequence[str], answers: Sequence[str],
                              samples: Sequence[RolloutSample], max_prompt_len: int, max_response_len: int,
                              reward_options: Gsm8kRewardOptions = Gsm8kRewardOptions(),
                              threads: int = 0, add_bos: bool = False, add_eos: bool = True) -> RolloutBatch:
    """``threads``: worker threads of the native builder (0: one per core, at most 16); -1 forces the Python loop.
    ``add_bos`` / ``add_eos``: the reference's ``RolloutBatchOptions`` (include/cverl/rollout/rollout_batch.h:36-41)."""
    if len(prompts) != len(answers):
        raise ValueError("prompts and answers must have the same length")
    if not samples:
        raise ValueError("no rollout samples")
    pad = tokenizer.pad_id if tokenizer.pad_id >= 0 else 0
    if threads >= 0 and type(tokenizer) in (ByteTokenizer, HfBpeTokenizer):
        return _build_native(tokenizer, prompts, answers, samples, max_prompt_len, max_response_len, reward_options,
                             pad, threads, add_bos, add_eos)
    prompt_opts = EncodeOptions(add_bos=add_bos, add_eos=False, max_tokens=max_prompt_len)
    response_opts = EncodeOptions(add_bos=False, add_eos=add_eos, max_tokens=max_response_len)
    cache: Dict[int, List[int]] = {}
    B = len(samples)
    prompt_ids = torch.full((B, max_prompt_len), pad, dtype=torch.int64)
    response_ids = torch.full((B, max_response_len), pad, dtype=torch.int64)
    mask = torch.zeros((B, max_response_len), dtype=torch.float32)
    token_rewards = torch.zeros((B, max_response_len), dtype=torch.float32)
    rewards = torch.zeros(B, dtype=torch.float32)
    group = torch.zeros(B, dtype=torch.int64)
    for b, s in enumerate(samples):
        if not (0 <= s.prompt_index < len(prompts)):
            raise ValueError("sample prompt_index out of range")
        if s.prompt_index not in cache:
            cache[s.prompt_index] = tokenizer.encode(prompts[s.prompt_index], prompt_opts)
        p = cache[s.prompt_index][-max_prompt_len:]          # already cut to the first max_prompt_len tokens
        if p:
            prompt_ids[b, max_prompt_len - len(p):] = torch.tensor(p, dtype=torch.int64)
        r = s.response_token_ids if s.response_token_ids else tokenizer.encode(s.response_text, response_opts)
        r = list(r)[:max_response_len]
        if r:
            response_ids[b, :len(r)] = torch.tensor(r, dtype=torch.int64)
            mask[b, :len(r)] = 1.0
        rew = compute_gsm8k_reward(s.response_text, answers[s.prompt_index], reward_options)
        rewards[b] = rew
        if r:
            token_rewards[b, len(r) - 1] = rew
        group[b] = s.prompt_index
    return RolloutBatch(prompt_ids, response_ids, mask, token_rewards, rewards, group)
