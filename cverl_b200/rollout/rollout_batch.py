"""Builds the tensor batch of a GRPO step from prompts, sampled responses and gold answers.

Prompts are tokenised once per prompt index, LEFT-padded and truncated keeping the tail;
responses are RIGHT-padded; ``response_mask`` marks real response tokens; ``group_ids`` is
the prompt index; the scalar GSM8K rule reward sits on the last real response token.
Reference: src/rollout/rollout_batch.cc:12-136.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..reward import Gsm8kRewardOptions, compute_gsm8k_reward
from ..text import EncodeOptions, Tokenizer


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


def build_gsm8k_rollout_batch(tokenizer: Tokenizer, prompts: Sequence[str], answers: Sequence[str],
                              samples: Sequence[RolloutSample], max_prompt_len: int, max_response_len: int,
                              reward_options: Gsm8kRewardOptions = Gsm8kRewardOptions()) -> RolloutBatch:
    if len(prompts) != len(answers):
        raise ValueError("prompts and answers must have the same length")
    if not samples:
        raise ValueError("no rollout samples")
    pad = tokenizer.pad_id if tokenizer.pad_id >= 0 else 0
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
            cache[s.prompt_index] = tokenizer.encode(prompts[s.prompt_index], EncodeOptions())
        p = cache[s.prompt_index][-max_prompt_len:]          # keep the tail
        if p:
            prompt_ids[b, max_prompt_len - len(p):] = torch.tensor(p, dtype=torch.int64)
        r = s.response_token_ids if s.response_token_ids is not None else tokenizer.encode(s.response_text)
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
