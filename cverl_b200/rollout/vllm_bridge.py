"""Bridge object for an external rollout engine (vLLM): live weights, update manifest, GRPO update.

``QwenPolicy`` owns the tokenizer, the trainable Qwen policy, a lazily created frozen reference copy
and an AdamW optimizer.  An online loop generates with the serving engine, calls
``gsm8k_grpo_update(prompts, responses, answers, prompt_indices, sample_indices, ...)`` for the
actor step, then pushes ``named_parameters()`` (live tensors under their Hugging Face names) with the
metadata from ``update_info()``.  Same surface and metric keys as the reference's pybind module
(python/cverl_vllm_bridge.cc:68-352); here it is plain Python because the framework layer already is.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..models.policy import Qwen3_5CausalLmPolicy
from ..reward.gsm8k import Gsm8kRewardOptions
from ..text.tokenizer import ByteTokenizer, HfBpeTokenizer
from ..trainer.gsm8k_grpo import GrpoUpdateConfig, grpo_update
from .rollout_batch import RolloutSample, build_gsm8k_rollout_batch

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


class QwenPolicy:
    def __init__(self, model_dir: str, tokenizer_path: str = "", device: str = "cuda:0", param_dtype: str = "float32",
                 max_layers: int = -1):
        if param_dtype not in _DTYPES:
            raise ValueError("param_dtype must be float32|bfloat16|float16")
        self.model_dir, self.device, self.dtype_name = model_dir, torch.device(device), param_dtype
        tok = tokenizer_path or f"{model_dir}/tokenizer.json"
        try:
            self.tokenizer = HfBpeTokenizer(tok)
        except Exception:
            self.tokenizer = ByteTokenizer()
        pad = self.tokenizer.pad_id if self.tokenizer.pad_id >= 0 else 0
        self.policy = Qwen3_5CausalLmPolicy.from_model_dir(model_dir, _DTYPES[param_dtype], device="cpu", pad_id=pad,
                                                           max_layers=max_layers)
        self.policy.to_device(self.device)
        self.reference: Optional[Qwen3_5CausalLmPolicy] = None
        self.optimizer: Optional[torch.optim.Optimizer] = None
        self._opt_key = None

    def to_device(self, device: str) -> "QwenPolicy":
        self.device = torch.device(device)
        self.policy.to_device(self.device)
        if self.reference is not None:
            self.reference.to_device(self.device)
        self.optimizer = None      # state tensors lived on the old device
        return self

    def named_parameters(self) -> List[tuple]:
        """``[(hf_name, live tensor)]``: views of the policy's parameters, not copies."""
        return self.policy.named_hf_parameters()

    def update_info(self, packed: bool = True, packed_buffer_size_bytes: int = 1 << 30,
                    packed_num_buffers: int = 2) -> Dict:
        names, dtypes, shapes = [], [], []
        for n, t in self.named_parameters():
            names.append(n)
            dtypes.append(self.dtype_name)
            shapes.append(list(t.shape))
        return {"names": names, "dtype_names": dtypes, "shapes": shapes, "packed": packed,
                "packed_buffer_size_bytes": packed_buffer_size_bytes, "packed_num_buffers": packed_num_buffers,
                "is_checkpoint_format": False}

    def gsm8k_grpo_update(self, prompts: Sequence[str], responses: Sequence[str], answers: Sequence[str],
                          prompt_indices: Sequence[int], sample_indices: Sequence[int], max_prompt_tokens: int = 256,
                          max_response_tokens: int = 256, ppo_epochs: int = 1, learning_rate: float = 3.0e-6,
                          weight_decay: float = 0.0, clip_ratio: float = 0.2, kl_coef: float = 0.0,
                          reward_method: str = "flexible", measure_param_delta: bool = False) -> Dict[str, float]:
        """One actor update from externally generated responses.  ``responses[i]`` answers
        ``prompts[prompt_indices[i]]``; ``sample_indices`` numbers the samples of one prompt (kept for the
        caller's bookkeeping).  Returns the metrics dict of the last PPO epoch."""
        if not (len(responses) == len(prompt_indices) == len(sample_indices)):
            raise ValueError("responses, prompt_indices and sample_indices must have the same length")
        if len(prompts) != len(answers):
            raise ValueError("prompts and answers must have the same length")
        samples = [RolloutSample(int(pi), r) for pi, r in zip(prompt_indices, responses)]
        batch = build_gsm8k_rollout_batch(self.tokenizer, prompts, answers, samples, max_prompt_tokens,
                                          max_response_tokens, Gsm8kRewardOptions(method=reward_method)).to(self.device)
        key = (learning_rate, weight_decay)
        if self.optimizer is None or self._opt_key != key:
            self.optimizer = torch.optim.AdamW(self.policy.parameters(), lr=learning_rate, weight_decay=weight_decay)
            self._opt_key = key
        if kl_coef != 0.0 and self.reference is None:
            self.reference = self.policy.clone_as_reference()
        cfg = GrpoUpdateConfig(ppo_epochs=ppo_epochs, clip_ratio=clip_ratio, kl_coef=kl_coef)
        with torch.no_grad():
            from ..ops import rl
            adv, _ = rl.grpo_outcome_advantage(batch.token_rewards, batch.response_mask, batch.group_ids, cfg.epsilon,
                                               cfg.norm_adv_by_std)
            adv_abs_sum = float(adv.abs().sum())
        m = grpo_update(self.policy, self.reference, self.optimizer, batch, cfg)
        rewards = batch.rewards.float()
        out = {"total_seq": float(len(samples)), "mean_reward": float(rewards.mean()),
               "success_rate": float((rewards >= 0.999).float().mean()), "adv_abs_sum": adv_abs_sum,
               "loss": m["loss"], "pg_loss": m["pg_loss"], "kl_loss": m["kl_loss"], "ppo_kl": m["ppo_kl"],
               "clipfrac": m["clipfrac"], "param_delta": m["param_delta"] if measure_param_delta else 0.0}
        return out
