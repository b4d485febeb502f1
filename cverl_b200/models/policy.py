"""Causal-LM policies: the interface the rollout worker and the single-GPU trainers use.

``CausalLmPolicy.forward(prompt_ids [B,P], response_ids [B,R]) -> logits [B,R,V]`` where row
``t`` predicts ``response_ids[:, t]`` (include/cverl/torch/causal_lm_policy.h:30-58).
``TinyCausalLmPolicy`` is the toy model of the reference (embedding -> masked running mean of
the prefix -> Linear -> ReLU -> Linear, src/torch/tiny_causal_policy.cc:19-97);
``Qwen3_5CausalLmPolicy`` wraps ``Qwen35Model`` (src/torch/qwen3_5_causal_lm_policy.cc:12-175).
"""
from __future__ import annotations

import abc
import copy
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from .config import Qwen35TextConfig
from .hf_io import HfModelLoader, load_model_weights, save_hf_checkpoint
from .qwen3_5 import Qwen35Model


@dataclass
class CausalLmPolicyOptions:
    kind: str = "tiny"            # "tiny" or "qwen3_5"
    vocab_size: int = 260
    hidden_size: int = 64
    pad_id: int = 0
    model_dir: str = ""
    param_dtype: torch.dtype = torch.float32
    max_layers: int = -1


def response_log_probs(logits: torch.Tensor, response_ids: torch.Tensor) -> torch.Tensor:
    """log_softmax(logits)[b, t, response_ids[b, t]] -> [B, R] (fp32)."""
    return torch.log_softmax(logits.float(), dim=-1).gather(-1, response_ids.long().unsqueeze(-1)).squeeze(-1)


class CausalLmPolicy(nn.Module, abc.ABC):
    @abc.abstractmethod
    def forward(self, prompt_ids: torch.Tensor, response_ids: torch.Tensor) -> torch.Tensor: ...

    @property
    @abc.abstractmethod
    def vocab_size(self) -> int: ...

    @property
    @abc.abstractmethod
    def pad_id(self) -> int: ...

    def to_device(self, device) -> "CausalLmPolicy":
        return self.to(device)

    def clone_as_reference(self) -> "CausalLmPolicy":
        """A frozen deep copy (the KL reference policy)."""
        ref = copy.deepcopy(self)
        for p in ref.parameters():
            p.requires_grad_(False)
        ref.eval()
        return ref

    def save_hf_checkpoint(self, out_dir, dtype: Optional[torch.dtype] = None) -> None:
        raise NotImplementedError(f"{type(self).__name__} has no Hugging Face export")

    def response_log_probs(self, prompt_ids, response_ids) -> torch.Tensor:
        return response_log_probs(self.forward(prompt_ids, response_ids), response_ids)


class TinyCausalLmPolicy(CausalLmPolicy):
    def __init__(self, vocab_size: int = 260, hidden_size: int = 64, pad_id: int = 0):
        super().__init__()
        self._vocab, self._pad = vocab_size, pad_id
        self.embed = nn.Embedding(vocab_size, hidden_size)
        self.fc1 = nn.Linear(hidden_size, hidden_size)
        self.fc2 = nn.Linear(hidden_size, vocab_size)

    @property
    def vocab_size(self) -> int:
        return self._vocab

    @property
    def pad_id(self) -> int:
        return self._pad

    def forward(self, prompt_ids, response_ids):
        P = prompt_ids.shape[1]
        R = response_ids.shape[1]
        ids = torch.cat([prompt_ids, response_ids], dim=1).long()
        mask = (ids != self._pad).to(self.embed.weight.dtype).unsqueeze(-1)
        e = self.embed(ids) * mask
        csum = e.cumsum(1)
        cnt = mask.cumsum(1).clamp_min(1.0)
        mean = csum / cnt                                   # running mean over the prefix up to each position
        ctx = mean[:, P - 1:P - 1 + R]                      # position P-1+t has seen the prompt and response[:t]
        return self.fc2(torch.relu(self.fc1(ctx)))


class Qwen3_5CausalLmPolicy(CausalLmPolicy):
    """Policy over the full Qwen3.5 / Qwen3-MoE model (single rank, no tensor parallelism)."""

    def __init__(self, cfg: Qwen35TextConfig, param_dtype=torch.float32, device="cpu", model_dir: str = "",
                 pad_id: int = 0):
        super().__init__()
        self.model = Qwen35Model(cfg, dtype=param_dtype, device=device, with_main_grad=False)
        self.model_dir = model_dir
        self._pad = pad_id

    @classmethod
    def from_model_dir(cls, model_dir, param_dtype=torch.float32, device="cpu", pad_id: int = 0,
                       max_layers: int = -1):
        loader = HfModelLoader(model_dir).load_metadata()
        cfg = loader.config()
        if 0 < max_layers < cfg.num_hidden_layers:   # a truncated stack for smoke runs
            fields = {k: getattr(cfg, k) for k in cfg.__dataclass_fields__}
            fields.update(num_hidden_layers=max_layers, layer_types=cfg.layer_types[:max_layers])
            cfg = Qwen35TextConfig(**fields)
        pol = cls(cfg, param_dtype, device, str(model_dir), pad_id)
        load_model_weights(pol.model, loader)
        return pol

    @property
    def vocab_size(self) -> int:
        return self.model.cfg.vocab_size

    @property
    def pad_id(self) -> int:
        return self._pad

    def to_device(self, device):
        # the flat buffer and every view move together; a plain .to() would break the aliasing
        dev = torch.device(device)
        if self.model.flat.flat.device == dev:
            return self
        new = Qwen35Model(self.model.cfg, dtype=self.model.dtype, device=dev, with_main_grad=False)
        new.flat.flat.copy_(self.model.flat.flat)
        self.model = new
        return self

    def forward(self, prompt_ids, response_ids):
        P, R = prompt_ids.shape[1], response_ids.shape[1]
        ids = torch.cat([prompt_ids, response_ids], dim=1)
        logits = self.model.forward_logits(ids)
        return logits[:, P - 1:P - 1 + R]

    def response_log_probs(self, prompt_ids, response_ids):
        """Fused path: never materialises the logits."""
        ids = torch.cat([prompt_ids, response_ids], dim=1)
        return self.model.response_logprobs(ids, prompt_ids.shape[1])

    def clone_as_reference(self):
        ref = Qwen3_5CausalLmPolicy(self.model.cfg, self.model.dtype, self.model.flat.flat.device, self.model_dir,
                                    self._pad)
        ref.model.flat.flat.copy_(self.model.flat.flat)
        for p in ref.parameters():
            p.requires_grad_(False)
        return ref

    def save_hf_checkpoint(self, out_dir, dtype=None) -> None:
        save_hf_checkpoint(self.model, out_dir, self.model_dir or None, dtype)

    def named_hf_parameters(self):
        """Live tensors under their Hugging Face names (what a weight push to a rollout engine sends)."""
        return list(self.model.local_hf_tensors())


def make_causal_lm_policy(options: CausalLmPolicyOptions) -> CausalLmPolicy:
    if options.kind == "tiny":
        return TinyCausalLmPolicy(options.vocab_size, options.hidden_size, options.pad_id)
    if options.kind in ("qwen3_5", "qwen"):
        if not options.model_dir:
            raise ValueError("qwen3_5 policy requires model_dir")
        return Qwen3_5CausalLmPolicy.from_model_dir(options.model_dir, options.param_dtype, pad_id=options.pad_id,
                                                    max_layers=options.max_layers)
    raise ValueError(f"unknown policy kind {options.kind!r}")
