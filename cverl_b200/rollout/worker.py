"""Rollout workers: the generation interface and two native generators.

``RolloutWorker.generate(TokenBatch, GenerationConfig) -> GenerationOutput`` and
``actor_parameters()`` follow include/cverl/rollout/worker.h:14-53.

* ``PolicyRolloutWorker`` generates with any ``CausalLmPolicy`` by re-running the full
  forward over prompt + prefix every step, as the reference does
  (src/rollout/policy_worker.cc:22-135): greedy when temperature <= 0, top-k by masking to
  -inf, top-p by sort + cumulative sum, a per-row finished mask, and a host check only every
  ``eos_check_interval`` steps.
* ``CachedQwenRolloutWorker`` decodes a ``Qwen35Model`` with a KV cache for the full-attention
  layers and the (conv tail, recurrent state) pair for the linear-attention layers, so a new
  token costs one token of compute instead of a re-run of the prefix.
"""
from __future__ import annotations

import abc
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from ..parallel.collectives import Collectives
from ..parallel.weight_sync import ParameterView, broadcast_parameters_from_root, module_parameter_views


@dataclass
class TokenBatch:
    token_ids: torch.Tensor                         # [B, T] left-padded prompts
    attention_mask: Optional[torch.Tensor] = None   # [B, T], optional as in the reference
    lengths: Optional[torch.Tensor] = None          # [B], optional


@dataclass
class GenerationConfig:
    """Defaults are the reference's (include/cverl/rollout/worker.h:20-31): ``top_k <= 0`` keeps every token,
    ``eos_check_interval = 0`` never reads the finished mask on the host inside the loop."""
    max_new_tokens: int = 256
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    eos_token_id: int = -1
    eos_check_interval: int = 0
    seed: int = 0


@dataclass
class GenerationOutput:
    token_ids: torch.Tensor   # [B, N]
    logprobs: torch.Tensor    # [B, N]
    lengths: torch.Tensor     # [B]


class RolloutWorker(abc.ABC):
    @abc.abstractmethod
    def generate(self, batch: TokenBatch, config: GenerationConfig) -> GenerationOutput: ...

    @abc.abstractmethod
    def actor_parameters(self) -> List[ParameterView]: ...


def synchronize_rollout_actor_weights(worker: RolloutWorker, comm: Collectives, trainer_root: int,
                                      group: Optional[Sequence[int]] = None):
    """Broadcast the trainer's weights into the worker's live parameters (src/rollout/worker.cc:5-12)."""
    return broadcast_parameters_from_root(worker.actor_parameters(), comm, trainer_root, group)


def sample_next_tokens(logits: torch.Tensor, cfg: GenerationConfig, gen: Optional[torch.Generator]):
    """logits [B, V] -> (tokens [B], logprobs [B]) under temperature / top-k / top-p sampling."""
    logits = logits.float()
    if cfg.temperature <= 0.0:
        lp = torch.log_softmax(logits, dim=-1)
        tok = lp.argmax(-1)
        return tok, lp.gather(-1, tok.unsqueeze(-1)).squeeze(-1)
    logits = logits / cfg.temperature
    if cfg.top_k and cfg.top_k > 0 and cfg.top_k < logits.shape[-1]:
        kth = logits.topk(cfg.top_k, dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if cfg.top_p < 1.0:
        sorted_logits, idx = logits.sort(dim=-1, descending=True)
        probs = torch.softmax(sorted_logits, dim=-1)
        cum = probs.cumsum(-1)
        drop = (cum - probs) >= cfg.top_p          # keep the smallest prefix whose mass reaches top_p
        sorted_logits = sorted_logits.masked_fill(drop, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, idx, sorted_logits)
    lp = torch.log_softmax(logits, dim=-1)
    tok = torch.multinomial(lp.exp(), 1, generator=gen).squeeze(-1)
    return tok, lp.gather(-1, tok.unsqueeze(-1)).squeeze(-1)


def _generator(device, seed: int) -> Optional[torch.Generator]:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


class PolicyRolloutWorker(RolloutWorker):
    def __init__(self, policy):
        self.policy = policy
        self.forward_calls = 0

    def actor_parameters(self) -> List[ParameterView]:
        return module_parameter_views(self.policy)

    @torch.no_grad()
    def generate(self, batch: TokenBatch, config: GenerationConfig) -> GenerationOutput:
        prompts = batch.token_ids
        B = prompts.shape[0]
        dev = prompts.device
        N = config.max_new_tokens
        pad = self.policy.pad_id
        out = torch.full((B, N), pad, dtype=torch.long, device=dev)
        lps = torch.zeros((B, N), dtype=torch.float32, device=dev)
        lengths = torch.zeros(B, dtype=torch.long, device=dev)
        finished = torch.zeros(B, dtype=torch.bool, device=dev)
        gen = _generator(dev, config.seed)
        for step in range(N):
            # the policy predicts response[:, t] from prompt + response[:, :t]: feed step+1 columns
            logits = self.policy.forward(prompts, out[:, :step + 1])[:, -1]
            self.forward_calls += 1
            tok, lp = sample_next_tokens(logits, config, gen)
            active = ~finished
            out[:, step] = torch.where(active, tok, out[:, step])
            lps[:, step] = torch.where(active, lp, lps[:, step])
            lengths += active.long()
            if config.eos_token_id >= 0:
                finished |= active & (tok == config.eos_token_id)
                if config.eos_check_interval > 0 and (step + 1) % config.eos_check_interval == 0:
                    if bool(finished.all()):   # the only host sync of the loop
                        break
        return GenerationOutput(out, lps, lengths)


class CachedQwenRolloutWorker(RolloutWorker):
    """Cached decode over a ``Qwen35Model`` (see ``cverl_b200.models.decode``)."""

    def __init__(self, model, pad_id: int = 0):
        self.model = model
        self.pad_id = pad_id

    def actor_parameters(self) -> List[ParameterView]:
        return [ParameterView(n, t) for n, t in self.model.flat.named_tensors()]

    @torch.no_grad()
    def generate(self, batch: TokenBatch, config: GenerationConfig) -> GenerationOutput:
        from ..models.decode import DecodeState, decode_step, prefill
        prompts = batch.token_ids
        B = prompts.shape[0]
        dev = prompts.device
        N = config.max_new_tokens
        out = torch.full((B, N), self.pad_id, dtype=torch.long, device=dev)
        lps = torch.zeros((B, N), dtype=torch.float32, device=dev)
        lengths = torch.zeros(B, dtype=torch.long, device=dev)
        finished = torch.zeros(B, dtype=torch.bool, device=dev)
        gen = _generator(dev, config.seed)
        state, logits = prefill(self.model, prompts, max_len=prompts.shape[1] + N)
        graphed = None
        if prompts.is_cuda and N > 4:
            from ..models.decode import GraphedDecoder, native_decode_supported
            if native_decode_supported(self.model):
                graphed = GraphedDecoder(self.model, state, B)     # one CUDA graph replayed per token
        for step in range(N):
            tok, lp = sample_next_tokens(logits, config, gen)
            active = ~finished
            out[:, step] = torch.where(active, tok, out[:, step])
            lps[:, step] = torch.where(active, lp, lps[:, step])
            lengths += active.long()
            if config.eos_token_id >= 0:
                finished |= active & (tok == config.eos_token_id)
                if config.eos_check_interval > 0 and (step + 1) % config.eos_check_interval == 0:
                    if bool(finished.all()):
                        break
            if step + 1 < N:
                logits = graphed.step(tok) if graphed is not None else decode_step(self.model, state, tok)
        return GenerationOutput(out, lps, lengths)
