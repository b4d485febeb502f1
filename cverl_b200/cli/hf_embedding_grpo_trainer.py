"""GRPO on a policy built from a real model's token embedding.

``python -m cverl_b200.cli.hf_embedding_grpo_trainer MODEL_DIR [--steps 8] [--prompts 4] [--responses 4]
[--seq-len 8] [--vocab-subset 64] [--ppo-epochs 2] [--lr 1e-3]``

Loads the first ``--vocab-subset`` rows of the embedding table from a Hugging Face directory with the native
safetensors reader, keeps them frozen as the input encoding, and trains an identity-initialised adapter plus an
LM head initialised to the same rows: ``logits = head(silu(adapter(E[targets]))) / sqrt(hidden)``.  The task is
to reproduce the target ids; one CSV row per step (reference: tools/model/hf_embedding_grpo_trainer.cc).
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from ..models.hf_io import HfModelLoader
from ..trainer.accuracy_grpo import CSV_HEADER, accuracy_grpo_step, csv_row


class EmbeddingPolicy(torch.nn.Module):
    def __init__(self, embedding_subset: torch.Tensor):
        super().__init__()
        v, h = embedding_subset.shape
        self.register_buffer("frozen_embedding", embedding_subset.clone())
        self.adapter = torch.nn.Linear(h, h, bias=False)
        self.lm_head = torch.nn.Linear(h, v, bias=True)
        with torch.no_grad():
            self.adapter.weight.copy_(torch.eye(h))
            self.lm_head.weight.copy_(embedding_subset)
            self.lm_head.bias.zero_()

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        hidden = self.adapter(self.frozen_embedding[token_ids])
        return self.lm_head(torch.nn.functional.silu(hidden)) / math.sqrt(hidden.shape[-1])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("model_dir")
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--prompts", type=int, default=4)
    ap.add_argument("--responses", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=8)
    ap.add_argument("--vocab-subset", type=int, default=64)
    ap.add_argument("--ppo-epochs", type=int, default=2)
    ap.add_argument("--lr", type=float, default=1e-3)
    a = ap.parse_args(argv)
    torch.manual_seed(41)
    loader = HfModelLoader(a.model_dir).load_metadata()
    cfg = loader.config()
    emb = loader.load_tensor(cfg.embed_name).float()
    if not (1 < a.vocab_subset <= emb.shape[0]):
        print("invalid vocab subset size", file=sys.stderr)
        return 2
    policy = EmbeddingPolicy(emb[:a.vocab_subset].contiguous())
    opt = torch.optim.AdamW(policy.parameters(), lr=a.lr)
    print(f"loaded_model={a.model_dir}")
    print(f"model_type={cfg.model_type}")
    print(f"embedding_subset={list(policy.frozen_embedding.shape)}")
    print(CSV_HEADER)
    for step in range(1, a.steps + 1):
        targets = torch.randint(a.vocab_subset, (a.prompts, a.seq_len))
        print(csv_row(accuracy_grpo_step(policy, opt, targets, a.responses, a.ppo_epochs, step)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
