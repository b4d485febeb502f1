"""Single-device end-to-end GRPO on a prompt/answer JSONL: generate -> reward -> GRPO -> PPO epochs.

``python -m cverl_b200.trainer.gsm8k_grpo --dataset data.jsonl [--policy tiny|qwen --model-dir DIR] ...``

Flow and flags follow the reference executable (tools/rollout/gsm8k_grpo_trainer.cc:233-492): each
step takes ``--prompts`` examples, samples ``--n`` responses per prompt from the current policy,
scores them with the GSM8K rule reward, forms GRPO outcome advantages per prompt group, runs
``--ppo-epochs`` clipped-PPO updates (optionally with a KL term against a frozen reference copy),
and prints one CSV row.  Generation goes through a ``RolloutWorker`` (cached decode for the Qwen
policy; the reference re-runs the full forward per token).  ``grpo_update`` is also what the
serving bridge calls.
"""
from __future__ import annotations

import argparse
import sys
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..data.jsonl import load_prompt_answer_jsonl
from ..models.policy import CausalLmPolicy, CausalLmPolicyOptions, make_causal_lm_policy
from ..ops import rl
from ..optim.adamw import clone_detached, parameter_delta_sum
from ..reward.gsm8k import Gsm8kRewardOptions
from ..rollout.rollout_batch import RolloutBatch, RolloutSample, build_gsm8k_rollout_batch
from ..rollout.worker import GenerationConfig, PolicyRolloutWorker, TokenBatch
from ..text.tokenizer import ByteTokenizer, EncodeOptions, HfBpeTokenizer

CSV_HEADER = "step,rollout,total_seq,mean_reward,success_rate,no_answer,loss,pg_loss,kl_loss,ppo_kl,clipfrac,param_delta,seconds"


@dataclass
class GrpoUpdateConfig:
    ppo_epochs: int = 2
    clip_ratio: float = 0.2
    clip_ratio_c: float = 3.0
    kl_coef: float = 0.0
    kl_penalty: str = "k1"
    epsilon: float = 1e-6
    norm_adv_by_std: bool = True


def grpo_update(policy: CausalLmPolicy, ref_policy: Optional[CausalLmPolicy], optimizer: torch.optim.Optimizer,
                batch: RolloutBatch, cfg: GrpoUpdateConfig) -> Dict[str, float]:
    """GRPO advantages + ``ppo_epochs`` PPO-clip steps on one rollout batch; returns the last epoch's metrics."""
    with torch.no_grad():
        old_lp = policy.response_log_probs(batch.prompt_ids, batch.response_ids).float()
        ref_lp = None
        if ref_policy is not None and cfg.kl_coef != 0.0:
            ref_lp = ref_policy.response_log_probs(batch.prompt_ids, batch.response_ids).float()
        adv, _ = rl.grpo_outcome_advantage(batch.token_rewards, batch.response_mask, batch.group_ids, cfg.epsilon,
                                           cfg.norm_adv_by_std)
    before = clone_detached(list(policy.parameters()))
    out: Dict[str, float] = {}
    for _ in range(cfg.ppo_epochs):
        lp = policy.response_log_probs(batch.prompt_ids, batch.response_ids).float()
        res = rl.ppo_clipped_loss(old_lp, lp, adv, batch.response_mask, cfg.clip_ratio, -1.0, -1.0, cfg.clip_ratio_c,
                                  rl.AGG_TOKEN_MEAN)
        loss = res.pg_loss
        kl_loss = torch.zeros((), device=loss.device)
        if ref_lp is not None:
            kl_loss = rl.masked_mean(rl.kl_penalty(lp, ref_lp, cfg.kl_penalty), batch.response_mask)
            loss = loss + cfg.kl_coef * kl_loss
        optimizer.zero_grad(set_to_none=True)
        loss.backward()
        optimizer.step()
        out = {"loss": loss.item(), "pg_loss": res.pg_loss.item(), "kl_loss": kl_loss.item(),
               "ppo_kl": res.ppo_kl.item(), "clipfrac": res.pg_clipfrac.item()}
    out["param_delta"] = float(parameter_delta_sum(before, list(policy.parameters())))
    return out


def generate_samples(worker, tokenizer, prompts: Sequence[str], n: int, gen_cfg: GenerationConfig,
                     max_prompt_tokens: int, device) -> List[RolloutSample]:
    """Samples ``n`` responses per prompt (batched over all prompts and repeats)."""
    pad = tokenizer.pad_id if tokenizer.pad_id >= 0 else 0
    enc = [tokenizer.encode(p, EncodeOptions())[-max_prompt_tokens:] for p in prompts]
    width = max(1, max(len(e) for e in enc))
    ids = torch.full((len(prompts) * n, width), pad, dtype=torch.long)
    att = torch.zeros_like(ids)
    owner = []
    for i, e in enumerate(enc):
        for r in range(n):
            row = i * n + r
            if e:
                ids[row, width - len(e):] = torch.tensor(e)
                att[row, width - len(e):] = 1
            owner.append(i)
    batch = TokenBatch(ids.to(device), att.to(device), att.sum(-1).to(device))
    out = worker.generate(batch, gen_cfg)
    toks, lens = out.token_ids.cpu(), out.lengths.cpu()
    samples = []
    for row, i in enumerate(owner):
        t = toks[row, :int(lens[row])].tolist()
        samples.append(RolloutSample(i, tokenizer.decode(t), t))
    return samples


def _parse(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--dataset", required=True)
    ap.add_argument("--prompts", type=int, default=4)
    ap.add_argument("--n", type=int, default=4)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--ppo-epochs", type=int, default=2)
    ap.add_argument("--max-prompt-tokens", type=int, default=128)
    ap.add_argument("--max-response-tokens", type=int, default=128)
    ap.add_argument("--hidden-dim", type=int, default=32)
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--clip-ratio", type=float, default=0.2)
    ap.add_argument("--lr", type=float, default=3.0e-3)
    ap.add_argument("--weight-decay", type=float, default=0.0)
    ap.add_argument("--kl-coef", type=float, default=0.0)
    ap.add_argument("--kl-penalty", default="k1", choices=["k1", "abs", "k2", "k3"])
    ap.add_argument("--seed", type=int, default=17)
    ap.add_argument("--reward-method", default="strict", choices=["strict", "flexible"])
    ap.add_argument("--tokenizer", default="byte", choices=["byte", "hf"])
    ap.add_argument("--tokenizer-path", default="")
    ap.add_argument("--policy", default="tiny", choices=["tiny", "qwen"])
    ap.add_argument("--model-dir", default="")
    ap.add_argument("--qwen-max-layers", type=int, default=-1)
    ap.add_argument("--param-dtype", default="float32", choices=["float32", "bfloat16", "float16"])
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--export-dir", default="")
    ap.add_argument("--export-every", type=int, default=0)
    ap.add_argument("--export-dtype", default="bfloat16", choices=["float32", "bfloat16", "float16"])
    a = ap.parse_args(argv)
    if a.policy == "qwen" and not a.model_dir:
        ap.error("--policy qwen requires --model-dir")
    if a.export_every < 0:
        ap.error("--export-every must be >= 0")
    return a


def main(argv=None) -> int:
    a = _parse(argv)
    torch.manual_seed(a.seed)
    device = torch.device(a.device)
    dt = getattr(torch, a.param_dtype)
    if a.tokenizer == "hf":
        tokenizer = HfBpeTokenizer(a.tokenizer_path or (a.model_dir + "/tokenizer.json"))
    else:
        tokenizer = ByteTokenizer()
    examples = load_prompt_answer_jsonl(a.dataset)
    if not examples:
        raise SystemExit("dataset is empty")
    pad = tokenizer.pad_id if tokenizer.pad_id >= 0 else 0
    policy = make_causal_lm_policy(CausalLmPolicyOptions(
        kind="tiny" if a.policy == "tiny" else "qwen3_5", vocab_size=tokenizer.vocab_size, hidden_size=a.hidden_dim,
        pad_id=pad, model_dir=a.model_dir, param_dtype=dt, max_layers=a.qwen_max_layers)).to_device(device)
    ref = policy.clone_as_reference() if a.kl_coef != 0.0 else None
    optimizer = torch.optim.AdamW(policy.parameters(), lr=a.lr, weight_decay=a.weight_decay)
    worker = PolicyRolloutWorker(policy)
    ucfg = GrpoUpdateConfig(ppo_epochs=a.ppo_epochs, clip_ratio=a.clip_ratio, kl_coef=a.kl_coef,
                            kl_penalty=a.kl_penalty)
    ropt = Gsm8kRewardOptions(method=a.reward_method)
    print(CSV_HEADER)
    cursor = 0
    for step in range(1, a.steps + 1):
        t0 = time.time()
        chunk = [examples[(cursor + i) % len(examples)] for i in range(a.prompts)]
        cursor += a.prompts
        prompts, answers = [e.prompt for e in chunk], [e.answer for e in chunk]
        gen_cfg = GenerationConfig(max_new_tokens=min(a.max_tokens, a.max_response_tokens), temperature=a.temperature,
                                   top_p=a.top_p, eos_token_id=tokenizer.eos_id, eos_check_interval=8,
                                   seed=a.seed + step)
        samples = generate_samples(worker, tokenizer, prompts, a.n, gen_cfg, a.max_prompt_tokens, device)
        batch = build_gsm8k_rollout_batch(tokenizer, prompts, answers, samples, a.max_prompt_tokens,
                                          a.max_response_tokens, ropt).to(device)
        m = grpo_update(policy, ref, optimizer, batch, ucfg)
        rewards = batch.rewards.float().cpu()
        no_answer = sum(1 for s in samples if "####" not in s.response_text) / max(1, len(samples))
        print(f"{step},{len(samples)},{len(samples)},{float(rewards.mean()):.6f},"
              f"{float((rewards >= 0.999).float().mean()):.6f},{no_answer:.6f},{m['loss']:.6f},{m['pg_loss']:.6f},"
              f"{m['kl_loss']:.6f},{m['ppo_kl']:.6f},{m['clipfrac']:.6f},{m['param_delta']:.6f},{time.time() - t0:.3f}")
        sys.stdout.flush()
        if a.export_dir and a.export_every and step % a.export_every == 0:
            policy.save_hf_checkpoint(f"{a.export_dir}/step_{step:06d}", getattr(torch, a.export_dtype))
    return 0


if __name__ == "__main__":
    sys.exit(main())
