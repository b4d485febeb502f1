"""Online GRPO loop against an external rollout engine (or an oracle), with rollout dumps for the trainer.

``python -m cverl_b200.cli.online_grpo --model-dir DIR --dataset data.jsonl --rollout oracle --steps 4``
``python -m cverl_b200.cli.online_grpo ... --rollout http --server http://127.0.0.1:8000 --served-model NAME``

Per step: take ``--prompts`` examples, obtain ``--n`` responses per prompt, update the policy through the
bridge (``QwenPolicy.gsm8k_grpo_update``), and optionally

* ``--dump-rollout-dir DIR``: write ``rollout_step_%06d.json`` ({"step", "sequences": [{prompt_ids,
  response_ids, advantage, reward}]}) which the distributed trainer consumes with ``--rollout-dir``
  (``--skip-train`` writes the files without updating, for a static trainer / rollout split);
* ``--push-weights``: after the update, hand the live ``named_parameters()`` and ``update_info()`` to a weight
  sender callback (for vLLM: its NCCL weight-transfer engine; here a hook that records what would be sent).

Rollout sources: ``oracle`` needs no server (it fabricates responses from the gold answers: correct with
probability ``--oracle-accuracy``, otherwise off by one), ``http`` posts to an OpenAI-style ``/v1/completions``
endpoint such as ``vllm serve``.  Reference: tools/rollout/vllm_online_grpo.py.
"""
from __future__ import annotations

import argparse
import json
import random
import sys
import time
import urllib.request
from pathlib import Path
from typing import List, Sequence, Tuple

from ..data.jsonl import load_prompt_answer_jsonl
from ..reward.gsm8k import Gsm8kRewardOptions, compute_gsm8k_reward, normalize_gsm8k_ground_truth


def oracle_rollout(prompts: Sequence[str], answers: Sequence[str], n: int, accuracy: float,
                   rng: random.Random) -> Tuple[List[str], List[int], List[int]]:
    responses, pidx, sidx = [], [], []
    for i, gold in enumerate(answers):
        truth = normalize_gsm8k_ground_truth(gold)
        for s in range(n):
            if rng.random() < accuracy:
                text = f"The answer is #### {truth}"
            else:
                try:
                    text = f"The answer is #### {int(float(truth)) + 1}"
                except ValueError:
                    text = "I do not know"
            responses.append(text)
            pidx.append(i)
            sidx.append(s)
    return responses, pidx, sidx


def http_rollout(server: str, model: str, prompts: Sequence[str], n: int, max_tokens: int, temperature: float,
                 timeout_s: float, top_p: float = 1.0) -> Tuple[List[str], List[int], List[int]]:
    responses, pidx, sidx = [], [], []
    for i, p in enumerate(prompts):
        body = json.dumps({"model": model, "prompt": p, "n": n, "max_tokens": max_tokens,
                           "temperature": temperature, "top_p": top_p}).encode()
        req = urllib.request.Request(server.rstrip("/") + "/v1/completions", data=body,
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=timeout_s) as r:
            out = json.loads(r.read())
        for s, ch in enumerate(out["choices"][:n]):
            responses.append(ch["text"])
            pidx.append(i)
            sidx.append(s)
    return responses, pidx, sidx


def group_advantages(rewards: Sequence[float], pidx: Sequence[int], eps: float = 1e-6) -> List[float]:
    """GRPO outcome advantage per response (group = prompt): (r - mean) / (std + eps), 0 for singletons."""
    by = {}
    for r, i in zip(rewards, pidx):
        by.setdefault(i, []).append(r)
    out = []
    for r, i in zip(rewards, pidx):
        g = by[i]
        if len(g) < 2:
            out.append(0.0)
            continue
        mean = sum(g) / len(g)
        var = sum((x - mean) ** 2 for x in g) / (len(g) - 1)
        out.append((r - mean) / (var ** 0.5 + eps))
    return out


def dump_rollout(path: Path, step: int, tokenizer, prompts, responses, pidx, rewards, advantages,
                 max_prompt_tokens: int, max_response_tokens: int, answers=None, sidx=None) -> None:
    """Writes ``rollout_step_%06d.json`` for the trainer's zero-based ``step``: file number and ``"step"`` field
    are ``step + 1`` (reference: tools/model/qwen3_5_pp_tp_ppo_trainer.cc:745-757,1496-1503).  The file carries
    both the token-id rows this package's trainer reads and the reference's text fields."""
    seqs = []
    for text, i, rew, adv in zip(responses, pidx, rewards, advantages):
        seqs.append({"prompt_index": i, "prompt_ids": tokenizer.encode(prompts[i])[-max_prompt_tokens:],
                     "response_ids": tokenizer.encode(text)[:max_response_tokens], "reward": rew, "advantage": adv,
                     "response_text": text})
    path.mkdir(parents=True, exist_ok=True)
    doc = {"step": step + 1, "sequences": seqs, "prompts": list(prompts), "responses": list(responses),
           "prompt_indices": [int(i) for i in pidx],
           "sample_indices": [int(i) for i in (sidx if sidx is not None else range(len(responses)))]}
    if answers is not None:
        doc["answers"] = list(answers)
    tmp = path / f"rollout_step_{step + 1:06d}.json.tmp"
    tmp.write_text(json.dumps(doc))
    tmp.rename(path / f"rollout_step_{step + 1:06d}.json")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    # Every option of the reference's tool (tools/rollout/vllm_online_grpo.py:190-241) is accepted under its own
    # name; where this tool had another spelling both are kept.
    ap.add_argument("--model-dir", required=True)
    ap.add_argument("--dataset", required=True)
    ap.add_argument("--prompt-field", default="prompt")
    ap.add_argument("--answer-field", default="answer")
    ap.add_argument("--max-examples", type=int, default=-1)
    ap.add_argument("--tokenizer-path", default="")
    ap.add_argument("--rollout", "--rollout-backend", dest="rollout", default="oracle",
                    choices=["oracle", "http", "vllm"], help="vllm = http: an OpenAI-style completions endpoint")
    ap.add_argument("--server", "--base-url", dest="server", default="http://127.0.0.1:8000")
    ap.add_argument("--served-model", "--served-model-name", dest="served_model", default="")
    ap.add_argument("--oracle-accuracy", type=float, default=0.5)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--first-step", type=int, default=0, help="number of the first rollout file / step")
    ap.add_argument("--prompts", type=int, default=4)
    ap.add_argument("--n", type=int, default=4)
    ap.add_argument("--max-tokens", type=int, default=0, help="tokens requested from the engine (0: --max-response-tokens)")
    ap.add_argument("--max-prompt-tokens", type=int, default=128)
    ap.add_argument("--max-response-tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--ppo-epochs", type=int, default=1)
    ap.add_argument("--lr", type=float, default=3e-6)
    ap.add_argument("--weight-decay", type=float, default=0.0)
    ap.add_argument("--clip-ratio", type=float, default=0.2)
    ap.add_argument("--kl-coef", type=float, default=0.0)
    ap.add_argument("--reward-method", choices=["strict", "flexible"], default="flexible")
    ap.add_argument("--measure-param-delta", action="store_true")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--param-dtype", default="float32",
                    choices=["float32", "fp32", "bfloat16", "bf16", "float16", "fp16"])
    ap.add_argument("--max-layers", "--qwen-max-layers", dest="max_layers", type=int, default=-1)
    ap.add_argument("--skip-train", action="store_true")
    ap.add_argument("--dump-rollout-dir", default="")
    ap.add_argument("--push-weights", action="store_true")
    ap.add_argument("--weight-sync", default="none", choices=["none", "nccl"],
                    help="nccl: after every update, push the live weights into the vLLM server at --server "
                         "(pause, update manifest + NCCL transfer, resume)")
    ap.add_argument("--no-weight-sync", action="store_true", help="overrides --weight-sync")
    ap.add_argument("--sync-every", type=int, default=1, help="push the weights after every k-th update")
    ap.add_argument("--sync-initial", action="store_true", help="push the weights once before the first rollout")
    ap.add_argument("--weight-master-address", "--master-address", dest="weight_master_address", default="127.0.0.1")
    ap.add_argument("--weight-master-port", "--master-port", dest="weight_master_port", type=int, default=0)
    ap.add_argument("--weight-world-size", "--world-size", dest="weight_world_size", type=int, default=0,
                    help="trainer rank + all vLLM worker ranks")
    ap.add_argument("--weight-rank-offset", "--rank-offset", dest="weight_rank_offset", type=int, default=1)
    ap.add_argument("--packed", action=argparse.BooleanOptionalAction, default=True)
    ap.add_argument("--packed-buffer-size-bytes", type=int, default=1 << 30)
    ap.add_argument("--packed-num-buffers", type=int, default=2)
    ap.add_argument("--checkpoint-format", action=argparse.BooleanOptionalAction, default=True,
                    help="send Hugging Face checkpoint names and let the server map them onto its own parameters")
    ap.add_argument("--sleep-during-train", "--sleep-vllm-for-train", dest="sleep_during_train", action="store_true",
                    help="put the server to sleep while the actor update runs and wake it before the sync")
    ap.add_argument("--vllm-sleep-level", type=int, default=1)
    ap.add_argument("--vllm-sleep-mode", choices=["abort", "wait", "keep"], default="wait")
    ap.add_argument("--http-timeout", "--timeout", dest="http_timeout", type=float, default=120.0)
    ap.add_argument("--seed", type=int, default=17)
    a = ap.parse_args(argv)
    from ..rollout.vllm_bridge import QwenPolicy
    if a.rollout == "vllm":
        a.rollout = "http"
    if a.no_weight_sync:
        a.weight_sync = "none"
    a.param_dtype = {"fp32": "float32", "bf16": "bfloat16", "fp16": "float16"}.get(a.param_dtype, a.param_dtype)
    rng = random.Random(a.seed)
    examples = load_prompt_answer_jsonl(a.dataset, a.prompt_field, a.answer_field, a.max_examples)
    if not examples:
        raise SystemExit("dataset is empty")
    policy = QwenPolicy(a.model_dir, tokenizer_path=a.tokenizer_path, device=a.device, param_dtype=a.param_dtype,
                        max_layers=a.max_layers)
    ropt = Gsm8kRewardOptions(method=a.reward_method)
    sync = control = None
    if a.weight_sync == "nccl" or a.sleep_during_train:
        from ..rollout.vllm_control import VllmControl, VllmNcclSync
        control = VllmControl(a.server, a.http_timeout)
        if a.weight_sync == "nccl":
            if a.weight_master_port <= 0 or a.weight_world_size <= 1:
                raise SystemExit("--weight-sync nccl needs --weight-master-port and --weight-world-size >= 2")
            sync = VllmNcclSync(control, a.weight_master_address, a.weight_master_port, a.weight_world_size,
                                a.weight_rank_offset, packed=a.packed,
                                packed_buffer_size_bytes=a.packed_buffer_size_bytes,
                                packed_num_buffers=a.packed_num_buffers, checkpoint_format=a.checkpoint_format)

    def update_info():
        info = policy.update_info(a.packed, a.packed_buffer_size_bytes, a.packed_num_buffers)
        info["is_checkpoint_format"] = bool(a.checkpoint_format)
        return info

    def push() -> int:
        if sync is not None:
            return sync.sync(policy.named_parameters(), update_info())["bytes"]
        if a.push_weights:
            info = update_info()
            assert len(info["names"]) == len(policy.named_parameters())
            return sum(t.numel() * t.element_size() for _, t in policy.named_parameters())
        return 0
    if a.sync_initial:
        push()
    cursor = 0
    for step in range(a.first_step, a.first_step + a.steps):
        t0 = time.time()
        chunk = [examples[(cursor + i) % len(examples)] for i in range(a.prompts)]
        cursor += a.prompts
        prompts, answers = [e.prompt for e in chunk], [e.answer for e in chunk]
        if a.rollout == "oracle":
            responses, pidx, sidx = oracle_rollout(prompts, answers, a.n, a.oracle_accuracy, rng)
        else:
            responses, pidx, sidx = http_rollout(a.server, a.served_model or a.model_dir, prompts, a.n,
                                                 a.max_tokens or a.max_response_tokens, a.temperature, a.http_timeout,
                                                 a.top_p)
        rewards = [compute_gsm8k_reward(r, answers[i], ropt) for r, i in zip(responses, pidx)]
        if a.dump_rollout_dir:
            dump_rollout(Path(a.dump_rollout_dir), step, policy.tokenizer, prompts, responses, pidx, rewards,
                         group_advantages(rewards, pidx), a.max_prompt_tokens, a.max_response_tokens, answers, sidx)
        metrics = {"total_seq": float(len(responses)), "mean_reward": sum(rewards) / max(1, len(rewards))}
        if a.sleep_during_train and control is not None and not a.skip_train:
            control.sleep(a.vllm_sleep_level, a.vllm_sleep_mode)
        if not a.skip_train:
            metrics = policy.gsm8k_grpo_update(prompts, responses, answers, pidx, sidx, a.max_prompt_tokens,
                                               a.max_response_tokens, a.ppo_epochs, a.lr, a.weight_decay,
                                               a.clip_ratio, a.kl_coef, a.reward_method, True)
        if a.sleep_during_train and control is not None and not a.skip_train:
            control.wake()
        pushed = 0
        if not a.skip_train and (step - a.first_step + 1) % max(a.sync_every, 1) == 0:
            pushed = push()
        print(json.dumps({"step": step, "seconds": round(time.time() - t0, 3), "pushed_bytes": pushed,
                          **{k: round(v, 6) for k, v in metrics.items()}}), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
