"""Distributed PPO / GRPO / SFT trainer for Qwen3.5 and Qwen3-MoE over DP x PP x CP x TP x EP.

One process per GPU (``torchrun`` or any launcher that sets RANK / WORLD_SIZE / LOCAL_RANK):

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m cverl_b200.trainer.ppo_trainer --config qwen3_5_0_8b --dp 4 --tp 2 --steps 5

The step is the reference trainer's (tools/model/qwen3_5_pp_tp_ppo_trainer.cc:2200-2742): barrier and
device sync, batch acquisition, micro-batches in 1F1B order (one sequence group per micro-batch), PPO
clipped loss (+ KL) or SFT NLL divided by micro_batches * grad_accum_steps, CP / TP-replicated gradient
sync, the optimizer step, ``step_time_s`` as the max over ranks, the step metrics all-gathered over the world,
one ``key=value`` line and a CSV row on rank 0, rank-local checkpoints with a manifest, and an exit code
that reflects ``all_ranks_have_grad`` / ``all_ranks_updated``.

Optimizer modes (reference flags, trainer.cc:1877-1879): ``--dp-shard-optimizer true
--dp-flat-shard-optimizer true`` (the default HERE; the reference defaults to the unsharded mode) is the flat
ZeRO shard with FlatAdamW; ``--dp-shard-optimizer true --dp-flat-shard-optimizer false`` is ZeRO-1 with one
owner rank per parameter and owner broadcasts; ``--dp-shard-optimizer false`` is the bucketed data-parallel
all-reduce with per-tensor ``Fp32MasterAdamW`` on every rank.

Batch sources, first match wins (trainer.cc:2226-2262): SFT JSONL, a rollout rank sending ``GpuRolloutBatch``
over a communicator of its own (``--rollout-nccl-*``), CUDA-IPC manifests (``--rollout-ipc-json`` /
``--rollout-ipc-dir``), rollout JSON files (``--rollout-json`` / ``--rollout-dir``), synthetic rows.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Optional

import torch

from .. import _native
from ..models.config import Qwen35TextConfig
from ..models.hf_io import HfModelLoader, load_model_weights
from ..models.qwen3_5 import Qwen35Model
from ..ops import rl
from ..optim import AdamWOptions
from ..parallel.mesh import build_context
from ..parallel.pipeline import PipelineStage, pipeline_peers
from ..parallel.dp_sync import TensorwiseOptimizer
from ..parallel.zero import FlatZeroOptimizer
from ..utils import checkpoint as ckpt
from ..utils import fallbacks as _fallbacks
from ..utils.metrics import MetricsCsv, format_line
from ..utils.watchdog import Heartbeat, PeerFailure, Watchdog
from ..utils.fault_injection import HostFault
from .actor import ActorConfig, ActorEngine

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "float16": torch.float16}


def _flag(v) -> bool:
    """Boolean flag values as the reference's launch scripts pass them (``--master-weights false``)."""
    if isinstance(v, bool):
        return v
    low = str(v).strip().lower()
    if low in ("1", "true", "yes", "on"):
        return True
    if low in ("0", "false", "no", "off", ""):
        return False
    raise argparse.ArgumentTypeError(f"expected true or false, got {v!r}")


def _add_flag(g, *names, default=False, help=None):
    g.add_argument(*names, nargs="?", const=True, default=default, type=_flag, help=help)


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    g = ap.add_argument_group("model")
    g.add_argument("model_dir_positional", nargs="?", default="", help="model directory (the reference's argv[1])")
    g.add_argument("--model-dir", default="")
    g.add_argument("--config", default="tiny", help="built-in shape when no --model-dir: qwen3_5_0_8b, qwen3_30b_a3b, tiny, tiny_moe")
    g.add_argument("--max-layers", "--layers", type=int, default=-1)
    g.add_argument("--dtype", default="bfloat16")
    g = ap.add_argument_group("parallelism")
    for name in ("dp", "pp", "cp", "tp", "ep", "sp"):
        g.add_argument(f"--{name}", f"--{name}-size", type=int, default=1)
    g.add_argument("--global-rank", type=int, default=-1, help="overrides RANK (the reference's launcher passes it)")
    g.add_argument("--device", type=int, default=-1, help="overrides LOCAL_RANK")
    g.add_argument("--micro-batches", type=int, default=1)
    g.add_argument("--micro-batch-seqs", type=int, default=1, help="sequences per micro-batch (the reference uses 1)")
    g.add_argument("--grad-accum-steps", type=int, default=1)
    g.add_argument("--backend", default="auto", choices=["auto", "nccl", "gloo"])
    g = ap.add_argument_group("data")
    g.add_argument("--prompt-len", type=int, default=8)
    g.add_argument("--response-len", type=int, default=8)
    g.add_argument("--rows", type=int, default=64, help="rows of the synthetic batch table")
    g.add_argument("--sft-jsonl", "--jsonl-input", default="")
    g.add_argument("--jsonl-max-examples", type=int, default=0, help="0 = --rows")
    g.add_argument("--rollout-json", default="", help="one rollout JSON file used at every step")
    g.add_argument("--rollout-dir", default="", help="directory of rollout_step_%%06d.json files (1-based step)")
    g.add_argument("--rollout-ipc-json", default="", help="one CUDA-IPC batch manifest used at every step")
    g.add_argument("--rollout-ipc-dir", default="", help="directory of rollout_ipc_step_%%06d.json manifests")
    g.add_argument("--rollout-nccl-id-file", default="",
                   help="rendezvous file of the rollout-data communicator (rollout ranks + trainer ranks)")
    g.add_argument("--rollout-nccl-world-size", type=int, default=0)
    g.add_argument("--rollout-nccl-rank-offset", type=int, default=0)
    g.add_argument("--rollout-nccl-source-rank", type=int, default=0)
    g.add_argument("--tokenizer-json", default="")
    _add_flag(g, "--vary-tokens-by-step", default=True,
              help="synthetic rows advance with the step (false: the same rows every step)")
    g = ap.add_argument_group("algorithm")
    g.add_argument("--mode", "--train-mode", default="ppo", choices=["ppo", "sft"])
    g.add_argument("--steps", type=int, default=2)
    g.add_argument("--lr", type=float, default=1e-8)
    g.add_argument("--weight-decay", type=float, default=0.01)
    g.add_argument("--clip-ratio", type=float, default=0.2)
    g.add_argument("--clip-ratio-c", type=float, default=3.0)
    g.add_argument("--kl-coef", type=float, default=0.0)
    g.add_argument("--kl-penalty", default="k1")
    g.add_argument("--advantage-scale", type=float, default=1.0)
    g.add_argument("--max-grad-norm", type=float, default=1.0)
    g.add_argument("--zero-stage", type=int, default=1, choices=[1, 2],
                   help="2: per-layer gradient buckets on rotating buffers, reduce-scattered from inside the backward "
                        "pass on a side stream (no full fp32 gradient copy; flat mode, --tp 1 --pp 1 --cp 1 --ep 1)")
    _add_flag(g, "--activation-checkpointing",
              help="keep only each layer's input for the backward pass and run the layer again there")
    g.add_argument("--zero-grad-slots", type=int, default=2, help="gradient bucket buffers in flight for --zero-stage 2")
    g.add_argument("--zero-comm", default="nccl", choices=["nccl", "symm"],
                   help="ZeRO gradient reduce-scatter / parameter all-gather: library collectives, or this "
                        "package's kernels over peer-mapped memory (CUDA, bf16 parameters, same node)")
    g.add_argument("--tp-comm", default="nccl", choices=["nccl", "symm", "sp"],
                   help="tensor-parallel communication: NCCL all-reduces; symm = all-reduce fused into the GEMM "
                        "epilogue over peer-mapped memory; sp = token-sharded residual stream with the "
                        "reduce-scatter in the GEMM epilogue and the all-gather in the norm kernels (dense models, "
                        "--pp 1 --cp 1, tokens per micro-batch a multiple of 128 * tp)")
    g.add_argument("--ep-comm", default="nccl", choices=["nccl", "symm"],
                   help="expert-parallel dispatch / combine: NCCL all-to-all, or row scatter / gather kernels over "
                        "peer-mapped memory (no host read)")
    g.add_argument("--cp-comm", default="nccl", choices=["nccl", "symm"],
                   help="context-parallel attention: ring send/recv, or K / V pulled from the owners by the kernels")
    g.add_argument("--cp-attn", default="zigzag", choices=["zigzag", "ring"],
                   help="context-parallel attention: zigzag = q | k | v resharded so that every rank does the same "
                        "causal work (with --cp-comm nccl); ring = contiguous shards")
    g.add_argument("--ep-capacity-factor", type=float, default=2.0,
                   help="receive-buffer rows per rank for --ep-comm symm, as a multiple of the balanced load")
    _add_flag(g, "--master-weights")
    _add_flag(g, "--dp-shard-optimizer", default=True,
              help="shard optimizer state over the data-parallel group (false: every rank keeps all of it)")
    _add_flag(g, "--dp-flat-shard-optimizer", default=True,
              help="with --dp-shard-optimizer: flat ZeRO shard (true) or one owner rank per parameter (false)")
    _add_flag(g, "--skip-optimizer-step")
    _add_flag(g, "--measure-param-delta",
              help="clone the parameters before the step and report sum |delta| (costs a copy per step)")
    _add_flag(g, "--nccl-sync-after-collective", help="accepted for launcher compatibility; collectives here "
                                                         "are stream-ordered")
    g.add_argument("--dp-grad-comm-dtype", default="float32")
    g.add_argument("--tp-grad-comm-dtype", default="model")
    g.add_argument("--dp-grad-bucket-mb", type=int, default=25)
    g.add_argument("--tp-grad-bucket-mb", type=int, default=25)
    g.add_argument("--id-prefix", default="", help="accepted for launcher compatibility (rendezvous is torchrun's)")
    g.add_argument("--seed", type=int, default=1234)
    g = ap.add_argument_group("output")
    g.add_argument("--metrics-csv", default="")
    g.add_argument("--checkpoint-dir", default="")
    g.add_argument("--checkpoint-every", type=int, default=0)
    _add_flag(g, "--flat-checkpoint-save-model-params")
    g.add_argument("--resume-checkpoint", default="")
    g.add_argument("--heartbeat-timeout-s", type=float, default=0.0, help="> 0 enables the peer watchdog")
    return ap


def _builtin_config(name: str) -> Qwen35TextConfig:
    return {"qwen3_5_0_8b": Qwen35TextConfig.qwen3_5_0_8b, "qwen3_30b_a3b": Qwen35TextConfig.qwen3_30b_a3b,
            "tiny": lambda: Qwen35TextConfig.tiny(False), "tiny_moe": lambda: Qwen35TextConfig.tiny(True)}[name]()


def synthetic_token_row(row: int, seq_len: int, vocab: int, device) -> torch.Tensor:
    """``ids = (arange(1..S) + offset) mod (V-1)``, clamped to >= 1 (reference: trainer.cc:1833-1835)."""
    ids = (torch.arange(1, seq_len + 1, device=device) + row * 17) % (vocab - 1)
    return ids.clamp_min(1)


def batch_row_index(step, accum, accum_steps, m, micro_batches, dp, ep, dp_rank, ep_rank, rows) -> int:
    """Reference batch indexing (trainer.cc:2276-2278,2321)."""
    return (((step * accum_steps + accum) * micro_batches + m) * dp * ep + dp_rank * ep + ep_rank) % rows


@dataclass
class StepBatch:
    """One step's rollout rows as device tensors, plus the three reward metrics of the log line."""
    prompt_ids: torch.Tensor                     # [rows, P] int64
    response_ids: torch.Tensor                   # [rows, R] int64
    response_mask: torch.Tensor                  # [rows, R] float32
    advantages: Optional[torch.Tensor] = None    # [rows, R] float32
    old_log_probs: Optional[torch.Tensor] = None
    ref_log_probs: Optional[torch.Tensor] = None
    mean_reward: float = 0.0
    success_rate: float = 0.0
    adv_abs_sum: float = 0.0

    @property
    def rows(self) -> int:
        return self.prompt_ids.shape[0]

    def set_metrics(self, rewards: Optional[torch.Tensor], threshold: float = 1.0 - 1e-6) -> "StepBatch":
        """mean reward, share of rewards >= ``threshold``, sum |advantage| (reference: trainer.cc:624-649);
        one small device->host copy per step, outside the micro-batch loop."""
        if self.advantages is None:
            return self
        parts = [self.advantages.float().abs().sum()]
        if rewards is not None and rewards.numel() > 0:
            r = rewards.to(self.advantages.device).float()
            parts += [r.mean(), (r >= threshold).float().mean()]
        host = torch.stack(parts).cpu()
        self.adv_abs_sum = float(host[0])
        if len(parts) == 3:
            self.mean_reward, self.success_rate = float(host[1]), float(host[2])
        return self


def _fit(t: torch.Tensor, length: int, pad, left: bool) -> torch.Tensor:
    """[rows, n] -> [rows, length]: truncated (keeping the tail when ``left``) or padded with ``pad``."""
    n = t.shape[1]
    if n == length:
        return t
    if n > length:
        return t[:, n - length:] if left else t[:, :length]
    filler = torch.full((t.shape[0], length - n), pad, dtype=t.dtype, device=t.device)
    return torch.cat([filler, t], 1) if left else torch.cat([t, filler], 1)


def step_batch_from_tensors(tensors: Dict[str, torch.Tensor], prompt_len: int, response_len: int, device,
                            exact: bool = True) -> StepBatch:
    """A received ``GpuRolloutBatch`` / IPC batch as a ``StepBatch`` (reference: trainer.cc:1674-1701).
    Advantages come with the batch, or are formed here as GRPO outcome advantages from rewards and group ids."""
    for need in ("prompt_ids", "response_ids", "response_mask"):
        if need not in tensors:
            raise RuntimeError(f"rollout batch is missing required tensor '{need}'")
    p, r = tensors["prompt_ids"].to(device), tensors["response_ids"].to(device)
    if exact and (p.shape[1] != prompt_len or r.shape[1] != response_len):
        raise RuntimeError("rollout batch prompt/response length mismatch")
    mask = tensors["response_mask"].to(device).float()
    adv = tensors.get("advantages")
    rewards = tensors.get("rewards")
    if adv is None:
        if rewards is None or "group_ids" not in tensors:
            raise RuntimeError("rollout batch carries neither advantages nor rewards + group ids")
        tr = torch.zeros_like(mask)
        last = (mask.sum(-1).long() - 1).clamp_min(0)
        tr[torch.arange(mask.shape[0], device=mask.device), last] = rewards.to(device).float()
        adv, _ = rl.grpo_outcome_advantage(tr, mask, tensors["group_ids"].to(device), 1e-6, True)
    adv = adv.to(device).float()
    if adv.dim() == 1:
        adv = adv.unsqueeze(1) * mask

    def opt(name):
        t = tensors.get(name)
        return None if t is None else t.to(device).float().contiguous()
    sb = StepBatch(_fit(p, prompt_len, 0, True).contiguous(), _fit(r, response_len, 0, False).contiguous(),
                   _fit(mask, response_len, 0.0, False).contiguous(), _fit(adv, response_len, 0.0, False).contiguous(),
                   opt("old_log_probs"), opt("ref_log_probs"))
    return sb.set_metrics(rewards)


class BatchSource:
    """The step's batch: SFT examples, a rollout rank over its own communicator, CUDA-IPC manifests, rollout
    JSON files, or synthetic rows - in that order of precedence (reference: trainer.cc:2226-2262)."""

    def __init__(self, args, cfg: Qwen35TextConfig, device, global_rank: int = 0, needs_batch: bool = True):
        self.args, self.cfg, self.device = args, cfg, device
        self.S = args.prompt_len + args.response_len
        self.sft = None
        self.needs_batch = needs_batch
        self._tok = None
        self.rollout_comm = None
        if args.rollout_nccl_id_file and args.mode != "sft":
            from ..parallel.file_rendezvous import FileRendezvousCollectives
            world = int(os.environ.get("WORLD_SIZE", "1"))
            if args.rollout_nccl_world_size <= world:
                raise SystemExit("rollout communicator must hold the rollout ranks plus every trainer rank")
            data_rank = args.rollout_nccl_rank_offset + global_rank
            if not (0 <= data_rank < args.rollout_nccl_world_size):
                raise SystemExit("rollout communicator rank out of range")
            self.rollout_comm = FileRendezvousCollectives(args.rollout_nccl_id_file, data_rank,
                                                          args.rollout_nccl_world_size, device)
        if args.sft_jsonl:
            from ..data import load_prompt_answer_jsonl
            tok = self.tokenizer()
            self.sft = []
            limit = args.jsonl_max_examples or args.rows
            for ex in load_prompt_answer_jsonl(args.sft_jsonl, max_examples=limit):
                p = tok.encode(ex.prompt)[-args.prompt_len:]
                r = tok.encode(ex.answer)[:args.response_len]
                ids = torch.full((self.S,), max(tok.pad_id, 0), dtype=torch.long)
                ids[args.prompt_len - len(p):args.prompt_len] = torch.tensor(p, dtype=torch.long) % cfg.vocab_size
                ids[args.prompt_len:args.prompt_len + len(r)] = torch.tensor(r, dtype=torch.long) % cfg.vocab_size
                mask = torch.zeros(args.response_len)
                mask[:len(r)] = 1.0
                self.sft.append((ids, mask))
            if not self.sft:
                raise ValueError("--sft-jsonl has no rows")

    def tokenizer(self):
        if self._tok is None:
            from ..text import ByteTokenizer, HfBpeTokenizer
            self._tok = HfBpeTokenizer(self.args.tokenizer_json) if self.args.tokenizer_json else ByteTokenizer()
        return self._tok

    # ---- per-step acquisition ---------------------------------------------------------------------------
    def _path(self, single: str, directory: str, pattern: str, step: int) -> str:
        if single:
            return single
        if not directory:
            return ""
        return str(Path(directory) / (pattern % (step + 1)))

    def acquire(self, step: int) -> Optional[StepBatch]:
        a = self.args
        if a.mode == "sft":
            return None
        if self.rollout_comm is not None:
            sb = None
            if self.needs_batch:        # first and last pipeline stage score / embed; middle stages only relay
                from ..rollout.gpu_batch_transport import GpuBatchReceiver
                b = GpuBatchReceiver(self.rollout_comm, self.device).recv(a.rollout_nccl_source_rank)
                if b.step != step + 1:
                    raise RuntimeError(f"rollout NCCL batch step mismatch: got {b.step}, expected {step + 1}")
                sb = step_batch_from_tensors(b.tensors, a.prompt_len, a.response_len, self.device)
            self.rollout_comm.barrier()
            return sb
        ipc = self._path(a.rollout_ipc_json, a.rollout_ipc_dir, "rollout_ipc_step_%06d.json", step)
        if ipc:
            return self._from_ipc(ipc, step)
        js = self._path(a.rollout_json, a.rollout_dir, "rollout_step_%06d.json", step)
        if js:
            return self._from_json(js, step)
        return None

    def _from_ipc(self, path: str, step: int) -> StepBatch:
        """A manifest of CUDA-IPC handles written by a rollout process on the same node (reference:
        trainer.cc:1570-1672): ``{"step": n, "tensors": [handle...]}``."""
        from ..rollout.gpu_ipc import import_batch
        text = Path(path).read_text()
        doc = json.loads(text)
        if "step" in doc and int(doc["step"]) != step + 1:
            raise RuntimeError(f"rollout IPC batch step mismatch for {path}: expected {step + 1}, got {doc['step']}")
        tensors = import_batch(text)
        # clone: the exporting process may reuse its buffers for the next step
        return step_batch_from_tensors({k: v.clone() for k, v in tensors.items()}, self.args.prompt_len,
                                       self.args.response_len, self.device)

    def _from_json(self, path: str, step: int) -> StepBatch:
        a = self.args
        if not Path(path).exists():
            raise FileNotFoundError(f"rollout file for step {step} not found: {path}")
        doc = json.loads(Path(path).read_text())
        if "step" in doc and int(doc["step"]) != step + 1:
            raise RuntimeError(f"rollout batch step mismatch for {path}: expected {step + 1}, got {doc['step']}")
        if "sequences" in doc:                 # token-id form written by cverl_b200.cli.online_grpo
            seqs = doc["sequences"]
            n = len(seqs)
            P, R = a.prompt_len, a.response_len
            prompt = torch.ones(n, P, dtype=torch.long)
            resp = torch.ones(n, R, dtype=torch.long)
            mask = torch.zeros(n, R)
            adv = torch.zeros(n, R)
            old = torch.zeros(n, R)
            ref = torch.zeros(n, R)
            have_old = all("old_log_probs" in s for s in seqs)
            have_ref = all("ref_log_probs" in s for s in seqs)
            rewards = torch.tensor([float(s.get("reward", 0.0)) for s in seqs])
            for i, s in enumerate(seqs):
                p = s["prompt_ids"][-P:]
                if p:
                    prompt[i, P - len(p):] = torch.tensor(p, dtype=torch.long) % self.cfg.vocab_size
                r = s["response_ids"][:R]
                k = len(r)
                if k:
                    resp[i, :k] = torch.tensor(r, dtype=torch.long) % self.cfg.vocab_size
                mask[i, :k] = 1.0
                adv[i, :k] = float(s.get("advantage", a.advantage_scale))
                if have_old:
                    old[i, :k] = torch.tensor(s["old_log_probs"][:k])
                if have_ref:
                    ref[i, :k] = torch.tensor(s["ref_log_probs"][:k])
            t = {"prompt_ids": prompt, "response_ids": resp, "response_mask": mask, "advantages": adv}
            if have_old:
                t["old_log_probs"] = old
            if have_ref:
                t["ref_log_probs"] = ref
            if any("reward" in s for s in seqs):
                t["rewards"] = rewards
            return step_batch_from_tensors(t, P, R, self.device)
        # text form written by the reference's online loop (trainer.cc:1485-1552): prompts, answers, responses
        # with prompt / sample indices; tokenised, scored with the GSM8K rule and turned into GRPO advantages here
        from ..reward.gsm8k import Gsm8kRewardOptions
        from ..rollout.rollout_batch import RolloutSample, build_gsm8k_rollout_batch
        responses, pidx = doc["responses"], doc["prompt_indices"]
        if len(responses) != len(pidx) or len(responses) != len(doc.get("sample_indices", pidx)):
            raise RuntimeError(f"rollout JSON response/index size mismatch: {path}")
        samples = [RolloutSample(int(pi), txt) for pi, txt in zip(pidx, responses)]
        rb = build_gsm8k_rollout_batch(self.tokenizer(), doc["prompts"], doc["answers"], samples, a.prompt_len,
                                       a.response_len, Gsm8kRewardOptions(method="flexible"))
        t = {"prompt_ids": rb.prompt_ids % self.cfg.vocab_size, "response_ids": rb.response_ids % self.cfg.vocab_size,
             "response_mask": rb.response_mask, "rewards": rb.rewards, "group_ids": rb.group_ids}
        return step_batch_from_tensors(t, a.prompt_len, a.response_len, self.device)

    # ---- micro-batches --------------------------------------------------------------------------------------
    def micro_batch(self, rows: List[int], rollout: Optional[StepBatch]) -> Dict[str, torch.Tensor]:
        a, dev = self.args, self.device
        if rollout is not None:
            idx = torch.tensor([r % rollout.rows for r in rows], dtype=torch.long, device=rollout.prompt_ids.device)
            out = {"input_ids": torch.cat([rollout.prompt_ids[idx], rollout.response_ids[idx]], 1),
                   "response_mask": rollout.response_mask[idx]}
            for k in ("advantages", "old_log_probs", "ref_log_probs"):
                t = getattr(rollout, k)
                if t is not None:
                    out[k] = t[idx]
            return out
        ids, masks = [], []
        for row in rows:
            if self.sft is not None:
                t, m = self.sft[row % len(self.sft)]
                ids.append(t)
                masks.append(m)
            else:
                ids.append(synthetic_token_row(row, self.S, self.cfg.vocab_size, "cpu"))
                masks.append(torch.ones(a.response_len))
        return {"input_ids": torch.stack(ids).to(dev), "response_mask": torch.stack(masks).to(dev)}


def _score(ecfg: ActorConfig, lp: torch.Tensor, batch: Dict[str, torch.Tensor], grad_scale: float):
    """Loss of one micro-batch from its response log-probs: returns (gradient seed d loss / d log-prob,
    metrics[6] = pg_loss | nll, clipfrac, ppo_kl, clipfrac_lower, kl_loss, tokens)."""
    mask = batch["response_mask"]
    if ecfg.mode == "sft":
        denom = mask.sum() + rl.EPS
        seed = (-mask / denom) * grad_scale
        nll = -(lp.detach() * mask).sum() / denom
        z = nll.new_zeros(())
        return seed, torch.stack([nll, z, z, z, z, mask.sum()])
    adv = batch.get("advantages")
    adv = adv if adv is not None else torch.full_like(lp, ecfg.advantage_scale).detach()
    old = batch.get("old_log_probs")
    old = old if old is not None else lp.detach()
    ref = None
    if ecfg.kl_coef > 0.0:
        ref = batch.get("ref_log_probs")
        if ref is None:
            raise RuntimeError("--kl-coef > 0 requires ref_log_probs in the rollout batch")
    metrics, seed = rl.actor_loss(old, lp.detach(), adv, mask, ref, clip_ratio=ecfg.clip_ratio,
                                  clip_ratio_c=ecfg.clip_ratio_c, kl_coef=ecfg.kl_coef,
                                  kl_penalty_kind=ecfg.kl_penalty, loss_scale=grad_scale)
    return seed.to(lp.dtype), metrics


def _loss_and_seed(model, engine_cfg: ActorConfig, hidden, batch, prompt_len, grad_scale):
    """Last-stage scoring of one micro-batch: returns (log-probs, gradient seed, metrics[6])."""
    B, S = batch["input_ids"].shape
    R = S - prompt_len
    if model.ctx.cp_size > 1:          # the stage holds this context-parallel rank's shard of every sequence
        lp = model.cp_response_logprobs(hidden, batch["input_ids"], prompt_len)
    else:
        h = hidden.view(B, S, -1)[:, prompt_len - 1:prompt_len - 1 + R]
        lp = model.token_logprobs(h, batch["input_ids"][:, prompt_len:])
    seed, metrics = _score(engine_cfg, lp, batch, grad_scale)
    return lp, seed, metrics


def run(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.model_dir_positional and not args.model_dir:
        args.model_dir = args.model_dir_positional
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = args.global_rank if args.global_rank >= 0 else int(os.environ.get("RANK", "0"))
    local_rank = args.device if args.device >= 0 else int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available() and args.backend != "gloo"
    device = torch.device("cuda", local_rank) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    import torch.distributed as dist
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if use_cuda else "gloo")
    if args.dp * args.pp * args.cp * args.tp * args.ep != world:
        raise SystemExit(f"world size {world} != dp*pp*cp*tp*ep")
    if args.cp > 1 and args.tp > 1:
        # The reference refuses this pair (trainer.cc:1931-1933).  Here the ring exchanges K | V of the local heads,
        # the state hand-off carries the local heads' states, and the row-parallel sums run inside each context
        # shard; the tensor-parallel exchanges stay on the collective path (the peer-memory forms size their
        # buffers for an unsharded sequence).
        if args.tp_comm != "nccl" and rank == 0:
            print("note: --cp > 1 with --tp > 1 uses --tp-comm nccl", flush=True)
        args.tp_comm = "nccl"
    if args.sp != 1:
        raise SystemExit("sequence parallelism (--sp) is declared in the topology but is not a trainer mode")
    if args.mode == "sft" and not args.sft_jsonl:
        raise SystemExit("--train-mode sft requires --jsonl-input")
    if args.mode == "sft" and (args.rollout_json or args.rollout_dir or args.rollout_ipc_json or args.rollout_ipc_dir
                               or args.rollout_nccl_id_file):
        raise SystemExit("--train-mode sft consumes jsonl gold answers and cannot also consume rollout batches")
    if args.kl_coef < 0 or args.dp_grad_bucket_mb <= 0 or args.tp_grad_bucket_mb <= 0:
        raise SystemExit("--kl-coef must be non-negative and the bucket sizes positive")
    opt_mode = "flat" if (args.dp_shard_optimizer and args.dp_flat_shard_optimizer) else (
        "zero1" if args.dp_shard_optimizer else "dense")
    torch.manual_seed(args.seed + rank)
    dtype = _DTYPES[args.dtype]

    ctx = build_context(world, rank, tp=args.tp, dp=args.dp, pp=args.pp, cp=args.cp, ep=args.ep,
                        micro_batches=max(args.micro_batches, args.pp))
    topo, info = ctx.topology, ctx.rank_info
    if args.model_dir:
        loader = HfModelLoader(args.model_dir).load_metadata()
        cfg = loader.config()
    else:
        loader, cfg = None, _builtin_config(args.config)
    if args.max_layers > 0:
        cfg = Qwen35TextConfig(**{**{k: getattr(cfg, k) for k in cfg.__dataclass_fields__},
                                  "num_hidden_layers": args.max_layers,
                                  "layer_types": cfg.layer_types[:args.max_layers]})
    lb, le = topo.pipeline_layer_range(cfg.num_hidden_layers, info.pipeline_rank)
    first, last = info.pipeline_rank == 0, info.pipeline_rank == args.pp - 1
    fused_comm = None
    zero2 = args.zero_stage == 2
    if zero2 and (opt_mode != "flat" or args.skip_optimizer_step):
        raise SystemExit("--zero-stage 2 needs the flat sharded optimizer and an optimizer step")
    if zero2 and args.tp > 1:
        # the sequence-parallel and mirror-store layer paths do not carry the bucket boundaries
        if args.tp_comm != "nccl" and rank == 0:
            print("note: --zero-stage 2 with --tp > 1 uses --tp-comm nccl", flush=True)
        args.tp_comm = "nccl"
    if zero2 and (args.tp > 1 or args.cp > 1 or args.ep > 1 or args.pp > 1) and args.zero_comm == "symm":
        if rank == 0:
            print("note: --zero-stage 2 with model parallelism uses --zero-comm nccl", flush=True)
        args.zero_comm = "nccl"
    if args.zero_comm == "symm" and args.dp > 1 and opt_mode == "flat":
        if not use_cuda or dtype != torch.bfloat16:
            raise SystemExit("--zero-comm symm needs CUDA and --dtype bfloat16")
        from ..parallel.symm import FusedZeroComm, SymmetricHeap
        if zero2:
            from ..parallel.zero2 import FusedZero2Comm
            fused_comm = FusedZero2Comm(SymmetricHeap(ctx.dp_group, device))
        else:
            fused_comm = FusedZeroComm(SymmetricHeap(ctx.dp_group, device))
    symm_ok = use_cuda and dtype == torch.bfloat16
    seq_local = (args.prompt_len + args.response_len) // max(args.cp, 1)
    rows = args.micro_batch_seqs * seq_local
    if args.activation_checkpointing:
        # the peer-memory paths hand per-layer buffers from the forward to the backward pass in launch order; a layer
        # that runs a second time in the middle of the backward pass is only validated on the collective paths
        for name in ("tp_comm", "ep_comm", "cp_comm"):
            if getattr(args, name) in ("sp", "symm"):
                if rank == 0 and getattr(args, name.split("_")[0]) > 1:
                    print(f"note: --activation-checkpointing uses --{name.replace('_', '-')} nccl", flush=True)
                setattr(args, name, "nccl")
    if args.tp_comm == "symm" and args.tp > 2 and symm_ok:
        # the mirror-store all-reduce sends every partial N-1 times: measured faster than NCCL at TP=2 only
        if rank == 0:
            print("note: --tp-comm symm is used at --tp 2 only; falling back to NCCL all-reduces", flush=True)
        args.tp_comm = "nccl"
    if args.tp_comm == "sp" and args.tp > 1:
        if not symm_ok or args.pp > 1 or args.cp > 1 or cfg.is_qwen3_moe or rows % (128 * args.tp):
            raise SystemExit("--tp-comm sp needs CUDA, bf16, a dense model, --pp 1 --cp 1 and a micro-batch whose "
                             "token count is a multiple of 128 * tp")
        from ..parallel.tp_sp import TpSp
        ctx.tp_sp = TpSp(ctx.tp_group, device, rows, cfg.hidden_size, arena_slots=2 * cfg.num_hidden_layers + 1)
    if args.tp_comm == "symm" and args.tp > 1 and symm_ok:
        from ..parallel.tp_symm import TpSymm
        ctx.tp_symm = TpSymm(ctx.tp_group, device, rows, cfg.hidden_size)
    if args.ep_comm == "symm" and args.ep > 1 and symm_ok and cfg.is_qwen3_moe:
        from ..parallel.ep_symm import EpSymm
        cap = int(rows * cfg.num_experts_per_tok * args.ep_capacity_factor) + 128
        ctx.ep_symm = EpSymm(ctx.ep_group, device, cap, cfg.hidden_size)
    ctx.cp_zigzag = args.cp > 1 and args.cp_attn == "zigzag" and args.cp_comm != "symm"
    if args.cp_comm == "symm" and args.cp > 1 and symm_ok:
        if args.pp > 1:
            # the peer-mapped K / V buffers hold ONE micro-batch per layer; 1F1B keeps several in flight
            if rank == 0:
                print("note: --cp-comm symm is not combined with --pp > 1; using the NCCL ring", flush=True)
        else:
            from ..parallel.cp_symm import CpSymm
            ctx.cp_symm = CpSymm(ctx.cp_group, device)
    model = Qwen35Model(cfg, dtype=dtype, device=device, ctx=ctx, layer_begin=lb, layer_end=le, first_stage=first,
                        last_stage=last, pad_multiple=args.dp * 8,
                        flat_allocator=fused_comm.allocator if fused_comm else None, grad_buckets=zero2,
                        bucket_align=args.dp * 8, grad_slots=args.zero_grad_slots,
                        activation_checkpointing=args.activation_checkpointing)
    if loader is not None:
        load_model_weights(model, loader)
    else:
        model.init_weights(seed=args.seed, per_tensor=True)     # a stage starts from the one-stage model's weights
    comm_dtype = None if args.dp_grad_comm_dtype in ("float32", "model") else _DTYPES[args.dp_grad_comm_dtype]
    adam_opts = AdamWOptions(lr=args.lr, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=args.weight_decay,
                             use_master_weights=args.master_weights)
    if zero2:
        from ..parallel.zero2 import BucketedZero2Optimizer
        opt = BucketedZero2Optimizer(model, adam_opts, dp_group=ctx.dp_group, dp_rank=ctx.dp_rank, dp_size=args.dp,
                                     norm_group=None, norm_world=world, max_grad_norm=args.max_grad_norm,
                                     fused_comm=fused_comm, comm_dtype=None if fused_comm is not None else comm_dtype)
    elif opt_mode == "flat":
        opt = FlatZeroOptimizer(model.flat, adam_opts, dp_group=ctx.dp_group, dp_rank=ctx.dp_rank, dp_size=args.dp,
                                norm_group=None, norm_world=world, max_grad_norm=args.max_grad_norm,
                                comm_dtype=comm_dtype, fused_comm=fused_comm)
    else:
        # gradients are identical over the data-parallel group after the all-reduce: the norm is summed over
        # one model replica (reference: trainer.cc:2483-2494)
        replica_world = world // args.dp
        opt = TensorwiseOptimizer(model.flat, adam_opts, mode=opt_mode, dp_group=ctx.dp_group, dp_rank=ctx.dp_rank,
                                  dp_size=args.dp, norm_group=getattr(ctx, "model_group", None),
                                  norm_world=replica_world, max_grad_norm=args.max_grad_norm, comm_dtype=comm_dtype,
                                  bucket_bytes=args.dp_grad_bucket_mb * 1024 * 1024)
    ecfg = ActorConfig(mode=args.mode, micro_batch_size=args.micro_batch_seqs, clip_ratio=args.clip_ratio,
                       clip_ratio_c=args.clip_ratio_c, kl_coef=args.kl_coef, kl_penalty=args.kl_penalty,
                       advantage_scale=args.advantage_scale)
    rank_info = {"data_rank": info.data_rank, "pipeline_rank": info.pipeline_rank, "context_rank": info.context_rank,
                 "tensor_rank": info.tensor_rank, "expert_rank": info.expert_rank, "layer_begin": lb, "layer_end": le}
    start_step = 0
    if args.resume_checkpoint:
        if opt_mode == "flat":
            start_step = ckpt.load_rank_checkpoint(args.resume_checkpoint, rank, model, opt, rank_info)
            shard = model.flat.flat[opt.begin:opt.end] if not zero2 else None
            if zero2:
                opt.all_gather_params()
            elif args.dp > 1:  # rebuild the full parameters from the DP shards
                if use_cuda:
                    dist.all_gather_into_tensor(model.flat.flat, shard.clone(), group=ctx.dp_group)
                else:
                    parts = [torch.empty_like(shard) for _ in range(args.dp)]
                    dist.all_gather(parts, shard.clone(), group=ctx.dp_group)
                    model.flat.flat.copy_(torch.cat(parts))
        else:
            start_step = ckpt.load_rank_checkpoint_v2(args.resume_checkpoint, rank, opt.names, opt.tensors, opt.adam,
                                                      opt.optimizer_param_indices, rank_info)
    source = BatchSource(args, cfg, device, global_rank=rank, needs_batch=first or last)
    csv = MetricsCsv(args.metrics_csv if rank == 0 else None)
    watchdog = None
    if args.heartbeat_timeout_s > 0 and world > 1:
        store = dist.distributed_c10d._get_default_store()
        hb = Heartbeat(store, rank, world)
        hb.beat()
        hb.start_background(max(args.heartbeat_timeout_s / 4.0, 0.05))   # host thread: step length does not matter
        watchdog = Watchdog(hb, args.heartbeat_timeout_s)
        _ACTIVE_HEARTBEAT[0] = hb
        watchdog.wait_for_peers(max(10.0 * args.heartbeat_timeout_s, 60.0))  # peers may still be loading weights
    S = args.prompt_len + args.response_len
    mbs = args.micro_batch_seqs
    stage = None
    if args.pp > 1:
        peers = pipeline_peers(info.pipeline_group, info.pipeline_rank)
        from ..parallel.context_parallel import padded_shard_len
        stage = PipelineStage(peers, info.pipeline_rank, args.pp, args.micro_batches,
                              (mbs * (padded_shard_len(S, args.cp) if args.cp > 1 else S), cfg.hidden_size), dtype,
                              device)
    engine = ActorEngine(model, opt, ecfg)
    exit_ok = True
    log_lines = []
    fault = HostFault.from_env()
    for step in range(start_step, args.steps):
        if fault is not None:           # tests only: a host-side failure between steps, nothing in flight
            fault.fire(rank, step, sync=torch.cuda.synchronize if use_cuda else None)
        if watchdog is not None:
            watchdog.hb.beat(step)
            watchdog.check()            # host-side: raises before any kernel of this step is launched
        if world > 1:
            dist.barrier()
        if use_cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        before = model.flat.flat.detach().clone() if args.measure_param_delta else None
        rollout = source.acquire(step)
        total = torch.zeros(6, dtype=torch.float32, device=device)
        grad_scale = 1.0 / (args.micro_batches * args.grad_accum_steps * args.cp)
        data_step = step if args.vary_tokens_by_step else 0
        for accum in range(args.grad_accum_steps):
            def rows_of(m):
                base = batch_row_index(data_step, accum, args.grad_accum_steps, m, args.micro_batches, args.dp,
                                       args.ep, info.data_rank, info.expert_rank, args.rows)
                return [(base + j * 7919) % args.rows for j in range(mbs)]
            if stage is None:
                for m in range(args.micro_batches):
                    batch = source.micro_batch(rows_of(m), rollout)
                    lp = model.response_logprobs(batch["input_ids"], args.prompt_len)
                    seed, metrics = _score(ecfg, lp, batch, grad_scale)
                    lp.backward(seed.to(lp.dtype))
                    total += metrics.to(device)
            else:
                batches = {m: source.micro_batch(rows_of(m), rollout) if (first or last) else None
                           for m in range(args.micro_batches)}
                seeds = {}

                def forward_fn(m, x):
                    b = batches[m]
                    s_stage = model.cp_shard_len(S) if args.cp > 1 else S
                    if first:
                        x = model.cp_embed(b["input_ids"]) if args.cp > 1 else model.embed(b["input_ids"])
                    return model.forward_layers(x, mbs, s_stage)

                def loss_fn(m, hidden):
                    lp, seed, metrics = _loss_and_seed(model, ecfg, hidden, batches[m], args.prompt_len, grad_scale)
                    seeds[m] = metrics
                    return lp, seed
                stage.run(forward_fn, loss_fn)
                for mt in seeds.values():
                    total += mt.to(device)
        if not zero2:      # bucketed gradients: folded and summed bucket by bucket as the backward pass completes them
            engine.fold_autograd_grads()
            model.sync_replicated_grads()
            if args.cp > 1:
                dist.all_reduce(model.flat.main_grad, group=ctx.cp_group)
        if args.pp > 1 and cfg.lm_head_name == cfg.embed_name and (first or last) and not zero2:
            # the tied embedding lives on the first and the last stage: sum its two gradient halves so
            # that both copies take the same update (the reference leaves them unsynchronised)
            dist.all_reduce(model.param(cfg.embed_name).main_grad, group=ctx.embed_group)
        if args.ep > 1 and not zero2:  # EP ranks are data-parallel replicas for the non-expert parameters
            _average_non_expert_grads(model, ctx)
        if args.skip_optimizer_step:
            grad_abs = model.flat.main_grad.float().norm()
            model.flat.main_grad.zero_()
        else:
            opt.step()
            # norm of this rank's share of the REDUCED gradient times the clip scale: what the reference reports
            # (trainer.cc:2463-2467,2520-2523), and positive on a rank whose own rows happened to give no gradient
            grad_abs = opt.last_metrics[0].sqrt() * opt.last_metrics[2]
        delta = ((model.flat.flat.float() - before.float()).abs().sum() if before is not None
                 else torch.zeros((), device=device))
        if use_cuda:
            torch.cuda.synchronize()
        step_time = time.perf_counter() - t0
        # kernel status word (a bounded wait that ran out) and the expert-parallel receive-buffer overflow flag ride
        # along with the metrics, so a corrupted step is seen at the step's one host read
        status = _native.status_word(device).float().reshape(()) if use_cuda else torch.zeros((), device=device)
        eps = getattr(ctx, "ep_symm", None)
        overflow = eps.overflow.float().reshape(()) if eps is not None else torch.zeros((), device=device)
        local = torch.stack([total[0], total[4], total[2], total[1], grad_abs, opt.last_metrics[1].sqrt(),
                             opt.last_metrics[2], delta, torch.tensor(step_time, device=device), status,
                             overflow]).float()
        if world > 1:
            gathered = torch.empty(world, local.numel(), dtype=torch.float32, device=device)
            if use_cuda:
                dist.all_gather_into_tensor(gathered, local)
            else:
                parts = [torch.empty_like(local) for _ in range(world)]
                dist.all_gather(parts, local)
                gathered = torch.stack(parts)
        else:
            gathered = local.unsqueeze(0)
        g = gathered.cpu()                                  # the step's one metrics read
        if bool((g[:, 9] != 0).any()) or bool((g[:, 10] != 0).any()):
            bad = [int(r) for r in torch.nonzero((g[:, 9] != 0) | (g[:, 10] != 0)).flatten()]
            what = ("a kernel's bounded wait ran out (status " + str([int(x) for x in g[:, 9]]) + ")"
                    if bool((g[:, 9] != 0).any()) else "an expert-parallel receive buffer overflowed "
                    "(raise --ep-capacity-factor)")
            if use_cuda:
                _native.status_word(device).zero_()
            raise RuntimeError(f"step {step}: {what} on ranks {bad}; the step's results are not trustworthy, "
                               f"no checkpoint is written")
        have_grad = bool((g[:, 4] > 0).all())
        if args.measure_param_delta:
            updated, any_updated = bool((g[:, 7] > 0).all()), bool((g[:, 7] > 0).any())
        else:
            updated = any_updated = not args.skip_optimizer_step
        last_stage_rows = g[g[:, 0] != 0] if (g[:, 0] != 0).any() else g
        tokens = args.micro_batches * args.grad_accum_steps * mbs * S * args.dp * args.ep
        values = {
            "step": step, "train_mode": args.mode, "dp": args.dp, "pp": args.pp, "cp": args.cp, "tp": args.tp,
            "ep": args.ep, "sp": args.sp,
            "micro_batches": args.micro_batches, "grad_accum_steps": args.grad_accum_steps,
            "prompt_len": args.prompt_len, "response_len": args.response_len, "seq_len": S, "tokens": tokens,
            "step_time_s": float(g[:, 8].max()), "tokens_per_second": tokens / max(float(g[:, 8].max()), 1e-9),
            "dtype": args.dtype, "dp_grad_comm_dtype": args.dp_grad_comm_dtype,
            "tp_grad_comm_dtype": args.tp_grad_comm_dtype,
            "flat_shard_optimizer": opt_mode == "flat", "dp_shard_optimizer": opt_mode != "dense",
            "master_weights": args.master_weights,
            "rollout_rows": rollout.rows if rollout is not None else 0, "kl_coef": args.kl_coef,
            "mean_reward": rollout.mean_reward if rollout is not None else 0.0,
            "success_rate": rollout.success_rate if rollout is not None else 0.0,
            "adv_abs_sum": rollout.adv_abs_sum if rollout is not None else 0.0,
            "loss_sum": float(last_stage_rows[:, 0].sum()),
            "kl_loss_sum": float(last_stage_rows[:, 1].sum()), "ppo_kl_sum": float(last_stage_rows[:, 2].sum()),
            "clipfrac_sum": float(last_stage_rows[:, 3].sum()), "grad_norm_sum": float(g[:, 4].sum()),
            "global_grad_norm": float(g[0, 5]), "grad_clip_scale": float(g[0, 6]),
            "param_delta_sum": float(g[:, 7].sum()), "all_ranks_have_grad": have_grad,
            "all_ranks_updated": updated, "any_rank_updated": any_updated,
            "native_fallbacks": _fallbacks.total(),
        }
        exit_ok = exit_ok and have_grad and (args.skip_optimizer_step or any_updated)
        if rank == 0:
            line = format_line(values)
            print(line, flush=True)
            log_lines.append(line)
            csv.append(values)
        if args.checkpoint_dir and args.checkpoint_every > 0 and (step + 1) % args.checkpoint_every == 0:
            if opt_mode == "flat":
                ckpt.save_rank_checkpoint(args.checkpoint_dir, step + 1, rank, model, opt, rank_info,
                                          args.flat_checkpoint_save_model_params)
                optim_step = opt.adam.step_count
            else:
                ckpt.save_rank_checkpoint_v2(args.checkpoint_dir, step + 1, rank, opt.names, opt.tensors, opt.adam,
                                             opt.optimizer_param_indices, rank_info)
                optim_step = opt.step_count
            if world > 1:
                dist.barrier()
            if rank == 0:
                dims = {"dp": args.dp, "pp": args.pp, "cp": args.cp, "tp": args.tp, "ep": args.ep, "sp": args.sp}
                ckpt.write_manifest(args.checkpoint_dir, step + 1, world, dims, training_config(args, cfg, opt_mode),
                                    {"lr": args.lr, "beta1": 0.9, "beta2": 0.95, "eps": 1e-8,
                                     "weight_decay": args.weight_decay},
                                    with_params=args.flat_checkpoint_save_model_params, optimizer_step=optim_step,
                                    flat=opt_mode == "flat", use_master_weights=args.master_weights)
            if world > 1:
                dist.barrier()
    if watchdog is not None:
        watchdog.hb.stop()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if exit_ok else 2


_ACTIVE_HEARTBEAT: List[Optional[Heartbeat]] = [None]


def training_config(args, cfg, opt_mode: str) -> dict:
    """The ``training_config`` block of the checkpoint manifest (reference: trainer.cc:1106-1153)."""
    return {
        "dtype": args.dtype, "dp_grad_comm_dtype": args.dp_grad_comm_dtype,
        "tp_grad_comm_dtype": args.tp_grad_comm_dtype, "dp_grad_bucket_mb": args.dp_grad_bucket_mb,
        "tp_grad_bucket_mb": args.tp_grad_bucket_mb, "micro_batches": args.micro_batches,
        "grad_accum_steps": args.grad_accum_steps, "layers": cfg.num_hidden_layers, "context_parallel": args.cp,
        "expert_parallel": args.ep, "sequence_parallel": args.sp, "prompt_len": args.prompt_len,
        "response_len": args.response_len, "max_grad_norm": args.max_grad_norm, "clip_ratio": args.clip_ratio,
        "kl_coef": args.kl_coef, "kl_penalty": args.kl_penalty, "advantage_scale": args.advantage_scale,
        "use_master_weights": args.master_weights, "dp_shard_optimizer": opt_mode != "dense",
        "dp_flat_shard_optimizer": opt_mode == "flat",
        "flat_checkpoint_save_model_params": args.flat_checkpoint_save_model_params, "train_mode": args.mode,
        "micro_batch_seqs": args.micro_batch_seqs,
    }


def _average_non_expert_grads(model, ctx) -> None:
    """Expert-parallel ranks train different micro-batches: every parameter that is not an expert
    weight is a data-parallel replica over the EP group and its gradient is averaged there
    (reference: trainer.cc:560-566,2431)."""
    import torch.distributed as dist
    grads = [p.main_grad for n, p in model.flat.params.items() if not n.startswith("__packed_moe")]
    if not grads:
        return
    flat = torch.cat([g.reshape(-1) for g in grads])
    dist.all_reduce(flat, group=ctx.ep_group)
    flat /= ctx.ep_size
    off = 0
    for g in grads:
        g.copy_(flat[off:off + g.numel()].view_as(g))
        off += g.numel()


def main() -> None:
    try:
        sys.exit(run())
    except PeerFailure as exc:
        print(f"peer failure: {exc}", file=sys.stderr)
        sys.exit(3)
    except BaseException as exc:  # noqa: BLE001 - published to the peers, then re-raised
        hb = _ACTIVE_HEARTBEAT[0]
        if hb is not None and not isinstance(exc, SystemExit):
            try:
                hb.report_failure(f"{type(exc).__name__}: {exc}")
            except Exception:
                pass
        raise


if __name__ == "__main__":
    main()
