"""Distributed PPO / GRPO / SFT trainer for Qwen3.5 and Qwen3-MoE over DP x PP x CP x TP x EP.

One process per GPU (``torchrun`` or any launcher that sets RANK / WORLD_SIZE / LOCAL_RANK):

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m cverl_b200.trainer.ppo_trainer --config qwen3_5_0_8b --dp 4 --tp 2 --steps 5

The step is the reference trainer's (tools/model/qwen3_5_pp_tp_ppo_trainer.cc:2200-2742): barrier and
device sync, batch acquisition, micro-batches in 1F1B order (one sequence group per micro-batch), PPO
clipped loss (+ KL) or SFT NLL divided by micro_batches * grad_accum_steps, CP / TP-replicated gradient
sync, flat-sharded AdamW, ``step_time_s`` as the max over ranks, nine metrics all-gathered over the world,
one ``key=value`` line and a CSV row on rank 0, rank-local checkpoints with a manifest, and an exit code
that reflects ``all_ranks_have_grad`` / ``all_ranks_updated``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path
from typing import Dict, List, Optional

import torch

from ..models.config import Qwen35TextConfig
from ..models.hf_io import HfModelLoader, load_model_weights
from ..models.qwen3_5 import Qwen35Model
from ..ops import rl
from ..optim import AdamWOptions
from ..parallel.mesh import build_context
from ..parallel.pipeline import PipelineStage, pipeline_peers
from ..parallel.zero import FlatZeroOptimizer
from ..utils import checkpoint as ckpt
from ..utils.metrics import MetricsCsv, format_line
from ..utils.watchdog import Heartbeat, PeerFailure, Watchdog
from .actor import ActorConfig, ActorEngine

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "float16": torch.float16}


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    g = ap.add_argument_group("model")
    g.add_argument("--model-dir", default="")
    g.add_argument("--config", default="tiny", help="built-in shape when no --model-dir: qwen3_5_0_8b, qwen3_30b_a3b, tiny, tiny_moe")
    g.add_argument("--max-layers", type=int, default=-1)
    g.add_argument("--dtype", default="bfloat16")
    g = ap.add_argument_group("parallelism")
    for name in ("dp", "pp", "cp", "tp", "ep", "sp"):
        g.add_argument(f"--{name}", type=int, default=1)
    g.add_argument("--micro-batches", type=int, default=1)
    g.add_argument("--micro-batch-seqs", type=int, default=1, help="sequences per micro-batch (the reference uses 1)")
    g.add_argument("--grad-accum-steps", type=int, default=1)
    g.add_argument("--backend", default="auto", choices=["auto", "nccl", "gloo"])
    g = ap.add_argument_group("data")
    g.add_argument("--prompt-len", type=int, default=8)
    g.add_argument("--response-len", type=int, default=8)
    g.add_argument("--rows", type=int, default=64, help="rows of the synthetic batch table")
    g.add_argument("--sft-jsonl", default="")
    g.add_argument("--rollout-dir", default="", help="directory of rollout_step_%%06d.json files")
    g.add_argument("--tokenizer-json", default="")
    g = ap.add_argument_group("algorithm")
    g.add_argument("--mode", default="ppo", choices=["ppo", "sft"])
    g.add_argument("--steps", type=int, default=2)
    g.add_argument("--lr", type=float, default=1e-8)
    g.add_argument("--weight-decay", type=float, default=0.01)
    g.add_argument("--clip-ratio", type=float, default=0.2)
    g.add_argument("--clip-ratio-c", type=float, default=3.0)
    g.add_argument("--kl-coef", type=float, default=0.0)
    g.add_argument("--kl-penalty", default="k1")
    g.add_argument("--advantage-scale", type=float, default=1.0)
    g.add_argument("--max-grad-norm", type=float, default=1.0)
    g.add_argument("--zero-comm", default="nccl", choices=["nccl", "symm"],
                   help="ZeRO gradient reduce-scatter / parameter all-gather: library collectives, or this "
                        "package's kernels over peer-mapped memory (CUDA, bf16 parameters, same node)")
    g.add_argument("--tp-comm", default="nccl", choices=["nccl", "symm"],
                   help="tensor-parallel all-reduces: NCCL, or fused into the GEMM epilogue over peer-mapped memory")
    g.add_argument("--ep-comm", default="nccl", choices=["nccl", "symm"],
                   help="expert-parallel dispatch / combine: NCCL all-to-all, or row scatter / gather kernels over "
                        "peer-mapped memory (no host read)")
    g.add_argument("--cp-comm", default="nccl", choices=["nccl", "symm"],
                   help="context-parallel attention: ring send/recv, or K / V pulled from the owners by the kernels")
    g.add_argument("--ep-capacity-factor", type=float, default=2.0,
                   help="receive-buffer rows per rank for --ep-comm symm, as a multiple of the balanced load")
    g.add_argument("--master-weights", action="store_true")
    g.add_argument("--dp-grad-comm-dtype", default="float32")
    g.add_argument("--seed", type=int, default=1234)
    g = ap.add_argument_group("output")
    g.add_argument("--metrics-csv", default="")
    g.add_argument("--checkpoint-dir", default="")
    g.add_argument("--checkpoint-every", type=int, default=0)
    g.add_argument("--flat-checkpoint-save-model-params", action="store_true")
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


class BatchSource:
    """Synthetic rows, SFT examples from a JSONL file, or rollout JSON files written by a rollout process."""

    def __init__(self, args, cfg: Qwen35TextConfig, device):
        self.args, self.cfg, self.device = args, cfg, device
        self.S = args.prompt_len + args.response_len
        self.sft = None
        if args.sft_jsonl:
            from ..data import load_prompt_answer_jsonl
            from ..text import ByteTokenizer, HfBpeTokenizer
            tok = HfBpeTokenizer(args.tokenizer_json) if args.tokenizer_json else ByteTokenizer()
            self.sft = []
            for ex in load_prompt_answer_jsonl(args.sft_jsonl, max_examples=args.rows):
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

    def rollout_step(self, step: int) -> Optional[dict]:
        if not self.args.rollout_dir:
            return None
        path = Path(self.args.rollout_dir) / f"rollout_step_{step:06d}.json"
        if not path.exists():
            raise FileNotFoundError(f"rollout file for step {step} not found: {path}")
        data = json.loads(path.read_text())
        if int(data.get("step", step)) != step:
            raise RuntimeError(f"rollout step mismatch: file says {data.get('step')}, trainer is at {step}")
        return data

    def micro_batch(self, rows: List[int], rollout: Optional[dict]) -> Dict[str, torch.Tensor]:
        a, dev = self.args, self.device
        ids, masks, advs, olds = [], [], [], []
        for row in rows:
            if rollout is not None:
                seqs = rollout["sequences"]
                s = seqs[row % len(seqs)]
                full = (s["prompt_ids"][-a.prompt_len:] + s["response_ids"])[:self.S]
                t = torch.ones(self.S, dtype=torch.long)
                t[:len(full)] = torch.tensor(full, dtype=torch.long) % self.cfg.vocab_size
                n = min(len(s["response_ids"]), a.response_len)
                m = torch.zeros(a.response_len)
                m[:n] = 1.0
                ids.append(t)
                masks.append(m)
                advs.append(torch.full((a.response_len,), float(s.get("advantage", a.advantage_scale))) * m)
                if "old_log_probs" in s:
                    o = torch.zeros(a.response_len)
                    o[:n] = torch.tensor(s["old_log_probs"][:n])
                    olds.append(o)
            elif self.sft is not None:
                t, m = self.sft[row % len(self.sft)]
                ids.append(t)
                masks.append(m)
            else:
                ids.append(synthetic_token_row(row, self.S, self.cfg.vocab_size, "cpu"))
                masks.append(torch.ones(a.response_len))
        out = {"input_ids": torch.stack(ids).to(dev), "response_mask": torch.stack(masks).to(dev)}
        if advs:
            out["advantages"] = torch.stack(advs).to(dev)
        if olds and len(olds) == len(ids):
            out["old_log_probs"] = torch.stack(olds).to(dev)
        return out


def _loss_and_seed(model, engine_cfg: ActorConfig, hidden, batch, prompt_len, grad_scale):
    """Last-stage scoring of one micro-batch: returns (log-probs, gradient seed, metrics[6])."""
    B, S = batch["input_ids"].shape
    R = S - prompt_len
    h = hidden.view(B, S, -1)[:, prompt_len - 1:prompt_len - 1 + R]
    lp = model.token_logprobs(h, batch["input_ids"][:, prompt_len:])
    mask = batch["response_mask"]
    if engine_cfg.mode == "sft":
        denom = mask.sum() + rl.EPS
        seed = (-mask / denom) * grad_scale
        nll = -(lp.detach() * mask).sum() / denom
        z = nll.new_zeros(())
        return lp, seed, torch.stack([nll, z, z, z, z, mask.sum()])
    adv = batch.get("advantages")
    adv = adv if adv is not None else torch.full_like(lp, engine_cfg.advantage_scale).detach()
    old = batch.get("old_log_probs")
    old = old if old is not None else lp.detach()
    metrics, seed = rl.actor_loss(old, lp.detach(), adv, mask, None, clip_ratio=engine_cfg.clip_ratio,
                                  clip_ratio_c=engine_cfg.clip_ratio_c, loss_scale=grad_scale)
    return lp, seed.to(lp.dtype), metrics


def run(argv=None) -> int:
    args = build_parser().parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
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
        raise SystemExit("cp > 1 together with tp > 1 is not supported")
    if args.sp != 1:
        raise SystemExit("sequence parallelism (--sp) is declared in the topology but is not a trainer mode")
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
    if args.zero_comm == "symm" and args.dp > 1:
        if not use_cuda or dtype != torch.bfloat16:
            raise SystemExit("--zero-comm symm needs CUDA and --dtype bfloat16")
        from ..parallel.symm import FusedZeroComm, SymmetricHeap
        fused_comm = FusedZeroComm(SymmetricHeap(ctx.dp_group, device))
    symm_ok = use_cuda and dtype == torch.bfloat16
    seq_local = (args.prompt_len + args.response_len) // max(args.cp, 1)
    rows = args.micro_batch_seqs * seq_local
    if args.tp_comm == "symm" and args.tp > 2 and symm_ok:
        # the mirror-store all-reduce sends every partial N-1 times: measured faster than NCCL at TP=2 only
        if rank == 0:
            print("note: --tp-comm symm is used at --tp 2 only; falling back to NCCL all-reduces", flush=True)
        args.tp_comm = "nccl"
    if args.tp_comm == "symm" and args.tp > 1 and symm_ok:
        from ..parallel.tp_symm import TpSymm
        ctx.tp_symm = TpSymm(ctx.tp_group, device, rows, cfg.hidden_size)
    if args.ep_comm == "symm" and args.ep > 1 and symm_ok and cfg.is_qwen3_moe:
        from ..parallel.ep_symm import EpSymm
        cap = int(rows * cfg.num_experts_per_tok * args.ep_capacity_factor) + 128
        ctx.ep_symm = EpSymm(ctx.ep_group, device, cap, cfg.hidden_size)
    if args.cp_comm == "symm" and args.cp > 1 and symm_ok:
        from ..parallel.cp_symm import CpSymm
        ctx.cp_symm = CpSymm(ctx.cp_group, device)
    model = Qwen35Model(cfg, dtype=dtype, device=device, ctx=ctx, layer_begin=lb, layer_end=le, first_stage=first,
                        last_stage=last, pad_multiple=args.dp * 8,
                        flat_allocator=fused_comm.allocator if fused_comm else None)
    if loader is not None:
        load_model_weights(model, loader)
    else:
        model.init_weights(seed=args.seed)
    comm_dtype = None if args.dp_grad_comm_dtype in ("float32", "model") else _DTYPES[args.dp_grad_comm_dtype]
    opt = FlatZeroOptimizer(model.flat, AdamWOptions(lr=args.lr, beta1=0.9, beta2=0.95, eps=1e-8,
                                                     weight_decay=args.weight_decay,
                                                     use_master_weights=args.master_weights),
                            dp_group=ctx.dp_group, dp_rank=ctx.dp_rank, dp_size=args.dp, norm_group=None,
                            norm_world=world, max_grad_norm=args.max_grad_norm, comm_dtype=comm_dtype,
                            fused_comm=fused_comm)
    ecfg = ActorConfig(mode=args.mode, micro_batch_size=args.micro_batch_seqs, clip_ratio=args.clip_ratio,
                       clip_ratio_c=args.clip_ratio_c, kl_coef=args.kl_coef, kl_penalty=args.kl_penalty,
                       advantage_scale=args.advantage_scale)
    rank_info = {"data_rank": info.data_rank, "pipeline_rank": info.pipeline_rank, "context_rank": info.context_rank,
                 "tensor_rank": info.tensor_rank, "expert_rank": info.expert_rank, "layer_begin": lb, "layer_end": le}
    start_step = 0
    if args.resume_checkpoint:
        start_step = ckpt.load_rank_checkpoint(args.resume_checkpoint, rank, model, opt, rank_info)
        shard = model.flat.flat[opt.begin:opt.end]
        if args.dp > 1:  # rebuild the full parameters from the DP shards
            if use_cuda:
                dist.all_gather_into_tensor(model.flat.flat, shard.clone(), group=ctx.dp_group)
            else:
                parts = [torch.empty_like(shard) for _ in range(args.dp)]
                dist.all_gather(parts, shard.clone(), group=ctx.dp_group)
                model.flat.flat.copy_(torch.cat(parts))
    source = BatchSource(args, cfg, device)
    csv = MetricsCsv(args.metrics_csv if rank == 0 else None)
    watchdog = None
    if args.heartbeat_timeout_s > 0 and world > 1:
        store = dist.distributed_c10d._get_default_store()
        hb = Heartbeat(store, rank, world)
        hb.beat()
        watchdog = Watchdog(hb, args.heartbeat_timeout_s)
    S = args.prompt_len + args.response_len
    mbs = args.micro_batch_seqs
    stage = None
    if args.pp > 1:
        peers = pipeline_peers(info.pipeline_group, info.pipeline_rank)
        stage = PipelineStage(peers, info.pipeline_rank, args.pp, args.micro_batches,
                              (mbs * (S // args.cp if args.cp > 1 else S), cfg.hidden_size), dtype, device)
    exit_ok = True
    log_lines = []
    for step in range(start_step, args.steps):
        if watchdog is not None:
            watchdog.hb.beat(step)
            watchdog.check()            # host-side: raises before any kernel of this step is launched
        if world > 1:
            dist.barrier()
        if use_cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        before = model.flat.flat.detach().clone()
        rollout = source.rollout_step(step)
        total = torch.zeros(6, dtype=torch.float32, device=device)
        grad_scale = 1.0 / (args.micro_batches * args.grad_accum_steps * args.cp)
        for accum in range(args.grad_accum_steps):
            def rows_of(m):
                base = batch_row_index(step, accum, args.grad_accum_steps, m, args.micro_batches, args.dp, args.ep,
                                       info.data_rank, info.expert_rank, args.rows)
                return [(base + j * 7919) % args.rows for j in range(mbs)]
            if stage is None:
                for m in range(args.micro_batches):
                    batch = source.micro_batch(rows_of(m), rollout)
                    lp = model.response_logprobs(batch["input_ids"], args.prompt_len)
                    fake_hidden = None
                    mask = batch["response_mask"]
                    if ecfg.mode == "sft":
                        denom = mask.sum() + rl.EPS
                        seed = (-mask / denom) * grad_scale
                        nll = -(lp.detach() * mask).sum() / denom
                        z = nll.new_zeros(())
                        metrics = torch.stack([nll, z, z, z, z, mask.sum()])
                    else:
                        adv = batch.get("advantages")
                        adv = adv if adv is not None else torch.full_like(lp, ecfg.advantage_scale).detach()
                        old = batch.get("old_log_probs", lp.detach())
                        metrics, seed = rl.actor_loss(old, lp.detach(), adv, mask, None, clip_ratio=ecfg.clip_ratio,
                                                      clip_ratio_c=ecfg.clip_ratio_c, loss_scale=grad_scale)
                    lp.backward(seed.to(lp.dtype))
                    total += metrics.to(device)
            else:
                batches = {m: source.micro_batch(rows_of(m), rollout) for m in range(args.micro_batches)}
                seeds = {}

                def forward_fn(m, x):
                    b = batches[m]
                    if first:
                        x = model.embed(b["input_ids"])
                    return model.forward_layers(x, b["input_ids"].shape[0], S)

                def loss_fn(m, hidden):
                    lp, seed, metrics = _loss_and_seed(model, ecfg, hidden, batches[m], args.prompt_len, grad_scale)
                    seeds[m] = metrics
                    return lp, seed
                stage.run(forward_fn, loss_fn)
                for mt in seeds.values():
                    total += mt.to(device)
        engine = ActorEngine(model, opt, ecfg)
        engine.fold_autograd_grads()
        model.sync_replicated_grads()
        if args.cp > 1:
            dist.all_reduce(model.flat.main_grad, group=ctx.cp_group)
        if args.pp > 1 and cfg.lm_head_name == cfg.embed_name and (first or last):
            # the tied embedding lives on the first and the last stage: sum its two gradient halves so
            # that both copies take the same update (the reference leaves them unsynchronised)
            dist.all_reduce(model.param(cfg.embed_name).main_grad, group=ctx.embed_group)
        if args.ep > 1:  # EP ranks are data-parallel replicas for the non-expert parameters
            _average_non_expert_grads(model, ctx)
        grad_abs = model.flat.main_grad.abs().sum()
        opt.step()
        delta = (model.flat.flat.float() - before.float()).abs().sum()
        if use_cuda:
            torch.cuda.synchronize()
        step_time = time.perf_counter() - t0
        local = torch.stack([total[0], total[4], total[2], total[1], grad_abs, opt.last_metrics[1].sqrt(),
                             opt.last_metrics[2], delta, torch.tensor(step_time, device=device)]).float()
        if world > 1:
            gathered = torch.empty(world, 9, dtype=torch.float32, device=device)
            if use_cuda:
                dist.all_gather_into_tensor(gathered, local)
            else:
                parts = [torch.empty_like(local) for _ in range(world)]
                dist.all_gather(parts, local)
                gathered = torch.stack(parts)
        else:
            gathered = local.unsqueeze(0)
        g = gathered.cpu()                                  # the step's one metrics read
        have_grad = bool((g[:, 4] > 0).all())
        updated = bool((g[:, 7] > 0).all())
        last_stage_rows = g[g[:, 0] != 0] if (g[:, 0] != 0).any() else g
        tokens = args.micro_batches * args.grad_accum_steps * mbs * S * args.dp * args.ep
        values = {
            "step": step, "dp": args.dp, "pp": args.pp, "cp": args.cp, "tp": args.tp, "ep": args.ep, "sp": args.sp,
            "micro_batches": args.micro_batches, "grad_accum_steps": args.grad_accum_steps,
            "prompt_len": args.prompt_len, "response_len": args.response_len, "seq_len": S, "tokens": tokens,
            "step_time_s": float(g[:, 8].max()), "tokens_per_second": tokens / max(float(g[:, 8].max()), 1e-9),
            "dtype": args.dtype, "dp_grad_comm_dtype": args.dp_grad_comm_dtype, "tp_grad_comm_dtype": "model",
            "flat_shard_optimizer": True, "master_weights": args.master_weights, "mean_reward": 0.0,
            "success_rate": 0.0, "adv_abs_sum": 0.0, "loss_sum": float(last_stage_rows[:, 0].sum()),
            "kl_loss_sum": float(last_stage_rows[:, 1].sum()), "ppo_kl_sum": float(last_stage_rows[:, 2].sum()),
            "clipfrac_sum": float(last_stage_rows[:, 3].sum()), "grad_norm_sum": float(g[:, 4].sum()),
            "global_grad_norm": float(g[0, 5]), "grad_clip_scale": float(g[0, 6]),
            "param_delta_sum": float(g[:, 7].sum()), "all_ranks_have_grad": have_grad,
            "all_ranks_updated": updated, "any_rank_updated": bool((g[:, 7] > 0).any()),
        }
        exit_ok = exit_ok and have_grad and updated
        if rank == 0:
            line = format_line(values)
            print(line, flush=True)
            log_lines.append(line)
            csv.append(values)
        if args.checkpoint_dir and args.checkpoint_every > 0 and (step + 1) % args.checkpoint_every == 0:
            ckpt.save_rank_checkpoint(args.checkpoint_dir, step + 1, rank, model, opt, rank_info,
                                      args.flat_checkpoint_save_model_params)
            if world > 1:
                dist.barrier()
            if rank == 0:
                dims = {"dp": args.dp, "pp": args.pp, "cp": args.cp, "tp": args.tp, "ep": args.ep}
                tc = {k: getattr(args, k) for k in ("dtype", "dp_grad_comm_dtype", "micro_batches", "prompt_len",
                                                    "response_len", "clip_ratio", "kl_coef", "kl_penalty",
                                                    "master_weights", "mode")}
                ckpt.write_manifest(args.checkpoint_dir, step + 1, world, dims, tc,
                                    {"lr": args.lr, "beta1": 0.9, "beta2": 0.95, "eps": 1e-8,
                                     "weight_decay": args.weight_decay},
                                    args.flat_checkpoint_save_model_params)
            if world > 1:
                dist.barrier()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if exit_ok else 2


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


if __name__ == "__main__":
    main()
