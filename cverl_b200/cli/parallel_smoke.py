"""Multi-process smokes of the parallel model paths, one process per rank under ``torchrun``.

``torchrun --nproc-per-node 2 --master-addr 127.0.0.1 -m cverl_b200.cli.parallel_smoke --mode tp [--backend gloo]``

Modes (each prints ``<mode> smoke passed`` on rank 0 and exits non-zero on a mismatch):

* ``tp``      dense vs tensor-parallel hidden states and response log-probs, allclose(1e-4) in fp32
              (reference: tools/model/qwen3_5_tp_smoke.cc:85);
* ``dp_tp``   DP x TP: every data-parallel replica ends with the same averaged gradient as a single
              rank that saw both batches (reference: tools/model/qwen3_5_dp_tp_smoke.cc);
* ``pp_tp``   PP x TP 1F1B with a ``square().mean()`` loss on the last stage: every rank holds gradients
              and the parameters move (reference: tools/model/qwen3_5_pp_tp_train_smoke.cc).

``--model-dir`` loads real weights; without it a tiny random model is used.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

from ..models.config import Qwen35TextConfig
from ..models.hf_io import HfModelLoader, load_model_weights
from ..models.qwen3_5 import Qwen35Model
from ..optim.adamw import AdamWOptions
from ..parallel.mesh import build_context
from ..parallel.pipeline import PipelineStage, pipeline_peers
from ..parallel.zero import FlatZeroOptimizer


def _fold(model) -> None:
    for p in list(model.flat.params.values()) + list(model.fused.values()):
        if p.grad is not None:
            p.main_grad.add_(p.grad.float())
            p.grad = None


def _model(cfg, loader, device, dtype, **kw):
    m = Qwen35Model(cfg, dtype=dtype, device=device, **kw)
    if loader is not None:
        load_model_weights(m, loader)
    else:
        m.init_weights(seed=11)
    return m


def main(argv=None) -> int:
    import torch.distributed as dist
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--mode", required=True, choices=["tp", "dp_tp", "pp_tp"])
    ap.add_argument("--backend", default="nccl", choices=["nccl", "gloo"])
    ap.add_argument("--model-dir", default="")
    ap.add_argument("--max-layers", type=int, default=4)
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--seq", type=int, default=20)
    a = ap.parse_args(argv)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if a.backend == "nccl":
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=device)
    else:
        device = torch.device("cpu")
        dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    dtype = torch.float32
    loader = HfModelLoader(a.model_dir).load_metadata() if a.model_dir else None
    cfg = loader.config() if loader else Qwen35TextConfig.tiny(layers=a.max_layers)
    if loader and 0 < a.max_layers < cfg.num_hidden_layers:
        f = {k: getattr(cfg, k) for k in cfg.__dataclass_fields__}
        f.update(num_hidden_layers=a.max_layers, layer_types=cfg.layer_types[:a.max_layers])
        cfg = Qwen35TextConfig(**f)
    g = torch.Generator().manual_seed(3)
    prompt = 8

    if a.mode == "tp":
        if world != a.tp:
            raise SystemExit("--mode tp wants exactly --tp ranks")
        ctx = build_context(world, rank, tp=a.tp, dp=1)
        tp_model = _model(cfg, loader, device, dtype, ctx=ctx)
        dense = _model(cfg, loader, device, dtype)
        ids = torch.randint(0, cfg.vocab_size, (2, a.seq), generator=g).to(device)
        with torch.no_grad():
            h_tp, h_d = tp_model.forward_hidden(ids), dense.forward_hidden(ids)
            lp_tp, lp_d = tp_model.response_logprobs(ids, prompt), dense.response_logprobs(ids, prompt)
        torch.testing.assert_close(h_tp, h_d, rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(lp_tp, lp_d, rtol=1e-4, atol=1e-4)
    elif a.mode == "dp_tp":
        dp = world // a.tp
        ctx = build_context(world, rank, tp=a.tp, dp=dp)
        model = _model(cfg, loader, device, dtype, ctx=ctx, pad_multiple=dp * 8)
        all_ids = torch.randint(0, cfg.vocab_size, (2 * dp, a.seq), generator=g).to(device)
        ids = all_ids[2 * ctx.dp_rank:2 * ctx.dp_rank + 2]
        model.response_logprobs(ids, prompt).sum().backward()
        _fold(model)
        model.sync_replicated_grads()
        mine = model.flat.main_grad.clone()
        dist.all_reduce(mine, group=ctx.dp_group)
        mine /= dp
        # the same thing on one TP group that sees every replica's batch
        ref = _model(cfg, loader, device, dtype, ctx=ctx, pad_multiple=dp * 8)
        for r in range(dp):
            (ref.response_logprobs(all_ids[2 * r:2 * r + 2], prompt).sum() / dp).backward()
        _fold(ref)
        ref.sync_replicated_grads()
        torch.testing.assert_close(mine, ref.flat.main_grad, rtol=2e-3, atol=2e-5)
    else:
        pp = world // a.tp
        if pp < 2:
            raise SystemExit("--mode pp_tp wants at least 2 * --tp ranks")
        ctx = build_context(world, rank, tp=a.tp, dp=1, pp=pp)
        topo, info = ctx.topology, ctx.rank_info
        lb, le = topo.pipeline_layer_range(cfg.num_hidden_layers, info.pipeline_rank)
        first, last = info.pipeline_rank == 0, info.pipeline_rank == pp - 1
        model = _model(cfg, None, device, dtype, ctx=ctx, layer_begin=lb, layer_end=le, first_stage=first,
                       last_stage=last, pad_multiple=8)
        opt = FlatZeroOptimizer(model.flat, AdamWOptions(lr=1e-3, use_master_weights=False), max_grad_norm=0.0)
        before = model.flat.flat.clone()
        micro, mb = 2 * pp, 1
        ids = torch.randint(0, cfg.vocab_size, (micro * mb, a.seq), generator=g).to(device)
        peers = pipeline_peers(info.pipeline_group, info.pipeline_rank)
        stage = PipelineStage(peers, info.pipeline_rank, pp, micro, (mb * a.seq, cfg.hidden_size), dtype, device)

        def fwd(m, x):
            sl = ids[m * mb:(m + 1) * mb]
            if first:
                x = model.embed(sl)
            return model.forward_layers(x, mb, a.seq, final_norm=last)

        def loss(m, out):
            l = out.float().square().mean() / micro
            return l, torch.ones_like(l)
        stage.run(fwd, loss)
        _fold(model)
        has_grad = bool(model.flat.main_grad.abs().sum() > 0)
        opt.step()
        moved = bool((model.flat.flat - before).abs().sum() > 0)
        flags = torch.tensor([float(has_grad), float(moved)], device=device)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        if flags.min() < 1:
            raise SystemExit("pp_tp smoke: a rank had no gradient or did not update")
    dist.barrier()
    if rank == 0:
        print(f"{a.mode} smoke passed (world {world})", flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
