"""Trainer checkpoints in the reference's on-disk layout, and resume.

``<dir>/step_%06d/rank_<g>.pt``   tensor archive.  Flat mode keys: ``flat_param_shard``,
                                  ``flat_exp_avg``, ``flat_exp_avg_sq``, ``optim_step`` (+ ``param_<i>``
                                  when model parameters are saved too).  The file is a TorchScript
                                  module archive whose buffers carry those names, which is the container
                                  ``torch::serialize::OutputArchive`` writes, so either side can read the
                                  other's files.  Written to ``.tmp`` and renamed.
``<dir>/step_%06d/rank_<g>.json`` rank coordinates, layer range, optimizer kind, master mode, the flat shard
                                  metadata and the per-parameter table.
``<dir>/step_%06d/manifest.json`` written by rank 0 after a barrier once every rank file exists: format tag
                                  (``cverl_pp_tp_flat_shard_checkpoint_v4`` for shard-only flat checkpoints,
                                  ``..._rank_local_checkpoint_v3`` with parameters), ``complete: true``,
                                  parallel dims, training config, optimizer hyper-parameters and step,
                                  the rank file list.
``<dir>/latest_checkpoint.txt``   name of the newest complete step directory.

Resume verifies rank coordinates, parameter order / names / shapes, shard metadata and dtype, master mode,
format and completeness, and that the manifest step equals the archive step; resharding to another topology
is refused.  Reference: tools/model/qwen3_5_pp_tp_ppo_trainer.cc:773-1396.
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Dict, List, Optional

import torch

FORMAT_FLAT_SHARD = "cverl_pp_tp_flat_shard_checkpoint_v4"
FORMAT_FLAT_WITH_PARAMS = "cverl_pp_tp_rank_local_checkpoint_v3"
FORMAT_RANK_LOCAL = "cverl_pp_tp_rank_local_checkpoint_v2"


class _Holder(torch.nn.Module):
    """Buffers named by ``tensors``; a dotted name ``a.b`` becomes buffer ``b`` of sub-module ``a``, which
    is how a nested archive is laid out."""

    def __init__(self, tensors: Dict[str, torch.Tensor]):
        super().__init__()
        nested: Dict[str, Dict[str, torch.Tensor]] = {}
        for k, v in tensors.items():
            if "." in k:
                head, rest = k.split(".", 1)
                nested.setdefault(head, {})[rest] = v
            else:
                self.register_buffer(k, v.detach().cpu().contiguous())
        for head, sub in nested.items():
            self.add_module(head, _Holder(sub))


def save_archive(path, tensors: Dict[str, torch.Tensor]) -> None:
    """Writes ``tensors`` as a module archive (tmp + rename)."""
    path = Path(path)
    tmp = path.with_suffix(path.suffix + ".tmp")
    torch.jit.save(torch.jit.script(_Holder(tensors)), str(tmp))
    os.replace(tmp, path)


def load_archive(path) -> Dict[str, torch.Tensor]:
    mod = torch.jit.load(str(path), map_location="cpu")
    return {k: v for k, v in mod.named_buffers()}


def step_dir_name(step: int) -> str:
    return f"step_{step:06d}"


def _dtype_name(dt: torch.dtype) -> str:
    return str(dt).replace("torch.", "")


def save_rank_checkpoint(ckpt_dir, step: int, global_rank: int, model, optimizer, rank_info: dict,
                         save_model_params: bool = False) -> Path:
    """Writes this rank's archive + JSON for ``step``; returns the step directory."""
    d = Path(ckpt_dir) / step_dir_name(step)
    d.mkdir(parents=True, exist_ok=True)
    sd = optimizer.state_dict()
    tensors = {"flat_param_shard": sd["flat_param_shard"], "flat_exp_avg": sd["flat_exp_avg"],
               "flat_exp_avg_sq": sd["flat_exp_avg_sq"], "optim_step": sd["optim_step"]}
    params = []
    for i, (name, t) in enumerate(model.flat.named_tensors()):
        entry = {"index": i, "name": name, "dtype": _dtype_name(t.dtype), "shape": list(t.shape)}
        if save_model_params:
            tensors[f"param_{i}"] = t
            entry["checkpoint_key"] = f"param_{i}"
        params.append(entry)
    save_archive(d / f"rank_{global_rank}.pt", tensors)
    meta = dict(rank_info)
    meta.update({
        "global_rank": global_rank, "step": step, "optimizer_kind": "flat_adamw",
        "use_master_weights": optimizer.adam.master is not None, "model_parameters_saved": save_model_params,
        "flat_parameter_shard": {"original_numel": model.flat.numel, "padded_numel": model.flat.padded_numel,
                                 "shard_begin": optimizer.begin, "shard_end": optimizer.end,
                                 "numel": optimizer.shard_numel,
                                 "dtype": _dtype_name(optimizer.adam.parameter_shard.dtype)},
        "parameters": params,
    })
    tmp = d / f"rank_{global_rank}.json.tmp"
    tmp.write_text(json.dumps(meta, indent=1))
    os.replace(tmp, d / f"rank_{global_rank}.json")
    return d


def write_manifest(ckpt_dir, step: int, world: int, dims: dict, training_config: dict, optimizer_config: dict,
                   with_params: bool = False) -> bool:
    """Rank 0, after a barrier: writes the manifest and ``latest_checkpoint.txt`` when every rank file exists."""
    d = Path(ckpt_dir) / step_dir_name(step)
    files = [f"rank_{r}.pt" for r in range(world)]
    if not all((d / f).exists() and (d / f.replace(".pt", ".json")).exists() for f in files):
        return False
    manifest = {"format": FORMAT_FLAT_WITH_PARAMS if with_params else FORMAT_FLAT_SHARD, "complete": True,
                "step": step, "world_size": world, "parallel_dims": dims, "training_config": training_config,
                "optimizer": dict(optimizer_config, step=step), "rank_files": files}
    tmp = d / "manifest.json.tmp"
    tmp.write_text(json.dumps(manifest, indent=1))
    os.replace(tmp, d / "manifest.json")
    tmp = Path(ckpt_dir) / "latest_checkpoint.txt.tmp"
    tmp.write_text(step_dir_name(step))
    os.replace(tmp, Path(ckpt_dir) / "latest_checkpoint.txt")
    return True


def resolve_checkpoint_dir(path) -> Path:
    """Accepts a checkpoint root (follows ``latest_checkpoint.txt``) or a step directory."""
    p = Path(path)
    if (p / "manifest.json").exists():
        return p
    latest = p / "latest_checkpoint.txt"
    if latest.exists():
        return p / latest.read_text().strip()
    raise FileNotFoundError(f"no checkpoint under {p}")


def load_rank_checkpoint(path, global_rank: int, model, optimizer, rank_info: dict) -> int:
    """Restores this rank's optimizer shard; the caller then all-gathers the parameters. Returns the step."""
    d = resolve_checkpoint_dir(path)
    manifest = json.loads((d / "manifest.json").read_text())
    if not manifest.get("complete") or manifest.get("format") not in (FORMAT_FLAT_SHARD, FORMAT_FLAT_WITH_PARAMS):
        raise RuntimeError("checkpoint is incomplete or has an unsupported format")
    meta = json.loads((d / f"rank_{global_rank}.json").read_text())
    for k, v in rank_info.items():
        if meta.get(k) != v:
            raise RuntimeError(f"checkpoint topology mismatch on '{k}': saved {meta.get(k)!r}, running {v!r}")
    names = [(n, list(t.shape)) for n, t in model.flat.named_tensors()]
    saved = [(e["name"], e["shape"]) for e in meta["parameters"]]
    if names != saved:
        raise RuntimeError("checkpoint parameter order / names / shapes do not match this model")
    fs = meta["flat_parameter_shard"]
    want = (model.flat.numel, model.flat.padded_numel, optimizer.begin, optimizer.end, optimizer.shard_numel,
            _dtype_name(optimizer.adam.parameter_shard.dtype))
    got = (fs["original_numel"], fs["padded_numel"], fs["shard_begin"], fs["shard_end"], fs["numel"], fs["dtype"])
    if want != got:
        raise RuntimeError(f"checkpoint flat shard metadata mismatch: saved {got}, running {want}")
    if meta["use_master_weights"] != (optimizer.adam.master is not None):
        raise RuntimeError("checkpoint master-weight mode differs from this run")
    arch = load_archive(d / f"rank_{global_rank}.pt")
    step = int(arch["optim_step"])
    if step != manifest["step"] or step != meta["step"]:
        raise RuntimeError("manifest step does not match the archive step")
    optimizer.load_state_dict(arch)
    return step
