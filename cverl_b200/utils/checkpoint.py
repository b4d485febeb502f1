"""Trainer checkpoints in the reference's on-disk layout, and resume.

``<dir>/step_%06d/rank_<g>.pt``   tensor archive.  Flat mode keys: ``flat_param_shard``, ``flat_exp_avg``,
                                  ``flat_exp_avg_sq``, ``optim_step`` (+ ``param_<i>`` when model parameters
                                  are saved too).  Non-flat mode keys: ``param_<i>`` (the fp32 master copy where
                                  one is kept), ``optim_exp_avg_<k>``, ``optim_exp_avg_sq_<k>``, ``optim_step``.
                                  The file is a TorchScript module archive whose *parameters* carry those
                                  names - the container ``torch::serialize::OutputArchive::write`` produces -
                                  so either side reads the other's files.  Written to ``.tmp`` and renamed.
``<dir>/step_%06d/rank_<g>.json`` rank coordinates, layer range, ``param_file``, ``optimizer_step``,
                                  ``optimizer_kind``, master mode, ``optimizer_param_indices``, the flat shard
                                  metadata and the per-parameter table; dtype strings are c10 names
                                  (``BFloat16``, ``Float``).
``<dir>/step_%06d/manifest.json`` written by rank 0 after a barrier once every rank file exists: ``step``,
                                  ``format`` (``cverl_pp_tp_rank_local_checkpoint_v2`` non-flat,
                                  ``..._v3`` flat with parameters, ``cverl_pp_tp_flat_shard_checkpoint_v4``
                                  flat shard only), ``complete``, ``optimizer_kind``, master mode, the parallel
                                  sizes at top level, ``training_config``, ``optimizer`` hyper-parameters and
                                  step, ``rank_files`` as objects with the rank coordinates.
``<dir>/latest_checkpoint.txt``   name of the newest complete step directory.

``step`` everywhere is the number of optimizer steps taken (the reference's zero-based loop index + 1).
Resume verifies rank coordinates, parameter order / names / shapes, shard metadata and dtype, master mode,
optimizer ownership, format and completeness, and that the manifest's optimizer step equals the archive step;
resharding to another topology is refused.  Reference: tools/model/qwen3_5_pp_tp_ppo_trainer.cc:773-1396.
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import torch

FORMAT_FLAT_SHARD = "cverl_pp_tp_flat_shard_checkpoint_v4"
FORMAT_FLAT_WITH_PARAMS = "cverl_pp_tp_rank_local_checkpoint_v3"
FORMAT_RANK_LOCAL = "cverl_pp_tp_rank_local_checkpoint_v2"

_C10_NAMES = {torch.bfloat16: "BFloat16", torch.float32: "Float", torch.float16: "Half", torch.float64: "Double",
              torch.int64: "Long", torch.int32: "Int", torch.uint8: "Byte", torch.bool: "Bool"}


def c10_dtype_name(dt: torch.dtype) -> str:
    """The string ``c10::toString(ScalarType)`` gives, which the reference writes and compares on resume."""
    return _C10_NAMES[dt]


class _Holder(torch.nn.Module):
    """Parameters named by ``tensors``; a dotted name ``a.b`` becomes parameter ``b`` of sub-module ``a``,
    which is how a nested archive is laid out."""

    def __init__(self, tensors: Dict[str, torch.Tensor]):
        super().__init__()
        nested: Dict[str, Dict[str, torch.Tensor]] = {}
        for k, v in tensors.items():
            if "." in k:
                head, rest = k.split(".", 1)
                nested.setdefault(head, {})[rest] = v
            else:
                self.register_parameter(k, torch.nn.Parameter(v.detach().cpu().contiguous(), requires_grad=False))
        for head, sub in nested.items():
            self.add_module(head, _Holder(sub))


def save_archive(path, tensors: Dict[str, torch.Tensor]) -> None:
    """Writes ``tensors`` as a module archive (tmp + rename)."""
    path = Path(path)
    tmp = path.with_suffix(path.suffix + ".tmp")
    torch.jit.save(torch.jit.script(_Holder(tensors)), str(tmp))
    os.replace(tmp, path)


def load_archive(path) -> Dict[str, torch.Tensor]:
    """Every tensor of a module archive, whether it was stored as a parameter (``OutputArchive::write``'s
    default, and this module's writer) or as a buffer."""
    mod = torch.jit.load(str(path), map_location="cpu")
    out = {k: v.detach() for k, v in mod.named_parameters()}
    out.update({k: v for k, v in mod.named_buffers()})
    return out


def step_dir_name(step: int) -> str:
    return f"step_{step:06d}"


def _rank_meta_common(global_rank: int, rank_info: dict, optimizer_step: int) -> dict:
    meta = {"global_rank": global_rank}
    for k in ("data_rank", "pipeline_rank", "context_rank", "tensor_rank", "expert_rank", "layer_begin", "layer_end"):
        if k in rank_info:
            meta[k] = rank_info[k]
    meta["param_file"] = f"rank_{global_rank}.pt"
    meta["optimizer_step"] = optimizer_step
    return meta


def _write_json_atomic(path: Path, doc: dict) -> None:
    tmp = Path(str(path) + ".tmp")
    tmp.write_text(json.dumps(doc, indent=2) + "\n")
    os.replace(tmp, path)


def save_rank_checkpoint(ckpt_dir, step: int, global_rank: int, model, optimizer, rank_info: dict,
                         save_model_params: bool = False) -> Path:
    """Flat mode: writes this rank's archive + JSON for ``step``; returns the step directory."""
    d = Path(ckpt_dir) / step_dir_name(step)
    d.mkdir(parents=True, exist_ok=True)
    sd = optimizer.state_dict()
    tensors = {}
    params = []
    named = list(model.flat.named_tensors())
    for i, (name, t) in enumerate(named):
        entry = {"index": i, "name": name, "dtype": c10_dtype_name(t.dtype), "shape": list(t.shape)}
        if save_model_params:
            tensors[f"param_{i}"] = t
            entry["checkpoint_key"] = f"param_{i}"
        params.append(entry)
    tensors.update({"flat_param_shard": sd["flat_param_shard"], "flat_exp_avg": sd["flat_exp_avg"],
                    "flat_exp_avg_sq": sd["flat_exp_avg_sq"], "optim_step": sd["optim_step"]})
    if "bucket_chunks" in sd:      # bucket-sharded ZeRO-2: the shard is a concatenation of per-bucket pieces
        tensors["bucket_chunks"] = sd["bucket_chunks"]
    save_archive(d / f"rank_{global_rank}.pt", tensors)
    meta = _rank_meta_common(global_rank, rank_info, int(sd["optim_step"]))
    meta.update({
        "optimizer_kind": "FlatAdamW",
        "use_master_weights": optimizer.adam.master is not None, "model_parameters_saved": save_model_params,
        "optimizer_param_indices": list(range(len(named))),
        "flat_parameter_shard": {"original_numel": model.flat.numel, "padded_numel": model.flat.padded_numel,
                                 "shard_begin": optimizer.begin, "shard_end": optimizer.end,
                                 "numel": optimizer.shard_numel,
                                 "dtype": c10_dtype_name(optimizer.adam.parameter_shard.dtype)},
        "parameters": params,
    })
    if "bucket_chunks" in sd:
        meta["flat_parameter_shard"]["layout"] = "bucketed"
    _write_json_atomic(d / f"rank_{global_rank}.json", meta)
    return d


def save_rank_checkpoint_v2(ckpt_dir, step: int, global_rank: int, names: Sequence[str],
                            params: Sequence[torch.Tensor], optimizer, optimizer_param_indices: Sequence[int],
                            rank_info: dict) -> Path:
    """Non-flat mode (per-tensor ``Fp32MasterAdamW``, all parameters or this rank's ZeRO-1 share):
    ``param_<i>`` for every parameter (the master copy where this rank optimises it with master weights),
    moments for the optimised ones (reference: trainer.cc:797-887)."""
    d = Path(ckpt_dir) / step_dir_name(step)
    d.mkdir(parents=True, exist_ok=True)
    pos = {p: k for k, p in enumerate(optimizer_param_indices)}
    use_master = optimizer.options.use_master_weights
    tensors, table = {}, []
    for i, (name, t) in enumerate(zip(names, params)):
        k = pos.get(i, -1)
        src = optimizer.master[k] if (use_master and k >= 0) else t
        tensors[f"param_{i}"] = src
        entry = {"index": i, "name": name, "dtype": c10_dtype_name(t.dtype), "shape": list(t.shape),
                 "checkpoint_key": f"param_{i}", "optimizer_position": k}
        if k >= 0:
            entry["optimizer_exp_avg_key"] = f"optim_exp_avg_{k}"
            entry["optimizer_exp_avg_sq_key"] = f"optim_exp_avg_sq_{k}"
        table.append(entry)
    for k in range(len(optimizer_param_indices)):
        tensors[f"optim_exp_avg_{k}"] = optimizer.exp_avg[k]
        tensors[f"optim_exp_avg_sq_{k}"] = optimizer.exp_avg_sq[k]
    tensors["optim_step"] = torch.tensor(optimizer.step_count, dtype=torch.int64)
    save_archive(d / f"rank_{global_rank}.pt", tensors)
    meta = _rank_meta_common(global_rank, rank_info, optimizer.step_count)
    meta.update({"use_master_weights": use_master, "optimizer_param_indices": list(optimizer_param_indices),
                 "parameters": table})
    _write_json_atomic(d / f"rank_{global_rank}.json", meta)
    return d


def rank_coordinates(rank: int, dims: dict) -> dict:
    """Coordinates of a global rank in the rank-file table (EP innermost, then TP, CP, PP, DP)."""
    ep, tp, cp, pp = dims.get("ep", 1), dims.get("tp", 1), dims.get("cp", 1), dims.get("pp", 1)
    r = rank
    out = {"global_rank": rank}
    out["expert_rank"], r = r % ep, r // ep
    out["tensor_rank"], r = r % tp, r // tp
    out["context_rank"], r = r % cp, r // cp
    out["pipeline_rank"], r = r % pp, r // pp
    out["data_rank"] = r
    return out


def write_manifest(ckpt_dir, step: int, world: int, dims: dict, training_config: dict, optimizer_config: dict,
                   with_params: bool = False, optimizer_step: Optional[int] = None, flat: bool = True,
                   use_master_weights: bool = False) -> bool:
    """Rank 0, after a barrier: writes the manifest and ``latest_checkpoint.txt`` when every rank file exists."""
    d = Path(ckpt_dir) / step_dir_name(step)
    rank_files = []
    for r in range(world):
        pf, mf = f"rank_{r}.pt", f"rank_{r}.json"
        if not ((d / pf).exists() and (d / mf).exists()):
            return False
        rank_files.append(dict(rank_coordinates(r, dims), param_file=pf, metadata_file=mf))
    if flat:
        fmt, kind = (FORMAT_FLAT_WITH_PARAMS if with_params else FORMAT_FLAT_SHARD), "FlatAdamW"
    else:
        fmt, kind = FORMAT_RANK_LOCAL, "Fp32MasterAdamW"
    manifest = {"step": step, "format": fmt, "complete": True}
    if flat:
        manifest.update({"optimizer_kind": kind, "model_parameters_saved": with_params})
    manifest.update({
        "use_master_weights": use_master_weights, "world_size": world,
        "data_parallel": dims.get("dp", 1), "pipeline_parallel": dims.get("pp", 1),
        "context_parallel": dims.get("cp", 1), "tensor_parallel": dims.get("tp", 1),
        "expert_parallel": dims.get("ep", 1), "sequence_parallel": dims.get("sp", 1),
        "training_config": training_config,
        "optimizer": dict({"type": kind}, **optimizer_config, step=step if optimizer_step is None else optimizer_step),
        "rank_files": rank_files})
    _write_json_atomic(d / "manifest.json", manifest)
    tmp = Path(ckpt_dir) / "latest_checkpoint.txt.tmp"
    tmp.write_text(step_dir_name(step) + "\n")
    os.replace(tmp, Path(ckpt_dir) / "latest_checkpoint.txt")
    return True


def resolve_checkpoint_dir(path, global_rank: int = 0) -> Path:
    """Accepts a checkpoint root (follows ``latest_checkpoint.txt``) or a step directory."""
    p = Path(path)
    if (p / f"rank_{global_rank}.json").exists() or (p / "manifest.json").exists():
        return p
    latest = p / "latest_checkpoint.txt"
    if latest.exists():
        name = latest.read_text().strip()
        if not name:
            raise RuntimeError("latest_checkpoint.txt is empty")
        return p / name
    raise FileNotFoundError(f"no checkpoint under {p}")


def _check_rank_meta(meta: dict, global_rank: int, rank_info: dict) -> None:
    if meta.get("global_rank", global_rank) != global_rank:
        raise RuntimeError("checkpoint topology mismatch on 'global_rank'")
    for k, v in rank_info.items():
        if k in meta and meta[k] != v:
            raise RuntimeError(f"checkpoint topology mismatch on '{k}': saved {meta[k]!r}, running {v!r}")


def _check_param_table(meta: dict, names_shapes) -> None:
    saved = meta["parameters"]
    if len(saved) != len(names_shapes):
        raise RuntimeError("checkpoint parameter order / names / shapes do not match this model (count)")
    for i, ((name, shape), e) in enumerate(zip(names_shapes, saved)):
        if e["index"] != i or e["name"] != name or list(e["shape"]) != list(shape):
            raise RuntimeError(f"checkpoint parameter order / names / shapes do not match this model at index {i}")


def _manifest_step(d: Path, formats, meta: dict, kind: Optional[str]) -> (int, Optional[dict]):
    step = int(meta.get("optimizer_step", 0))
    manifest = None
    if (d / "manifest.json").exists():
        manifest = json.loads((d / "manifest.json").read_text())
        if manifest.get("format") not in formats or (kind is not None and manifest.get("optimizer_kind") != kind):
            raise RuntimeError("checkpoint is incomplete or has an unsupported format")
        if not manifest.get("complete", False):
            raise RuntimeError("checkpoint is incomplete: manifest is not marked complete")
        step = int(manifest["optimizer"]["step"])
    return step, manifest


def load_rank_checkpoint(path, global_rank: int, model, optimizer, rank_info: dict) -> int:
    """Flat mode: restores this rank's optimizer shard (and the parameters when they were saved); the caller
    then all-gathers the parameters.  Returns the optimizer step."""
    d = resolve_checkpoint_dir(path, global_rank)
    meta_path = d / f"rank_{global_rank}.json"
    if not meta_path.exists():
        raise FileNotFoundError(f"resume checkpoint missing rank metadata: {meta_path}")
    meta = json.loads(meta_path.read_text())
    _check_rank_meta(meta, global_rank, rank_info)
    if meta.get("optimizer_kind") != "FlatAdamW":
        raise RuntimeError("checkpoint was not written by the flat sharded optimizer")
    named = list(model.flat.named_tensors())
    _check_param_table(meta, [(n, t.shape) for n, t in named])
    fs = meta["flat_parameter_shard"]
    want = (model.flat.numel, model.flat.padded_numel, optimizer.begin, optimizer.end, optimizer.shard_numel)
    got = (fs["original_numel"], fs["padded_numel"], fs["shard_begin"], fs["shard_end"], fs["numel"])
    if want != got:
        raise RuntimeError(f"checkpoint flat shard metadata mismatch: saved {got}, running {want}")
    if "dtype" in fs and fs["dtype"] != c10_dtype_name(optimizer.adam.parameter_shard.dtype):
        raise RuntimeError("checkpoint flat shard dtype mismatch")
    if "use_master_weights" in meta and meta["use_master_weights"] != (optimizer.adam.master is not None):
        raise RuntimeError("checkpoint master-weight mode differs from this run")
    manifest_step, manifest = _manifest_step(d, (FORMAT_FLAT_SHARD, FORMAT_FLAT_WITH_PARAMS), meta, "FlatAdamW")
    params_saved = meta.get("model_parameters_saved", True)
    if manifest is not None:
        if "use_master_weights" in manifest and manifest["use_master_weights"] != (optimizer.adam.master is not None):
            raise RuntimeError("checkpoint manifest master-weight mode differs from this run")
        params_saved = manifest.get("model_parameters_saved", manifest["format"] == FORMAT_FLAT_WITH_PARAMS)
    arch = load_archive(d / meta.get("param_file", f"rank_{global_rank}.pt"))
    step = int(arch["optim_step"])
    if step != manifest_step:
        raise RuntimeError("manifest step does not match the archive step")
    if params_saved:
        with torch.no_grad():
            for i, (_, t) in enumerate(named):
                t.copy_(arch[f"param_{i}"].to(t.device, t.dtype))
    optimizer.load_state_dict(arch)
    return step


def load_rank_checkpoint_v2(path, global_rank: int, names: Sequence[str], params: Sequence[torch.Tensor], optimizer,
                            optimizer_param_indices: Sequence[int], rank_info: dict) -> int:
    """Non-flat mode: restores every parameter, and the master copies / moments of the ones this rank
    optimises (reference: trainer.cc:1155-1272)."""
    d = resolve_checkpoint_dir(path, global_rank)
    meta = json.loads((d / f"rank_{global_rank}.json").read_text())
    _check_rank_meta(meta, global_rank, rank_info)
    _check_param_table(meta, [(n, t.shape) for n, t in zip(names, params)])
    saved_idx = meta.get("optimizer_param_indices", list(range(len(params))))
    if list(saved_idx) != list(optimizer_param_indices):
        raise RuntimeError("checkpoint optimizer shard assignment mismatch")
    manifest_step, _ = _manifest_step(d, (FORMAT_RANK_LOCAL,), meta, None)
    arch = load_archive(d / meta.get("param_file", f"rank_{global_rank}.pt"))
    step = int(arch["optim_step"])
    if step != manifest_step:
        raise RuntimeError("manifest step does not match the archive step")
    with torch.no_grad():
        for i, t in enumerate(params):
            t.copy_(arch[f"param_{i}"].to(t.device, t.dtype))
    ck_params = [arch[f"param_{i}"] for i in optimizer_param_indices]
    m = [arch[f"optim_exp_avg_{k}"] for k in range(len(optimizer_param_indices))]
    v = [arch[f"optim_exp_avg_sq_{k}"] for k in range(len(optimizer_param_indices))]
    optimizer.load_state(ck_params, m, v, step)
    return step
