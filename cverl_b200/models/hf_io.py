"""Hugging Face model-directory IO on the native safetensors reader / writer.

``HfModelLoader`` indexes every ``*.safetensors`` shard of a directory and reads
tensors on demand (reference: src/model/hf_model_loader.cc:246-373);
``write_safetensors`` emits one file in the ``format: pt`` layout
(src/model/safetensors_writer.cc:92-159); ``save_hf_checkpoint`` copies the
non-weight files of a source model directory and writes a single
``model.safetensors`` (src/torch/qwen3_5_causal_lm_policy.cc:131-175);
``synthesize_model_dir`` writes a random-init model directory, which the
benchmarks and tests use in place of downloaded weights.
"""
from __future__ import annotations

import ctypes as C
import json
import shutil
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .. import _native as nv
from .config import Qwen35TextConfig

_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.int64, torch.int32, torch.uint8]
_DTYPE_NAMES = ["F32", "F16", "BF16", "I64", "I32", "U8"]


def _lib():
    lib = nv.host()
    if not getattr(lib, "_st_bound", False):
        lib.cverl_st_open.restype = C.c_void_p
        lib.cverl_st_open.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
        lib.cverl_st_close.argtypes = [C.c_void_p]
        lib.cverl_st_count.restype = C.c_int64
        lib.cverl_st_count.argtypes = [C.c_void_p]
        lib.cverl_st_name.restype = C.c_char_p
        lib.cverl_st_name.argtypes = [C.c_void_p, C.c_int64]
        lib.cverl_st_info.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_int), C.POINTER(C.c_int),
                                      C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
        lib.cverl_st_read.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_int64]
        lib.cverl_st_read_range.argtypes = [C.c_void_p, C.c_char_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int]
        lib.cverl_st_write.argtypes = [C.c_char_p, C.c_int64, C.POINTER(C.c_char_p), C.POINTER(C.c_int),
                                       C.POINTER(C.c_int), C.POINTER(C.c_int64), C.POINTER(C.c_void_p)]
        lib._st_bound = True
    return lib


class SafetensorInfo:
    def __init__(self, name: str, dtype: torch.dtype, shape: Tuple[int, ...], nbytes: int):
        self.name, self.dtype, self.shape, self.nbytes = name, dtype, shape, nbytes

    def __repr__(self):
        return f"SafetensorInfo({self.name!r}, {self.dtype}, {self.shape})"


class HfModelLoader:
    """Index of a model directory (or one ``.safetensors`` file) with on-demand tensor reads."""

    def __init__(self, model_dir):
        self.model_dir = str(model_dir)
        self._h = None
        self._infos: Dict[str, SafetensorInfo] = {}
        self.bytes_read = 0            # tensor bytes read through this loader

    def load_metadata(self) -> "HfModelLoader":
        if self._h is not None:
            return self
        lib = _lib()
        err = C.create_string_buffer(512)
        h = lib.cverl_st_open(self.model_dir.encode(), err, 512)
        if not h:
            raise RuntimeError(f"HfModelLoader: {err.value.decode()}")
        self._h = h
        for i in range(lib.cverl_st_count(h)):
            name = lib.cverl_st_name(h, i).decode()
            dt, nd, nb = C.c_int(), C.c_int(), C.c_int64()
            shape = (C.c_int64 * 8)()
            rc = lib.cverl_st_info(h, name.encode(), C.byref(dt), C.byref(nd), shape, C.byref(nb))
            if rc != 0:
                raise RuntimeError(f"HfModelLoader: unsupported tensor {name} (code {rc})")
            self._infos[name] = SafetensorInfo(name, _DTYPES[dt.value], tuple(shape[:nd.value]), nb.value)
        return self

    def names(self) -> List[str]:
        self.load_metadata()
        return list(self._infos)

    def info(self, name: str) -> SafetensorInfo:
        self.load_metadata()
        return self._infos[name]

    def has(self, name: str) -> bool:
        self.load_metadata()
        return name in self._infos

    def load_tensor(self, name: str) -> torch.Tensor:
        """Reads one tensor into a fresh CPU tensor of its stored dtype."""
        self.load_metadata()
        inf = self._infos.get(name)
        if inf is None:
            raise KeyError(f"tensor {name} not found in {self.model_dir}")
        out = torch.empty(inf.shape, dtype=inf.dtype)
        if inf.nbytes:
            rc = _lib().cverl_st_read(self._h, name.encode(), out.data_ptr(), inf.nbytes)
            if rc != 0:
                raise RuntimeError(f"HfModelLoader: read of {name} failed (code {rc})")
            self.bytes_read += inf.nbytes
        return out

    def load_rows(self, name: str, begin: int, end: int, threads: int = 0) -> torch.Tensor:
        """Rows ``[begin, end)`` of a tensor along its first dimension, reading only their bytes (rows of a
        row-major tensor are one contiguous range of the file)."""
        self.load_metadata()
        inf = self._infos.get(name)
        if inf is None:
            raise KeyError(f"tensor {name} not found in {self.model_dir}")
        if not inf.shape or not (0 <= begin <= end <= inf.shape[0]):
            raise ValueError(f"load_rows: rows [{begin}, {end}) out of range for {name} of shape {inf.shape}")
        row_bytes = inf.nbytes // inf.shape[0] if inf.shape[0] else 0
        out = torch.empty((end - begin, *inf.shape[1:]), dtype=inf.dtype)
        nbytes = (end - begin) * row_bytes
        if nbytes:
            rc = _lib().cverl_st_read_range(self._h, name.encode(), begin * row_bytes, nbytes, out.data_ptr(), threads)
            if rc != 0:
                raise RuntimeError(f"HfModelLoader: read of rows of {name} failed (code {rc})")
            self.bytes_read += nbytes
        return out

    def config(self) -> Qwen35TextConfig:
        return Qwen35TextConfig.from_model_dir(self.model_dir)

    def close(self):
        if self._h is not None:
            _lib().cverl_st_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def write_safetensors(path, tensors: Dict[str, torch.Tensor], dtype: Optional[torch.dtype] = None) -> None:
    """Single-file writer; tensors are cast to ``dtype`` (when given and floating) on the CPU."""
    names = list(tensors)
    cpu: List[torch.Tensor] = []
    for n in names:
        t = tensors[n].detach()
        if dtype is not None and t.is_floating_point():
            t = t.to(dtype)
        cpu.append(t.cpu().contiguous())
    n = len(names)
    c_names = (C.c_char_p * n)(*[s.encode() for s in names])
    c_dt = (C.c_int * n)(*[_DTYPES.index(t.dtype) for t in cpu])
    c_nd = (C.c_int * n)(*[t.dim() for t in cpu])
    flat_shapes = [int(s) for t in cpu for s in t.shape]
    c_sh = (C.c_int64 * max(1, len(flat_shapes)))(*flat_shapes)
    c_ptr = (C.c_void_p * n)(*[t.data_ptr() for t in cpu])
    rc = _lib().cverl_st_write(str(path).encode(), n, c_names, c_dt, c_nd, c_sh, c_ptr)
    if rc != 0:
        raise RuntimeError(f"write_safetensors failed with code {rc}")


def load_model_weights(model, loader: HfModelLoader) -> None:
    """Fills a ``Qwen35Model`` (this rank's shards) from a model directory."""
    loader.load_metadata()
    ctx = model.ctx
    for spec in model.specs:
        if not loader.has(spec.name):
            raise KeyError(f"model directory lacks required weight {spec.name}")
        if not model.holds(spec):
            continue                   # another expert-parallel rank's expert: not read at all
        if spec.tp is not None and ctx.tp_size > 1 and spec.tp[0] == "rows":
            # row-sharded: read this rank's rows of every section only (1 / tp of the tensor's bytes)
            pieces, begin = [], 0
            for section in spec.tp[1]:
                if section % ctx.tp_size:
                    raise ValueError(f"{spec.name}={section} is not divisible by tensor-parallel size {ctx.tp_size}")
                step = section // ctx.tp_size
                pieces.append(loader.load_rows(spec.name, begin + ctx.tp_rank * step, begin + (ctx.tp_rank + 1) * step))
                begin += section
            model.load_local_tensor(spec.name, pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=0))
        else:
            model.load_full_tensor(spec.name, loader.load_tensor(spec.name))


def save_hf_checkpoint(model, out_dir, source_dir=None, dtype: Optional[torch.dtype] = None) -> None:
    """Hugging Face export: non-weight files of ``source_dir`` + one ``model.safetensors``.

    ``model`` must hold full (unsharded) tensors, i.e. tensor-parallel size 1; sharded
    trainers gather through ``cverl_b200.utils.checkpoint.gather_full_state`` first.
    """
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    if source_dir is not None:
        for f in Path(source_dir).iterdir():
            if f.is_file() and not f.name.endswith(".safetensors") and f.name != "model.safetensors.index.json":
                shutil.copy2(f, out / f.name)
    if not (out / "config.json").exists():
        (out / "config.json").write_text(json.dumps(model.cfg.to_hf_config(), indent=1))
    tensors = {name: t for name, t in model.local_hf_tensors()}
    write_safetensors(out / "model.safetensors", tensors, dtype or model.dtype)


def synthesize_model_dir(cfg: Qwen35TextConfig, out_dir, seed: int = 1234, dtype=torch.bfloat16) -> Path:
    """Random-init model directory in the reference's naming scheme (config.json + model.safetensors)."""
    from .qwen3_5 import Qwen35Model
    model = Qwen35Model(cfg, dtype=dtype, with_main_grad=False)
    model.init_weights(seed=seed)
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text(json.dumps(cfg.to_hf_config(), indent=1))
    save_hf_checkpoint(model, out, None, dtype)
    return out
