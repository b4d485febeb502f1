"""CUDA-IPC tensor hand-off between processes on one node.

``GpuIpcTensorHandle`` carries ``{kind, dtype, device, ndim, sizes[4], strides[4], offset,
numel, 64-byte cudaIpcMemHandle}`` and serialises to hex for JSON manifests; ``export`` takes
the handle of a live CUDA tensor, ``import`` maps it in another process as a tensor that
aliases the exporter's memory and unmaps on release.
Reference: src/rollout/gpu_ipc_rollout_batch.cc:30-139.
"""
from __future__ import annotations

import ctypes as C
import json
from dataclasses import asdict, dataclass, field
from typing import Dict, List

import torch

from .. import _native as nv

TENSOR_KINDS = ("prompt_ids", "response_ids", "response_mask", "old_log_probs", "rewards", "advantages",
                "group_ids", "ref_log_probs")
_DTYPE_NAMES = {torch.float32: "float32", torch.float16: "float16", torch.bfloat16: "bfloat16",
                torch.int64: "int64", torch.int32: "int32", torch.uint8: "uint8"}
_NAME_DTYPES = {v: k for k, v in _DTYPE_NAMES.items()}
_TYPESTR = {torch.float32: "<f4", torch.float16: "<f2", torch.bfloat16: "<u2", torch.int64: "<i8",
            torch.int32: "<i4", torch.uint8: "|u1"}


@dataclass
class GpuIpcTensorHandle:
    kind: str
    dtype: str
    device: int
    ndim: int
    sizes: List[int]
    strides: List[int]
    offset: int          # byte offset of the tensor inside the exported allocation
    numel: int
    handle_hex: str      # 64-byte cudaIpcMemHandle as 128 hex characters

    def to_json(self) -> str:
        return json.dumps(asdict(self))

    @classmethod
    def from_json(cls, text: str) -> "GpuIpcTensorHandle":
        d = json.loads(text)
        h = cls(**d)
        if len(h.handle_hex) != 128 or h.ndim > 4 or len(h.sizes) != h.ndim or len(h.strides) != h.ndim:
            raise ValueError("malformed GpuIpcTensorHandle")
        bytes.fromhex(h.handle_hex)
        return h


def export_gpu_tensor(kind: str, t: torch.Tensor) -> GpuIpcTensorHandle:
    if not t.is_cuda:
        raise ValueError("export_gpu_tensor needs a CUDA tensor")
    if t.dim() > 4 or t.dtype not in _DTYPE_NAMES:
        raise ValueError("unsupported tensor for IPC export")
    raw = (C.c_ubyte * 64)()
    off = C.c_longlong()
    with torch.cuda.device(t.device):
        nv.check(nv.cuda().cvb_ipc_get_handle(t.data_ptr(), C.addressof(raw), C.addressof(off)), "cudaIpcGetMemHandle")
    return GpuIpcTensorHandle(kind, _DTYPE_NAMES[t.dtype], t.device.index or 0, t.dim(), list(t.shape),
                              list(t.stride()), off.value, t.numel(), bytes(raw).hex())


class _Mapped:
    """Owns one opened IPC mapping and exposes it through the CUDA array interface."""

    def __init__(self, h: GpuIpcTensorHandle):
        self.handle = h
        raw = (C.c_ubyte * 64).from_buffer_copy(bytes.fromhex(h.handle_hex))
        base = C.c_void_p()
        with torch.cuda.device(h.device):
            nv.check(nv.cuda().cvb_ipc_open_handle(C.addressof(raw), C.addressof(base)), "cudaIpcOpenMemHandle")
        self.base = base.value
        dt = _NAME_DTYPES[h.dtype]
        esz = torch.empty((), dtype=dt).element_size()
        self.__cuda_array_interface__ = {
            "shape": tuple(h.sizes), "typestr": _TYPESTR[dt], "data": (self.base + h.offset, False), "version": 3,
            "strides": tuple(s * esz for s in h.strides) if h.ndim else None,
        }

    def __del__(self):
        try:
            if self.base:
                nv.cuda().cvb_ipc_close_handle(self.base)
                self.base = None
        except Exception:
            pass


def import_gpu_tensor(h: GpuIpcTensorHandle) -> torch.Tensor:
    """Maps the exporter's memory; the tensor keeps the mapping alive until it is released."""
    m = _Mapped(h)
    t = torch.as_tensor(m, device=torch.device("cuda", h.device))
    dt = _NAME_DTYPES[h.dtype]
    if dt == torch.bfloat16:
        t = t.view(torch.bfloat16)
    t._cverl_ipc_owner = m
    return t


def export_batch(tensors: Dict[str, torch.Tensor]) -> str:
    """JSON manifest of a rollout batch (one handle per tensor kind)."""
    for k in tensors:
        if k not in TENSOR_KINDS:
            raise ValueError(f"unknown rollout tensor kind {k}")
    return json.dumps({"tensors": [asdict(export_gpu_tensor(k, t)) for k, t in tensors.items()]})


def import_batch(manifest: str) -> Dict[str, torch.Tensor]:
    d = json.loads(manifest)
    return {e["kind"]: import_gpu_tensor(GpuIpcTensorHandle(**e)) for e in d["tensors"]}
