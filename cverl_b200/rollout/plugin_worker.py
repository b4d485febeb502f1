"""``DynamicRolloutWorker``: a rollout worker loaded from a shared object at run time.

The plugin exports ``cverl_create_rollout_worker(const char* config_json)`` and
``cverl_destroy_rollout_worker`` (csrc/include/cverl/rollout_plugin.h); the native loader
(csrc/plugin_loader.cc) opens it with RTLD_NOW | RTLD_LOCAL and forwards both calls.
Reference: src/rollout/plugin_worker.cc:11-64.
"""
from __future__ import annotations

import ctypes as C
from typing import List

import torch

from .. import _native as nv
from ..parallel.weight_sync import ParameterView
from .worker import GenerationConfig, GenerationOutput, RolloutWorker, TokenBatch


class _GenCfg(C.Structure):
    _fields_ = [("max_new_tokens", C.c_int64), ("temperature", C.c_double), ("top_p", C.c_double),
                ("top_k", C.c_int64), ("eos_token_id", C.c_int64), ("eos_check_interval", C.c_int64),
                ("seed", C.c_uint64)]


class _GenArgs(C.Structure):
    _fields_ = [("token_ids", C.c_void_p), ("attention_mask", C.c_void_p), ("lengths", C.c_void_p),
                ("batch", C.c_int64), ("prompt_len", C.c_int64), ("config", _GenCfg),
                ("out_token_ids", C.c_void_p), ("out_logprobs", C.c_void_p), ("out_lengths", C.c_void_p)]


class _ParamView(C.Structure):
    _fields_ = [("name", C.c_char_p), ("data", C.c_void_p), ("dtype", C.c_int32), ("device", C.c_int32),
                ("ndim", C.c_int32), ("shape", C.c_int64 * 8)]


_DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def _lib():
    lib = nv.host()
    if not getattr(lib, "_plugin_bound", False):
        lib.cverl_plugin_load.restype = C.c_void_p
        lib.cverl_plugin_load.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, C.c_int]
        lib.cverl_plugin_generate.argtypes = [C.c_void_p, C.POINTER(_GenArgs)]
        lib.cverl_plugin_num_parameters.restype = C.c_int64
        lib.cverl_plugin_num_parameters.argtypes = [C.c_void_p]
        lib.cverl_plugin_parameter.argtypes = [C.c_void_p, C.c_int64, C.POINTER(_ParamView)]
        lib.cverl_plugin_unload.argtypes = [C.c_void_p]
        lib._plugin_bound = True
    return lib


class DynamicRolloutWorker(RolloutWorker):
    def __init__(self, path: str, config_json: str = "{}"):
        self._lib = _lib()
        err = C.create_string_buffer(512)
        self._h = self._lib.cverl_plugin_load(str(path).encode(), config_json.encode(), err, 512)
        if not self._h:
            raise RuntimeError(f"load_rollout_worker_plugin: {err.value.decode()}")

    def generate(self, batch: TokenBatch, config: GenerationConfig) -> GenerationOutput:
        ids = batch.token_ids.to("cpu", torch.int64).contiguous()
        mask = (batch.attention_mask if batch.attention_mask is not None
                else torch.ones_like(ids)).to("cpu", torch.int64).contiguous()
        lens = (batch.lengths if batch.lengths is not None
                else mask.sum(-1)).to("cpu", torch.int64).contiguous()
        B, P = ids.shape
        N = config.max_new_tokens
        out_ids = torch.zeros((B, N), dtype=torch.int64)
        out_lp = torch.zeros((B, N), dtype=torch.float32)
        out_len = torch.zeros(B, dtype=torch.int64)
        args = _GenArgs(ids.data_ptr(), mask.data_ptr(), lens.data_ptr(), B, P,
                        _GenCfg(N, config.temperature, config.top_p, config.top_k, config.eos_token_id,
                                config.eos_check_interval, config.seed),
                        out_ids.data_ptr(), out_lp.data_ptr(), out_len.data_ptr())
        rc = self._lib.cverl_plugin_generate(self._h, C.byref(args))
        if rc != 0:
            raise RuntimeError(f"plugin generate failed with code {rc}")
        dev = batch.token_ids.device
        return GenerationOutput(out_ids.to(dev), out_lp.to(dev), out_len.to(dev))

    def actor_parameters(self) -> List[ParameterView]:
        out = []
        for i in range(self._lib.cverl_plugin_num_parameters(self._h)):
            pv = _ParamView()
            if self._lib.cverl_plugin_parameter(self._h, i, C.byref(pv)) != 0:
                raise RuntimeError("plugin parameter query failed")
            if pv.device != 0:
                raise NotImplementedError("device-resident plugin parameters are exposed through CUDA IPC handles")
            shape = tuple(pv.shape[:pv.ndim])
            numel = 1
            for s in shape:
                numel *= s
            dt = _DTYPES[pv.dtype]
            nbytes = numel * torch.empty((), dtype=dt).element_size()
            buf = (C.c_ubyte * nbytes).from_address(pv.data)
            t = torch.frombuffer(buf, dtype=dt, count=numel).view(shape)  # aliases the plugin's memory
            out.append(ParameterView(pv.name.decode(), t))
        return out

    def close(self):
        if self._h:
            self._lib.cverl_plugin_unload(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def load_rollout_worker_plugin(path: str, config_json: str = "{}") -> DynamicRolloutWorker:
    return DynamicRolloutWorker(path, config_json)
