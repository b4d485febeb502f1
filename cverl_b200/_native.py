"""ctypes bindings of the two in-tree native libraries.

``cuda()`` returns ``libcverl_b200_cuda.so`` (sm_100a kernels, ``extern "C"``
launchers taking raw device pointers and a ``cudaStream_t``); ``host()``
returns ``libcverl.so`` (host runtime with the public C ABI).  Both are built
by :mod:`cverl_b200._build` and live under ``cverl_b200/lib``.  On a machine
with a GPU a missing kernel library is a hard error: there is no silent eager
fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_LIB_DIR = Path(__file__).resolve().parent / "lib"
_cuda_lib = None
_host_lib = None

c_void_p = C.c_void_p
c_ll = C.c_longlong
c_int = C.c_int
c_float = C.c_float


class GemmArgs(C.Structure):
    """Mirror of ``CvbGemmArgs`` (cuda/gemm_tcgen05.h)."""

    _fields_ = [
        ("A", c_void_p), ("B", c_void_p), ("C", c_void_p),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
        ("a_mn", C.c_int32), ("b_mn", C.c_int32),
        ("epi", C.c_int32), ("alpha", C.c_float),
        ("split_k", C.c_int32), ("block_n", C.c_int32), ("group_m", C.c_int32), ("max_ctas", C.c_int32),
        ("tile_group", c_void_p), ("b_group_rows", C.c_int64), ("b_total_rows", C.c_int64),
        ("k_group_offsets", c_void_p), ("num_groups", C.c_int32), ("c_group_stride", C.c_int64),
        ("targets", c_void_p), ("part_max", c_void_p), ("part_sum", c_void_p), ("tgt_logit", c_void_p),
        ("lse", c_void_p), ("gscale", c_void_p), ("status", c_void_p),
        ("mirror", c_void_p * 7), ("n_mirror", C.c_int32),
        ("scatter_base", c_void_p * 8), ("scatter_rows", C.c_int32),
        ("row_addr", c_void_p),
    ]


EPI_STORE_BF16, EPI_STORE_F32, EPI_ATOMIC_F32, EPI_LSE_PARTIAL, EPI_SOFTMAX_GRAD = range(5)


_CODES = {"p": c_void_p, "l": c_ll, "i": c_int, "f": c_float, "d": C.c_double}

# name -> argument codes (p pointer, l long long, i int, f float); every launcher returns int
_CUDA_PROTOS = {
    "cvb_rmsnorm_fwd": "ppppppplillff il p",
    "cvb_rmsnorm_bwd": "ppppppppplilllf illl p",
    "cvb_sp_add_rmsnorm_fwd": "p l i pp p i l pp l i ff p",
    "cvb_sp_add_rmsnorm_bwd": "p l i pppp p p i l p l i f p",
    "cvb_headnorm_rope_fwd": "ppppp lii ll i pp i ff i p",
    "cvb_headnorm_rope_bwd": "ppppppp lii ll i pp i f i p",
    "cvb_swiglu_fwd": "pp l i l p",
    "cvb_swiglu_bwd": "ppp l i l p",
    "cvb_siggate_fwd": "ppp l i ll ii p",
    "cvb_siggate_bwd": "ppppp l i ll ii ll i p",
    "cvb_conv1d_silu_fwd": "ppp l iii l p",
    "cvb_conv1d_silu_bwd": "ppppp l iii ll p",
    "cvb_conv1d_silu_bwd_tma": "ppppp l iii ll p p",
    "cvb_embedding_fwd": "ppp l i ll p",
    "cvb_embedding_bwd": "ppp l i ll p",
    "cvb_cast_f32_to_bf16": "pp l f p",
    "cvb_rl_workspace_doubles": "",
    "cvb_masked_sum_mean": "pp l i pp p",
    "cvb_masked_whiten": "pp l i pp p",
    "cvb_kl_penalty": "ppp l ii p",
    "cvb_gae": "pppppp l i ff p p",
    "cvb_grpo_advantage": "ppp f i ppp l i p",
    "cvb_ppo_loss": "pppppppp l i ffff i f i f p p",
    "cvb_sumsq_f32": "p l f p p",
    "cvb_clip_scale": "p f p p",
    "cvb_flat_adamw": "ppppppp l fffff f l i p",
    "cvb_lse_combine": "ppppppp l i p",
    "cvb_lse_merge_ranks": "ppppp l i p",
    "cvb_ipc_get_handle": "ppp",
    "cvb_ipc_open_handle": "pp",
    "cvb_ipc_close_handle": "p",
    "cvb_device_malloc": "pl",
    "cvb_device_free": "p",
    "cvb_device_memset": "pilp",
    "cvb_can_access_peer": "ii",
    "cvb_device_memcpy_async": "pp l p",
    "cvb_gdn_chunk_prep": "ppp l pp l ii ff pppppppp p p",
    "cvb_gdn_chunk_out": "ppppp l ii p p",
    "cvb_gdn_chunk_bwd": "ppp l p ppp pp pp p p l ii f ppp l pp p p",
    "cvb_gdn_gates_fwd": "pppp pp l i l p",
    "cvb_gdn_gates_bwd": "pp pppp pp pp l i ll p",
    "cvb_gdn_scan_fwd": "pppppppp l i p p",
    "cvb_gdn_scan_bwd": "pppppppppp l ii p p",
    "cvb_symm_barrier": "p iii p p",
    "cvb_reduce_scatter_sumsq": "p ii ll f pp p",
    "cvb_reduce_scatter_acc": "p ii ll f p ii p",
    "cvb_flat_adamw_allgather": "ppppp p ii ll fffff l p",
    "cvb_broadcast_store": "pp i l p",
    "cvb_sum_parts": "p l i p l p",
    "cvb_multimem_broadcast_store": "pp l i p",
    "cvb_multimem_reduce_scatter": "p ll f p i p i p",
    "cvb_multimem_allreduce_bf16": "p ll i p",
    "cvb_p2p_scatter_rows": "pp i pp ll l p p",
    "cvb_p2p_gather_rows": "pp i pp ll l p p",
    "cvb_attention_fwd": "ppppp l iiiii f i ll p p",
    "cvb_attention_bwd": "ppppp p pp ppp l iiiii f i ll p p",
    "cvb_attn_merge": "pppp l iiiiii p",
    "cvb_decode_attention": "p ll pp l ppp p iiiii f p p",
    "cvb_gdn_decode_step": "p l ii pp i p pp l pp pp i p",
    "cvb_router_topk_fwd": "p l iii pp p",
    "cvb_router_topk_bwd": "pppp l iii p p",
    "cvb_expert_layout": "p l ii ppp i pp p",
}


def _bind(lib, protos) -> None:
    for name, codes in protos.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:  # a stale library: fail loudly
            raise RuntimeError(f"native library lacks symbol {name}; rebuild with python -m cverl_b200._build") from exc
        fn.argtypes = [_CODES[c] for c in codes.replace(" ", "")]
        fn.restype = c_int


def _ensure_built() -> None:
    from . import _build
    if os.environ.get("CVERL_B200_NO_AUTOBUILD") == "1":
        return
    _build.build_all()


def cuda():
    """The CUDA kernel library; raises when it cannot be loaded."""
    global _cuda_lib
    if _cuda_lib is None:
        path = _LIB_DIR / "libcverl_b200_cuda.so"
        if not path.exists():
            _ensure_built()
        if not path.exists():
            raise RuntimeError(f"native CUDA library missing: {path} (run python -m cverl_b200._build)")
        lib = C.CDLL(str(path))
        lib.cvb_gemm_bf16.argtypes = [C.POINTER(GemmArgs), c_void_p]
        lib.cvb_gemm_bf16.restype = c_int
        _bind(lib, _CUDA_PROTOS)
        _cuda_lib = lib
    return _cuda_lib


def host():
    """The host runtime library (C ABI)."""
    global _host_lib
    if _host_lib is None:
        path = _LIB_DIR / "libcverl.so"
        if not path.exists():
            from . import _build
            _build.build_host()
        _host_lib = C.CDLL(str(path))
    return _host_lib


def have_cuda_kernels() -> bool:
    """True when CUDA tensors should run the native kernels (a GPU is present)."""
    return torch.cuda.is_available()


def ptr(t) -> int | None:
    """Device/host pointer of a tensor (None passes a null pointer)."""
    if t is None:
        return None
    return t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_status_words = {}


def status_word(device=None) -> torch.Tensor:
    """Per-device int32 status word that kernels with bounded waits write on a timeout."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status_words.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _status_words[key] = t
    return t


def check_status(device=None) -> int:
    """Host read of the status word (synchronises). Raises on a recorded kernel error."""
    t = status_word(device)
    code = int(t.item())
    if code != 0:
        t.zero_()
        raise RuntimeError(f"cverl_b200 kernel reported error status {code} (bounded wait ran out)")
    return code


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
