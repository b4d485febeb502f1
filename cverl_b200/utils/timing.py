"""Device timing (CUDA events, max over ranks), NVTX ranges and roofline fractions."""
from __future__ import annotations

import contextlib
import json
from pathlib import Path
from typing import Callable, Dict, Optional

import torch

_FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
NVLINK_PEER_GBS = 770.0  # measured peer copy per direction on this pool (900 nominal)


def measured_peaks(repo_root=None) -> Dict[str, float]:
    root = Path(repo_root) if repo_root else Path(__file__).resolve().parents[2]
    p = root / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        d["source"] = "measured"
        return d
    return dict(_FALLBACK_PEAKS)


def time_cuda(fn: Callable[[], None], warmup: int = 3, iters: int = 10, flush_l2: bool = True, group=None) -> float:
    """Median milliseconds of ``fn`` with CUDA events on the current stream, L2 flushed between
    iterations, max over the ranks of ``group``."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush_l2 else None
    ts = []
    for _ in range(iters):
        if scratch is not None:
            scratch.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    ms = torch.tensor([ts[len(ts) // 2]], device="cuda")
    if group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()):
        torch.distributed.all_reduce(ms, op=torch.distributed.ReduceOp.MAX, group=group)
    return float(ms.item())


def roofline_fraction(ms: float, flops: float = 0.0, hbm_bytes: float = 0.0, nvlink_bytes: float = 0.0,
                      sustained: bool = False, peaks: Optional[dict] = None) -> Dict[str, float]:
    """Achieved / target where the target time is the slowest of compute at the measured GEMM peak,
    bytes at the measured copy bandwidth, and NVLink bytes at the measured peer bandwidth."""
    pk = peaks or measured_peaks()
    tf = pk["bf16_tflops_sustained" if sustained else "bf16_tflops"] * 1e12
    t_compute = flops / tf if flops else 0.0
    t_hbm = hbm_bytes / (pk["hbm_gbs"] * 1e9) if hbm_bytes else 0.0
    t_link = nvlink_bytes / (NVLINK_PEER_GBS * 1e9) if nvlink_bytes else 0.0
    target = max(t_compute, t_hbm, t_link)
    return {"target_ms": target * 1e3, "fraction": (target * 1e3 / ms) if ms > 0 else 0.0,
            "bound": "compute" if target == t_compute else ("hbm" if target == t_hbm else "nvlink"),
            "peaks": pk.get("source", "measured")}


@contextlib.contextmanager
def nvtx_range(name: str):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class PhaseTimer:
    """Per-phase CUDA-event timing of a training step (forward/backward, grad sync, optimizer)."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self._open, self.ms = {}, {}

    def start(self, name: str) -> None:
        if self.enabled:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._open[name] = e

    def stop(self, name: str) -> None:
        if self.enabled and name in self._open:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._open[name] = (self._open[name], e)

    def collect(self) -> Dict[str, float]:
        if not self.enabled:
            return {}
        torch.cuda.synchronize()
        for k, v in self._open.items():
            if isinstance(v, tuple):
                self.ms[k] = self.ms.get(k, 0.0) + v[0].elapsed_time(v[1])
        self._open = {}
        return dict(self.ms)
