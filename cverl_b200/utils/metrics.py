"""Step metrics: one ``key=value`` line per step on rank 0 and an appended CSV.

Fields follow the reference trainer's line / 34-column CSV (tools/model/
qwen3_5_pp_tp_ppo_trainer.cc:1442-1447,2694-2740): parallel dims, shapes, ``step_time_s`` (max over
ranks), dtypes, sharding flags, reward / loss / KL / clip sums, gradient norms, clip scale, parameter
delta, and the health booleans that decide the exit code.  Metrics stay on the device inside the
micro-batch loop and cross to the host once per step.
"""
from __future__ import annotations

import csv
from pathlib import Path
from typing import Dict, Iterable, List, Optional

CSV_COLUMNS: List[str] = [
    "step", "dp", "pp", "cp", "tp", "ep", "sp", "micro_batches", "grad_accum_steps", "prompt_len",
    "response_len", "seq_len", "tokens", "step_time_s", "tokens_per_second", "dtype", "dp_grad_comm_dtype",
    "tp_grad_comm_dtype", "flat_shard_optimizer", "master_weights", "mean_reward", "success_rate",
    "adv_abs_sum", "loss_sum", "kl_loss_sum", "ppo_kl_sum", "clipfrac_sum", "grad_norm_sum",
    "global_grad_norm", "grad_clip_scale", "param_delta_sum", "all_ranks_have_grad", "all_ranks_updated",
    "any_rank_updated",
]


def format_line(values: Dict[str, object]) -> str:
    def fmt(v):
        if isinstance(v, bool):
            return "true" if v else "false"
        if isinstance(v, float):
            return f"{v:.6g}"
        return str(v)
    return " ".join(f"{k}={fmt(v)}" for k, v in values.items())


class MetricsCsv:
    def __init__(self, path: Optional[str]):
        self.path = Path(path) if path else None
        if self.path and not self.path.exists():
            self.path.parent.mkdir(parents=True, exist_ok=True)
            with self.path.open("w", newline="") as f:
                csv.writer(f).writerow(CSV_COLUMNS)

    def append(self, values: Dict[str, object]) -> None:
        if not self.path:
            return
        with self.path.open("a", newline="") as f:
            csv.writer(f).writerow([values.get(c, "") for c in CSV_COLUMNS])


def log_has_nonfinite(lines: Iterable[str]) -> bool:
    """The regression check of the reference's scripts: any nan/inf token in the log fails the run."""
    for ln in lines:
        low = ln.lower()
        if "=nan" in low or "=inf" in low or "=-inf" in low:
            return True
    return False
