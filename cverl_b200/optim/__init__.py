"""Optimizers: per-tensor fp32-master AdamW and the flat-shard AdamW used by ZeRO."""
from .adamw import AdamWOptions, FlatAdamW, Fp32MasterAdamW, clone_detached, parameter_delta_sum  # noqa: F401
