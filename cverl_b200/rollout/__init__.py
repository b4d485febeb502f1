"""Rollout layer: workers, plugin loader, transports, batch builder, GPU batch hand-off."""
from .worker import (CachedQwenRolloutWorker, GenerationConfig, GenerationOutput, PolicyRolloutWorker,  # noqa: F401
                     RolloutWorker, TokenBatch, sample_next_tokens, synchronize_rollout_actor_weights)
from .transport import (LoopbackRolloutTransport, RolloutRequest, RolloutResponse, RolloutSequence,  # noqa: F401
                        RolloutTransport, SharedMemoryRegion, SharedMemoryRolloutTransport)
from .plugin_worker import DynamicRolloutWorker, load_rollout_worker_plugin  # noqa: F401
from .rollout_batch import RolloutBatch, RolloutSample, build_gsm8k_rollout_batch  # noqa: F401
