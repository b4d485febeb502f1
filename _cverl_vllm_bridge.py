"""Import name of the reference's pybind module (python/cverl_vllm_bridge.cc:323-351): ``QwenPolicy`` with
``to_device``, ``named_parameters``, ``update_info`` and ``gsm8k_grpo_update``, so scripts written against the
reference (``import _cverl_vllm_bridge``) run unchanged.  The class lives in ``cverl_b200.rollout.vllm_bridge``."""
from cverl_b200.rollout.vllm_bridge import QwenPolicy  # noqa: F401

__all__ = ["QwenPolicy"]
