"""Rule-based rewards (GSM8K) on the native host library."""
from .gsm8k import (Gsm8kRewardOptions, compute_gsm8k_reward, compute_gsm8k_rewards, extract_gsm8k_answer,  # noqa: F401
                    normalize_gsm8k_ground_truth)
