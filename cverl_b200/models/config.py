"""Model configuration for the Qwen3.5 hybrid (Gated-DeltaNet + full attention)
and Qwen3-MoE text models.

Defaults are the Qwen3.5-0.8B shape, as in the reference
(include/cverl/model/qwen3_5_text.h:17-42); ``from_hf_config`` reads the same
``config.json`` keys as src/model/qwen3_5_text.cc:555-595, including the
Qwen3-MoE overrides (full rotary, every layer full attention).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import List


@dataclass
class Qwen35TextConfig:
    model_type: str = "qwen3_5"
    vocab_size: int = 248320
    hidden_size: int = 1024
    num_hidden_layers: int = 24
    num_attention_heads: int = 8
    num_key_value_heads: int = 2
    head_dim: int = 256
    intermediate_size: int = 3584
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 16
    linear_conv_kernel_dim: int = 4
    moe_intermediate_size: int = 0
    num_experts: int = 0
    num_experts_per_tok: int = 0
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e7
    partial_rotary_factor: float = 0.25
    norm_topk_prob: bool = True
    tie_word_embeddings: bool = True
    layer_types: List[str] = field(default_factory=list)

    def __post_init__(self):
        if self.is_qwen3_moe:
            self.partial_rotary_factor = 1.0
            self.layer_types = ["full_attention"] * self.num_hidden_layers
            if self.moe_intermediate_size <= 0 or self.num_experts <= 0 or self.num_experts_per_tok <= 0:
                raise ValueError("qwen3_moe config requires moe_intermediate_size/num_experts/num_experts_per_tok")
        elif not self.layer_types:
            self.layer_types = ["full_attention" if (i + 1) % 4 == 0 else "linear_attention"
                                for i in range(self.num_hidden_layers)]
        if len(self.layer_types) != self.num_hidden_layers:
            raise ValueError("layer_types length must equal num_hidden_layers")

    # ------------------------------------------------------------------
    @property
    def is_qwen3_moe(self) -> bool:
        return self.model_type == "qwen3_moe"

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def norm_weight_offset(self) -> float:
        """RMSNorm scale is ``1 + w`` for Qwen3.5 and ``w`` for Qwen3-MoE."""
        return 0.0 if self.is_qwen3_moe else 1.0

    @property
    def layer_root(self) -> str:
        return "model.layers." if self.is_qwen3_moe else "model.language_model.layers."

    @property
    def embed_name(self) -> str:
        return "model.embed_tokens.weight" if self.is_qwen3_moe else "model.language_model.embed_tokens.weight"

    @property
    def final_norm_name(self) -> str:
        return "model.norm.weight" if self.is_qwen3_moe else "model.language_model.norm.weight"

    @property
    def lm_head_name(self) -> str:
        return "lm_head.weight" if (self.is_qwen3_moe and not self.tie_word_embeddings) else self.embed_name

    @property
    def linear_key_dim(self) -> int:
        return self.linear_num_key_heads * self.linear_key_head_dim

    @property
    def linear_value_dim(self) -> int:
        return self.linear_num_value_heads * self.linear_value_head_dim

    @property
    def linear_conv_dim(self) -> int:
        return 2 * self.linear_key_dim + self.linear_value_dim

    # ------------------------------------------------------------------
    @classmethod
    def from_hf_config(cls, cfg: dict) -> "Qwen35TextConfig":
        text = cfg.get("text_config", cfg)
        known = {f for f in cls.__dataclass_fields__}
        kw = {k: v for k, v in text.items() if k in known}
        if "model_type" in cfg and "model_type" not in kw:
            kw["model_type"] = cfg["model_type"]
        mt = kw.get("model_type", "qwen3_5")
        kw["model_type"] = "qwen3_moe" if mt == "qwen3_moe" else "qwen3_5"
        if "rope_theta" not in kw and isinstance(text.get("rope_parameters"), dict):
            rp = text["rope_parameters"]
            if "rope_theta" in rp:
                kw["rope_theta"] = rp["rope_theta"]
            if "partial_rotary_factor" in rp:
                kw["partial_rotary_factor"] = rp["partial_rotary_factor"]
        if kw.get("layer_types") is None:
            kw.pop("layer_types", None)
        return cls(**kw)

    @classmethod
    def from_model_dir(cls, model_dir) -> "Qwen35TextConfig":
        return cls.from_hf_config(json.loads((Path(model_dir) / "config.json").read_text()))

    def to_hf_config(self) -> dict:
        d = {k: getattr(self, k) for k in self.__dataclass_fields__}
        d["architectures"] = ["Qwen3MoeForCausalLM" if self.is_qwen3_moe else "Qwen3_5ForCausalLM"]
        return d

    # ------------------------------------------------------------------
    @classmethod
    def qwen3_5_0_8b(cls) -> "Qwen35TextConfig":
        return cls()

    @classmethod
    def qwen3_30b_a3b(cls) -> "Qwen35TextConfig":
        return cls(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, num_hidden_layers=48,
                   num_attention_heads=32, num_key_value_heads=4, head_dim=128, intermediate_size=6144,
                   moe_intermediate_size=768, num_experts=128, num_experts_per_tok=8, rope_theta=1e6,
                   tie_word_embeddings=False, norm_topk_prob=True)

    @classmethod
    def tiny(cls, moe: bool = False, layers: int = 4, vocab: int = 512) -> "Qwen35TextConfig":
        """Small shape for tests; every dimension keeps the 8-element alignment the kernels need."""
        if moe:
            return cls(model_type="qwen3_moe", vocab_size=vocab, hidden_size=64, num_hidden_layers=layers,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=128,
                       moe_intermediate_size=64, num_experts=8, num_experts_per_tok=2, rope_theta=1e4,
                       tie_word_embeddings=False)
        return cls(vocab_size=vocab, hidden_size=64, num_hidden_layers=layers, num_attention_heads=4,
                   num_key_value_heads=2, head_dim=64, intermediate_size=128, linear_key_head_dim=64,
                   linear_value_head_dim=64, linear_num_key_heads=2, linear_num_value_heads=2, rope_theta=1e4)
