"""Cached autoregressive decode for ``Qwen35Model`` (single rank).

The reference generates by re-running the whole forward over prompt + prefix for every new
token (src/rollout/policy_worker.cc:99-102, O(N^2)).  Here ``prefill`` runs the prompt once
and keeps, per layer, either the rotated keys and the values (full attention) or the last
``conv_kernel-1`` pre-convolution rows plus the ``[dk, dv]`` recurrent state (Gated DeltaNet);
``decode_step`` then advances every sequence by one token with one token of compute.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List

import torch
import torch.nn.functional as F

from .. import ops
from ..ops.gdn import l2norm
from ..ops.norm import apply_rope_ref, rmsnorm_ref


@dataclass
class DecodeState:
    length: int                      # tokens already in the caches
    layers: List[dict] = field(default_factory=list)


def _lin(x, w):
    return (x.to(w.dtype) @ w.t())


@torch.no_grad()
def prefill(model, prompt_ids: torch.Tensor, max_len: int):
    """Runs the prompt; returns ``(state, logits [B, V] of the next token)``."""
    cfg = model.cfg
    B, S = prompt_ids.shape
    caches: List[dict] = []
    x = model.embed(prompt_ids)
    hidden = model.forward_layers(x, B, S, caches=caches).view(B, S, -1)
    for c in caches:
        if "k" in c:  # grow to the full decode length once, instead of a cat per step
            k = torch.zeros((B, max_len) + tuple(c["k"].shape[2:]), dtype=c["k"].dtype, device=c["k"].device)
            v = torch.zeros_like(k)
            k[:, :S], v[:, :S] = c["k"], c["v"]
            c["k"], c["v"] = k, v
    logits = hidden[:, -1].float() @ model.lm_head_weight().float().t()
    return DecodeState(S, caches), logits


@torch.no_grad()
def decode_step(model, state: DecodeState, tokens: torch.Tensor) -> torch.Tensor:
    """Feeds one token per sequence; returns the logits ``[B, V]`` of the following token."""
    cfg = model.cfg
    B = tokens.shape[0]
    pos = state.length
    eps, off = cfg.rms_norm_eps, cfg.norm_weight_offset
    h = ops.embedding(tokens.view(B), model.param(cfg.embed_name)).float()
    for li, i in enumerate(range(model.layer_begin, model.layer_end)):
        p = f"{cfg.layer_root}{i}."
        c = state.layers[li]
        n1 = rmsnorm_ref(h, model.param(p + "input_layernorm.weight"), eps, off)
        if cfg.layer_types[i] == "full_attention":
            a = _full_attention_step(model, n1, i, c, pos)
        else:
            a = _linear_attention_step(model, n1, i, c)
        h = h + a.float()
        n2 = rmsnorm_ref(h, model.param(p + "post_attention_layernorm.weight"), eps, off)
        h = h + model.mlp(n2.to(model.dtype), i).float()
    state.length += 1
    out = rmsnorm_ref(h, model.param(cfg.final_norm_name), eps, off)
    return out.float() @ model.lm_head_weight().float().t()


def _full_attention_step(model, x, i, c, pos):
    cfg = model.cfg
    p = f"{cfg.layer_root}{i}.self_attn."
    d, h, kvh = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    B = x.shape[0]
    qkv = _lin(x, model.fused[f"{i}.qkv"]).float()
    qmul = 1 if cfg.is_qwen3_moe else 2
    q_all, k, v = qkv.split([h * d * qmul, kvh * d, kvh * d], dim=-1)
    if cfg.is_qwen3_moe:
        q, gate = q_all.view(B, h, d), None
    else:
        q, gate = q_all.view(B, h, 2 * d).split([d, d], dim=-1)
    k = k.view(B, kvh, d)
    off = cfg.norm_weight_offset
    q = rmsnorm_ref(q, model.param(p + "q_norm.weight"), cfg.rms_norm_eps, off)
    k = rmsnorm_ref(k, model.param(p + "k_norm.weight"), cfg.rms_norm_eps, off)
    cos, sin = ops.rope_tables(1, cfg.rotary_dim, cfg.rope_theta, x.device, offset=pos)
    zeros = torch.zeros(B, dtype=torch.long, device=x.device)
    q = apply_rope_ref(q, cos, sin, zeros, cfg.rotary_dim)
    k = apply_rope_ref(k, cos, sin, zeros, cfg.rotary_dim)
    c["k"][:, pos] = k.to(c["k"].dtype)
    c["v"][:, pos] = v.view(B, kvh, d).to(c["v"].dtype)
    keys = c["k"][:, :pos + 1].float().repeat_interleave(h // kvh, dim=2)     # [B, L, h, d]
    vals = c["v"][:, :pos + 1].float().repeat_interleave(h // kvh, dim=2)
    scores = torch.einsum("bhd,blhd->bhl", q, keys) / math.sqrt(d)
    o = torch.einsum("bhl,blhd->bhd", torch.softmax(scores, dim=-1), vals)
    if gate is not None:
        o = o * torch.sigmoid(gate)
    return _lin(o.reshape(B, h * d), model.param(p + "o_proj.weight"))


def _linear_attention_step(model, x, i, c):
    cfg = model.cfg
    p = f"{cfg.layer_root}{i}.linear_attn."
    kh, vh = cfg.linear_num_key_heads, cfg.linear_num_value_heads
    kd, vd = cfg.linear_key_head_dim, cfg.linear_value_head_dim
    key_dim, value_dim = kh * kd, vh * vd
    conv_dim = 2 * key_dim + value_dim
    B = x.shape[0]
    proj = _lin(x, model.fused[f"{i}.lin_in"]).float()
    mixed, z, b, a = proj.split([conv_dim, value_dim, vh, vh], dim=-1)
    w = model.param(p + "conv1d.weight").view(conv_dim, cfg.linear_conv_kernel_dim).float()
    window = torch.cat([c["conv"].float(), mixed.unsqueeze(1)], dim=1)        # [B, KW, C]
    c["conv"] = window[:, 1:].to(c["conv"].dtype)
    conv = F.silu((window * w.t().unsqueeze(0)).sum(1))
    q, k, v = conv.split([key_dim, key_dim, value_dim], dim=-1)
    q, k, v = q.view(B, kh, kd), k.view(B, kh, kd), v.view(B, vh, vd)
    if vh // kh > 1:
        q, k = q.repeat_interleave(vh // kh, 1), k.repeat_interleave(vh // kh, 1)
    q = l2norm(q) / math.sqrt(kd)
    k = l2norm(k)
    beta = torch.sigmoid(b)
    g = -torch.exp(model.param(p + "A_log").float()) * F.softplus(a + model.param(p + "dt_bias").float())
    S = c["state"].float() * torch.exp(g).unsqueeze(-1).unsqueeze(-1)          # [B, vh, kd, vd]
    kv = (S * k.unsqueeze(-1)).sum(-2)
    delta = (v - kv) * beta.unsqueeze(-1)
    S = S + k.unsqueeze(-1) * delta.unsqueeze(-2)
    c["state"] = S
    o = (S * q.unsqueeze(-1)).sum(-2)
    y = rmsnorm_ref(o, model.param(p + "norm.weight"), cfg.rms_norm_eps, 0.0, gate=z.view(B, vh, vd))
    return _lin(y.reshape(B, value_dim), model.param(p + "out_proj.weight"))
