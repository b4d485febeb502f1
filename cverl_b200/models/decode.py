"""Cached autoregressive decode for ``Qwen35Model`` (one rank, or the ranks of a tensor-parallel group).

The reference generates by re-running the whole forward over prompt + prefix for every new
token (src/rollout/policy_worker.cc:99-102, O(N^2)).  Here ``prefill`` runs the prompt once
and keeps, per layer, either the rotated keys and the values (full attention) or the last
``conv_kernel-1`` pre-convolution rows plus the ``[dk, dv]`` recurrent state (Gated DeltaNet);
``decode_step`` then advances every sequence by one token with one token of compute.

On a GPU with bf16 parameters the step runs on the native kernels (``decode_step_native``): tcgen05 GEMMs for
every projection and the LM head, the fused norm / RoPE / gate kernels of training, ``cvb_decode_attention``
(appends the token's key / value to the cache and attends over it, reading the length from device memory) and
``cvb_gdn_decode_step`` (one read and one write of the recurrent state).  Nothing in that step depends on a
host-side shape or scalar, so ``GraphedDecoder`` captures it once in a CUDA graph and replays it per token.
The fp32 PyTorch statement below stays as the CPU path and the test oracle.  It also serves tensor parallelism:
every rank keeps the caches of its own heads, the row-parallel projections are summed over the group, the
embedding lookup is vocabulary-parallel and the LM head's logits are gathered; the native step and the CUDA graph
are single-rank (``native_decode_supported``), so a tensor-parallel decode on GPUs runs this statement.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.nn.functional as F

from .. import ops
from ..ops.gdn import l2norm
from ..ops.norm import apply_rope_ref, rmsnorm_ref


@dataclass
class DecodeState:
    length: int                      # tokens already in the caches
    layers: List[dict] = field(default_factory=list)
    dev: Optional[dict] = None       # device-side step counters and tables of the native path

    def to_native(self, model) -> None:
        """Device copies of what the native step reads: the length after this step (int32 [1]), the position of
        the new token per sequence (int32 [B]), the rotary tables up to the cache length."""
        cfg = model.cfg
        dev = model.flat.flat.device
        max_len = max([c["k"].shape[1] for c in self.layers if "k" in c] or [self.length + 1])
        B = next(iter(self.layers[0].values())).shape[0]
        cos, sin = ops.rope_tables(max_len, cfg.rotary_dim, cfg.rope_theta, dev)
        self.dev = {"len": torch.full((1,), self.length + 1, dtype=torch.int32, device=dev),
                    "pos": torch.full((B,), self.length, dtype=torch.int32, device=dev), "cos": cos, "sin": sin,
                    "max_len": max_len}
        for c in self.layers:
            if "state" in c:
                c["state"] = c["state"].float().contiguous()
            if "conv" in c:
                # ring cache of raw pre-convolution rows: the row of token t lives in slot t % KW.  The prefill
                # left the last KW - 1 rows (tokens length-KW+1 .. length-1) in order.
                kw = cfg.linear_conv_kernel_dim
                tail = c["conv"].to(model.dtype)
                ring = torch.zeros((tail.shape[0], kw, tail.shape[2]), dtype=model.dtype, device=dev)
                for r in range(kw - 1):
                    tok = self.length - (kw - 1) + r
                    if tok >= 0:
                        ring[:, tok % kw] = tail[:, r]
                c["conv_ring"] = ring.contiguous()
            if "k" in c:
                c["k"], c["v"] = c["k"].contiguous(), c["v"].contiguous()


def _lin(x, w):
    return (x.to(w.dtype) @ w.t())


def _tp_sum(model, t: torch.Tensor) -> torch.Tensor:
    """Sum of the tensor-parallel ranks' partial results (the output of a row-parallel projection)."""
    if model.ctx.tp_size > 1:
        import torch.distributed as dist
        t = t.contiguous()
        dist.all_reduce(t, group=model.ctx.tp_group)
    return t


def _full_logits(model, hidden: torch.Tensor) -> torch.Tensor:
    """hidden [B, H] -> fp32 logits [B, V]; the LM head is sharded over vocabulary rows under tensor parallelism."""
    logits = hidden.float() @ model.lm_head_weight().float().t()
    if model.ctx.tp_size > 1:
        import torch.distributed as dist
        parts = [torch.empty_like(logits) for _ in range(model.ctx.tp_size)]
        dist.all_gather(parts, logits.contiguous(), group=model.ctx.tp_group)
        logits = torch.cat(parts, dim=-1)
    return logits


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
    return DecodeState(S, caches), _full_logits(model, hidden[:, -1])


def native_decode_supported(model) -> bool:
    cfg = model.cfg
    p = model.flat.flat
    return (p.is_cuda and p.dtype == torch.bfloat16 and model.ctx.tp_size == 1 and not cfg.is_qwen3_moe
            and cfg.head_dim in (128, 256) and cfg.linear_key_head_dim == 128 and cfg.linear_value_head_dim == 128
            and cfg.num_attention_heads // cfg.num_key_value_heads in (1, 2, 4, 8)
            and model.first_stage and model.last_stage)


@torch.no_grad()
def decode_step(model, state: DecodeState, tokens: torch.Tensor) -> torch.Tensor:
    """Feeds one token per sequence; returns the logits ``[B, V]`` of the following token."""
    if native_decode_supported(model) and tokens.is_cuda:
        if state.dev is None:
            state.to_native(model)
        return decode_step_native(model, state, tokens)
    cfg = model.cfg
    B = tokens.shape[0]
    pos = state.length
    eps, off = cfg.rms_norm_eps, cfg.norm_weight_offset
    h = model.embed(tokens.view(B, 1)).float()          # vocabulary-parallel lookup + sum under tensor parallelism
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
    return _full_logits(model, out)


def _full_attention_step(model, x, i, c, pos):
    cfg = model.cfg
    p = f"{cfg.layer_root}{i}.self_attn."
    tp = model.ctx.tp_size                                # heads are sharded over the tensor-parallel ranks
    d, h, kvh = cfg.head_dim, cfg.num_attention_heads // tp, cfg.num_key_value_heads // tp
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
    return _tp_sum(model, _lin(o.reshape(B, h * d), model.param(p + "o_proj.weight")))


def _linear_attention_step(model, x, i, c):
    cfg = model.cfg
    p = f"{cfg.layer_root}{i}.linear_attn."
    tp = model.ctx.tp_size
    kh, vh = cfg.linear_num_key_heads // tp, cfg.linear_num_value_heads // tp
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
    return _tp_sum(model, _lin(y.reshape(B, value_dim), model.param(p + "out_proj.weight")))


# ---------------------------------------------------------------------------------------------------------
# native one-token step
# ---------------------------------------------------------------------------------------------------------
def _native_full_attention(model, x, i, c, dv):
    from .. import _native as nv
    from ..ops.gemm import count_launch
    cfg = model.cfg
    p = f"{cfg.layer_root}{i}.self_attn."
    d, h, kvh = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    B = x.shape[0]
    qkv = ops.linear(x, model.fused[f"{i}.qkv"])                       # [B, h*d*2 + 2*kvh*d] bf16
    q_all, k, v = qkv.split([h * d * 2, kvh * d, kvh * d], dim=-1)
    q, gate = q_all.view(B, h, 2 * d).split([d, d], dim=-1)            # strided views into the projection
    off = cfg.norm_weight_offset
    q = ops.headnorm_rope(q, model.param(p + "q_norm.weight"), dv["cos"], dv["sin"], dv["pos"], cfg.rotary_dim,
                          cfg.rms_norm_eps, off)
    k = ops.headnorm_rope(k.view(B, kvh, d), model.param(p + "k_norm.weight"), dv["cos"], dv["sin"], dv["pos"],
                          cfg.rotary_dim, cfg.rms_norm_eps, off)
    o = torch.empty((B, h, d), dtype=x.dtype, device=x.device)
    if k.stride(0) != v.stride(0):           # the kernel takes one row stride for the new key and value
        v = v.contiguous()
        k = k.contiguous()
    nv.check(nv.cuda().cvb_decode_attention(q.data_ptr(), q.stride(0), q.stride(1), k.data_ptr(), v.data_ptr(),
                                            k.stride(0), c["k"].data_ptr(), c["v"].data_ptr(), o.data_ptr(),
                                            dv["len"].data_ptr(), B, c["k"].shape[1], h, kvh, d,
                                            1.0 / math.sqrt(d), nv.status_word(x.device).data_ptr(), nv.stream()),
             "cvb_decode_attention")
    count_launch()
    o = ops.siggate(o, gate)
    return ops.linear(o.reshape(B, h * d), model.param(p + "o_proj.weight"))


def _native_linear_attention(model, x, i, c, dv):
    from .. import _native as nv
    from ..ops.gemm import count_launch
    cfg = model.cfg
    p = f"{cfg.layer_root}{i}.linear_attn."
    kh, vh = cfg.linear_num_key_heads, cfg.linear_num_value_heads
    kd, vd = cfg.linear_key_head_dim, cfg.linear_value_head_dim
    key_dim, value_dim = kh * kd, vh * vd
    conv_dim = 2 * key_dim + value_dim
    B = x.shape[0]
    proj = ops.linear(x, model.fused[f"{i}.lin_in"])                   # [B, conv_dim + value_dim + 2 vh]
    mixed, z, b, a = proj.split([conv_dim, value_dim, vh, vh], dim=-1)
    o = torch.empty((B, vh, vd), dtype=x.dtype, device=x.device)
    # convolution (ring cache of raw rows) + SiLU + l2norm + gates + state update + read-out: one kernel
    nv.check(nv.cuda().cvb_gdn_decode_step(proj.data_ptr(), proj.stride(0), kh, vh,
                                           model.param(p + "conv1d.weight").data_ptr(), c["conv_ring"].data_ptr(),
                                           cfg.linear_conv_kernel_dim, dv["len"].data_ptr(), b.data_ptr(),
                                           a.data_ptr(), proj.stride(0), model.param(p + "A_log").data_ptr(),
                                           model.param(p + "dt_bias").data_ptr(), c["state"].data_ptr(),
                                           o.data_ptr(), B, nv.stream()), "cvb_gdn_decode_step")
    count_launch()
    y = ops.gated_rmsnorm(o, z, model.param(p + "norm.weight"), cfg.rms_norm_eps)
    return ops.linear(y.reshape(B, value_dim), model.param(p + "out_proj.weight"))


@torch.no_grad()
def decode_step_native(model, state: DecodeState, tokens: torch.Tensor, advance: bool = True) -> torch.Tensor:
    """One token per sequence on the native kernels; logits ``[B, V]`` fp32.  Every length / position is read
    from ``state.dev`` on the device and advanced there, so the same launches serve every step."""
    cfg = model.cfg
    dv = state.dev
    B = tokens.shape[0]
    eps, off = cfg.rms_norm_eps, cfg.norm_weight_offset
    delta = ops.embedding(tokens.view(B), model.param(cfg.embed_name))
    resid = None
    for li, i in enumerate(range(model.layer_begin, model.layer_end)):
        p = f"{cfg.layer_root}{i}."
        c = state.layers[li]
        n1, resid = ops.add_rmsnorm(delta, resid, model.param(p + "input_layernorm.weight"), eps, off)
        if cfg.layer_types[i] == "full_attention":
            a = _native_full_attention(model, n1, i, c, dv)
        else:
            a = _native_linear_attention(model, n1, i, c, dv)
        n2, resid = ops.add_rmsnorm(a, resid, model.param(p + "post_attention_layernorm.weight"), eps, off)
        delta = model.mlp(n2, i)
    out, _ = ops.add_rmsnorm(delta, resid, model.param(cfg.final_norm_name), eps, off)
    logits = ops.gemm_nt(out, model.lm_head_weight(), out_dtype=torch.float32)
    if advance:
        dv["len"] += 1
        dv["pos"] += 1
        state.length += 1
    return logits


class GraphedDecoder:
    """The native decode step captured once in a CUDA graph and replayed per token.

    ``step(tokens)`` copies the tokens into the graph's input buffer, replays, and returns the graph's logits
    buffer (valid until the next ``step``).  The caches, the recurrent states, the length counter and the position
    vector are the tensors of ``state``; the graph updates them in place.
    """

    def __init__(self, model, state: DecodeState, batch: int, warmup: int = 2):
        if not native_decode_supported(model):
            raise RuntimeError("the native decode path does not support this model / device")
        if state.dev is None:
            state.to_native(model)
        self.model, self.state = model, state
        dev = model.flat.flat.device
        self.tokens = torch.zeros(batch, dtype=torch.long, device=dev)
        # warm-up steps run for real on a side stream (lazy initialisation, allocator pools) and are then undone:
        # the caches / states they touched are restored, the counters rewound
        snapshot = [{k: v.clone() for k, v in c.items() if k in ("state", "conv_ring")} for c in state.layers]
        len0, pos0, host_len = state.dev["len"].clone(), state.dev["pos"].clone(), state.length
        s = torch.cuda.Stream(device=dev)
        s.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(s):
            for _ in range(warmup):
                decode_step_native(model, state, self.tokens)
        torch.cuda.current_stream(dev).wait_stream(s)
        self._restore(snapshot, len0, pos0, host_len)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = decode_step_native(model, state, self.tokens)
        # capturing executed nothing, but the host-side counter moved: rewind it
        state.length = host_len
        self._restore(snapshot, len0, pos0, host_len)

    def _restore(self, snapshot, len0, pos0, host_len) -> None:
        for c, snap in zip(self.state.layers, snapshot):
            for k, v in snap.items():
                c[k].copy_(v)
        self.state.dev["len"].copy_(len0)
        self.state.dev["pos"].copy_(pos0)
        self.state.length = host_len

    @torch.no_grad()
    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        self.tokens.copy_(tokens.view(-1))
        self.graph.replay()
        self.state.length += 1
        return self.logits
