"""Qwen3.5 hybrid (Gated-DeltaNet + full attention) and Qwen3-MoE text model.

Activations are packed ``[B*S, H]`` (B equal-length sequences); every block is
a chain of the fused ops in ``cverl_b200.ops``:

    (delta, resid) -> add+RMSNorm -> mixer -> add+RMSNorm -> MLP/MoE -> ...

* full attention: one GEMM for q|gate|k|v, per-head RMSNorm + partial RoPE in
  one kernel, causal GQA attention, sigmoid output gate, o_proj
  (reference: src/model/qwen3_5_text.cc:1036-1082);
* linear attention: one GEMM for qkv|z|b|a, causal conv1d+SiLU, l2norm, gated
  delta rule scan, gated RMSNorm, out_proj (:1228-1272);
* SwiGLU MLP from one gate|up GEMM (:791-793), or the Qwen3-MoE router + experts
  (:761-790, :796-993);
* tied (or untied) LM head evaluated as fused log-probabilities (:1590-1630).

Tensor parallelism is Megatron column/row sharding with the mathematically
correct backward (the activation gradient entering a column-parallel GEMM is
all-reduced); the reference skips that all-reduce and averages replicated
parameters instead (tools/model/qwen3_5_pp_tp_ppo_trainer.cc:545-558), a
deviation made on purpose.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as _checkpoint

from .. import ops
from ..ops import attention as attn_ops
from ..ops import gdn as gdn_ops
from ..parallel.autograd_collectives import copy_to_tp, reduce_from_tp
from ..parallel.context import SINGLE, ParallelContext
from .config import Qwen35TextConfig
from .params import FlatParams, ParamSpec, model_param_specs, shard_tensor, unshard_tensor


def _packed_moe_names(layer: int) -> Tuple[str, str]:
    return (f"__packed_moe.layers.{layer}.gate_up.weight", f"__packed_moe.layers.{layer}.down.weight")


class Qwen35Model(torch.nn.Module):
    """One pipeline stage (by default the whole model) of the text model."""

    def __init__(self, cfg: Qwen35TextConfig, *, dtype=torch.bfloat16, device="cpu",
                 ctx: ParallelContext = SINGLE, layer_begin: int = 0, layer_end: Optional[int] = None,
                 first_stage: bool = True, last_stage: bool = True, pad_multiple: int = 1,
                 with_main_grad: bool = True, flat_allocator=None, grad_buckets: bool = False,
                 bucket_align: int = 8, grad_slots: int = 2, activation_checkpointing: bool = False):
        """``grad_buckets``: per-layer gradient buckets on ``grad_slots`` rotating buffers instead of a full fp32
        gradient twin (for ``BucketedZero2Optimizer``, which reduces a layer's gradients while the backward pass
        runs the next layer); the embedding and the head keep a buffer each.
        ``activation_checkpointing``: a layer keeps only its input between the forward and the backward pass and is
        run again when its backward starts (the reference declares the policy flag,
        include/cverl/distributed/topology.h:29, and implements recomputation only inside its two custom autograd
        functions)."""
        super().__init__()
        self.cfg = cfg
        self.activation_checkpointing = activation_checkpointing
        self.ctx = ctx
        self.dtype = dtype
        self.layer_begin = layer_begin
        self.layer_end = cfg.num_hidden_layers if layer_end is None else layer_end
        self.first_stage, self.last_stage = first_stage, last_stage
        tp = ctx.tp_size
        if tp > 1:
            if tp > cfg.num_key_value_heads:
                raise ValueError("tensor-parallel size must not exceed num_key_value_heads")
            if cfg.num_attention_heads % tp or cfg.num_key_value_heads % tp:
                raise ValueError("attention heads must divide by the tensor-parallel size")
        if cfg.is_qwen3_moe and cfg.num_experts % ctx.ep_size:
            raise ValueError("num_experts must divide by the expert-parallel size")
        self.specs: List[ParamSpec] = model_param_specs(cfg, self.layer_begin, self.layer_end, first_stage,
                                                        last_stage)
        self.spec_by_name: Dict[str, ParamSpec] = {s.name: s for s in self.specs}
        entries = self._flat_entries()
        buckets, pinned = None, ()
        if grad_buckets:
            buckets = [self._bucket_of_entry(n) for n, _ in entries]
            pinned = (0,)
        self.flat = FlatParams(entries, dtype=dtype, device=device, pad_multiple=pad_multiple,
                               with_main_grad=with_main_grad, allocator=flat_allocator, grad_buckets=buckets,
                               bucket_align=bucket_align, grad_slots=grad_slots, pinned_buckets=pinned)
        # ``backward_boundary(delta, resid, bucket)``: identity on the residual stream whose backward tells a
        # bucketed optimizer that the layers after this point have finished their backward pass
        self.backward_boundary = None
        for name, p in self.flat.params.items():
            self.register_parameter(name.replace(".", "/"), p)
        self._build_fused_views()
        self._rope_cache: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._cp_original_len: Optional[int] = None
        self._sp_active = False     # inside a sequence-parallel forward (see ``sequence_parallel``)

    # ------------------------------------------------------------------ layout
    def _bucket_of_entry(self, name: str) -> int:
        """Gradient bucket of a flat entry: 0 = everything outside the layers (embedding, final norm, untied
        head: they come first in the buffer), 1 + k = k-th layer of this stage."""
        root = self.cfg.layer_root
        for prefix in (root, "__packed_moe.layers."):
            if name.startswith(prefix):
                return 1 + int(name[len(prefix):].split(".")[0]) - self.layer_begin
        return 0

    def _flat_entries(self) -> List[Tuple[str, Tuple[int, ...]]]:
        cfg, tp, ep = self.cfg, self.ctx.tp_size, self.ctx.ep_size
        entries: List[Tuple[str, Tuple[int, ...]]] = []
        packed_done = set()
        for s in self.specs:
            if s.expert >= 0:
                layer = int(s.name[len(cfg.layer_root):].split(".")[0])
                if layer in packed_done:
                    continue
                packed_done.add(layer)
                e_local = cfg.num_experts // ep
                i_local = cfg.moe_intermediate_size // tp
                gu, dn = _packed_moe_names(layer)
                entries.append((gu, (e_local, 2 * i_local, cfg.hidden_size)))
                entries.append((dn, (e_local, cfg.hidden_size, i_local)))
            else:
                entries.append((s.name, s.local_shape(tp)))
        return entries

    def _build_fused_views(self) -> None:
        cfg, tp = self.cfg, self.ctx.tp_size
        self.fused: Dict[str, torch.nn.Parameter] = {}
        H = cfg.hidden_size
        for i in range(self.layer_begin, self.layer_end):
            p = f"{cfg.layer_root}{i}."
            if cfg.layer_types[i] == "full_attention":
                sa = p + "self_attn."
                names = [sa + "q_proj.weight", sa + "k_proj.weight", sa + "v_proj.weight"]
                rows = sum(self.flat.params[n].shape[0] for n in names)
                self.fused[f"{i}.qkv"] = self.flat.fused_view(names, (rows, H))
            else:
                la = p + "linear_attn."
                names = [la + "in_proj_qkv.weight", la + "in_proj_z.weight", la + "in_proj_b.weight",
                         la + "in_proj_a.weight"]
                rows = sum(self.flat.params[n].shape[0] for n in names)
                self.fused[f"{i}.lin_in"] = self.flat.fused_view(names, (rows, H))
            if not cfg.is_qwen3_moe:
                mp = p + "mlp."
                names = [mp + "gate_proj.weight", mp + "up_proj.weight"]
                rows = sum(self.flat.params[n].shape[0] for n in names)
                self.fused[f"{i}.gate_up"] = self.flat.fused_view(names, (rows, H))

    def param(self, name: str) -> torch.nn.Parameter:
        return self.flat.params[name]

    # ------------------------------------------------------------------ weights IO
    @torch.no_grad()
    def init_weights(self, seed: int = 1234, std: float = 0.02, per_tensor: bool = False) -> None:
        """Random initialisation (normal, std 0.02; norm weights 0 for ``1+w`` norms, 1 otherwise).

        The same full tensor is generated on every tensor-parallel rank and then
        sharded, so a TP run starts from the weights a dense run would.  ``per_tensor``: every tensor has its own
        generator, seeded by its name, so that a pipeline stage draws for its layers the values a one-stage model
        draws and the two copies of a tied embedding (first and last stage) start equal - the distributed trainer
        initialises this way; by default one generator runs through the stage's tensors in order.
        """
        import zlib
        cfg = self.cfg
        gen = torch.Generator(device="cpu").manual_seed(seed)
        for s in self.specs:
            if per_tensor:
                gen.manual_seed((seed * 1000003 + zlib.crc32(s.name.encode())) & 0x7FFFFFFFFFFFFFFF)
            if s.name.endswith("A_log"):
                full = torch.log(torch.empty(s.full_shape).uniform_(1.0, 8.0, generator=gen))
            elif s.name.endswith("dt_bias"):
                full = torch.empty(s.full_shape).uniform_(-1.0, 1.0, generator=gen)
            elif s.name.endswith("norm.weight") or s.name.endswith("layernorm.weight"):
                gated = s.name.endswith("linear_attn.norm.weight")
                base = 1.0 if (cfg.is_qwen3_moe or gated) else 0.0
                full = torch.full(s.full_shape, base)
            elif s.name.endswith("conv1d.weight"):
                full = torch.empty(s.full_shape).uniform_(-0.5, 0.5, generator=gen)
            else:
                full = torch.empty(s.full_shape).normal_(0.0, std, generator=gen)
            self.load_full_tensor(s.name, full)

    @torch.no_grad()
    def init_weights_on_device(self, seed: int = 1234, std: float = 0.02) -> None:
        """Random initialisation written straight into the flat buffer on its device, tensor by tensor: no full
        tensor is ever built on the host, so a 30 B-parameter model initialises in seconds.  The distributions are
        those of ``init_weights``; the values are not (each local tensor has its own generator, seeded by its
        name, plus the tensor-parallel rank for sharded tensors and the expert-parallel rank for packed expert
        weights, so replicas agree across data-parallel ranks)."""
        import zlib
        cfg, ctx = self.cfg, self.ctx
        dev = self.flat.flat.device
        gen = torch.Generator(device=dev)
        for name, p in self.flat.params.items():
            salt = zlib.crc32(name.encode())
            if name.startswith("__packed_moe"):
                salt ^= 0x9E3779B1 * (ctx.ep_rank + 1) & 0xFFFFFFFF
                sharded = ctx.tp_size > 1
            else:
                spec = self.spec_by_name[name]
                sharded = ctx.tp_size > 1 and tuple(spec.local_shape(ctx.tp_size)) != tuple(spec.full_shape)
            if sharded:
                salt ^= 0x85EBCA6B * (ctx.tp_rank + 1) & 0xFFFFFFFF
            gen.manual_seed((seed * 1000003 + salt) & 0x7FFFFFFFFFFFFFFF)
            t = p.data
            if name.endswith("A_log"):
                t.copy_(torch.log(torch.empty(t.shape, device=dev).uniform_(1.0, 8.0, generator=gen)))
            elif name.endswith("dt_bias"):
                t.copy_(torch.empty(t.shape, device=dev).uniform_(-1.0, 1.0, generator=gen))
            elif name.endswith("norm.weight") or name.endswith("layernorm.weight"):
                gated = name.endswith("linear_attn.norm.weight")
                t.fill_(1.0 if (cfg.is_qwen3_moe or gated) else 0.0)
            elif name.endswith("conv1d.weight"):
                t.copy_(torch.empty(t.shape, device=dev).uniform_(-0.5, 0.5, generator=gen))
            else:
                t.normal_(0.0, std, generator=gen)

    @torch.no_grad()
    def holds(self, spec: ParamSpec) -> bool:
        """False for an expert weight that lives on another expert-parallel rank."""
        if spec.expert < 0:
            return True
        e_local = self.cfg.num_experts // self.ctx.ep_size
        lo = self.ctx.ep_rank * e_local
        return lo <= spec.expert < lo + e_local

    def load_full_tensor(self, name: str, full: torch.Tensor) -> None:
        """Shard a full Hugging Face tensor for this rank and copy it into the flat buffer."""
        spec = self.spec_by_name[name]
        self.load_local_tensor(name, shard_tensor(spec, full, self.ctx.tp_rank, self.ctx.tp_size))

    def load_local_tensor(self, name: str, local: torch.Tensor) -> None:
        """Copy this rank's (already sharded) piece of a Hugging Face tensor into the flat buffer."""
        spec = self.spec_by_name[name]
        cfg, ctx = self.cfg, self.ctx
        if spec.expert >= 0:
            e_local = cfg.num_experts // ctx.ep_size
            lo = ctx.ep_rank * e_local
            if not (lo <= spec.expert < lo + e_local):
                return
            layer = int(name[len(cfg.layer_root):].split(".")[0])
            gu, dn = _packed_moe_names(layer)
            e = spec.expert - lo
            i_local = cfg.moe_intermediate_size // ctx.tp_size
            if name.endswith("gate_proj.weight"):
                self.flat.params[gu].data[e, :i_local].copy_(local)
            elif name.endswith("up_proj.weight"):
                self.flat.params[gu].data[e, i_local:].copy_(local)
            else:
                self.flat.params[dn].data[e].copy_(local)
            return
        self.flat.params[name].data.copy_(local.reshape(self.flat.params[name].shape))

    @torch.no_grad()
    def local_hf_tensors(self):
        """``(name, local shard)`` in Hugging Face naming (per-expert tensors unpacked)."""
        cfg, ctx = self.cfg, self.ctx
        for s in self.specs:
            if s.expert >= 0:
                e_local = cfg.num_experts // ctx.ep_size
                lo = ctx.ep_rank * e_local
                if not (lo <= s.expert < lo + e_local):
                    continue
                layer = int(s.name[len(cfg.layer_root):].split(".")[0])
                gu, dn = _packed_moe_names(layer)
                e = s.expert - lo
                i_local = cfg.moe_intermediate_size // ctx.tp_size
                if s.name.endswith("gate_proj.weight"):
                    yield s.name, self.flat.params[gu].data[e, :i_local]
                elif s.name.endswith("up_proj.weight"):
                    yield s.name, self.flat.params[gu].data[e, i_local:]
                else:
                    yield s.name, self.flat.params[dn].data[e]
            else:
                yield s.name, self.flat.params[s.name].data

    def tp_partial_grad_names(self) -> List[str]:
        """Replicated parameters that act on head-sharded activations: each tensor-parallel rank
        holds only its heads' share of their gradient, so the shares must be summed over TP."""
        cfg = self.cfg
        names = []
        for i in range(self.layer_begin, self.layer_end):
            p = f"{cfg.layer_root}{i}."
            if cfg.layer_types[i] == "full_attention":
                names += [p + "self_attn.q_norm.weight", p + "self_attn.k_norm.weight"]
            else:
                names.append(p + "linear_attn.norm.weight")
            if cfg.is_qwen3_moe:
                # the routing weights multiply expert outputs that are partial sums over the split FFN dimension
                names.append(p + "mlp.gate.weight")
            if self.sequence_parallel:
                # token-sharded layer norms: every rank holds the gradient of its rows only
                names += [p + "input_layernorm.weight", p + "post_attention_layernorm.weight"]
        if self.sequence_parallel and self.last_stage:
            names.append(cfg.final_norm_name)
        return names

    @property
    def sequence_parallel(self) -> bool:
        """True when the tensor-parallel group runs with the residual stream sharded by token rows
        (``parallel/tp_sp.py``); the training forward then requires shapes that path accepts."""
        return getattr(self.ctx, "tp_sp", None) is not None and self.ctx.tp_size > 1

    @torch.no_grad()
    def sync_replicated_grads(self) -> None:
        """Sum the partial gradients of ``tp_partial_grad_names`` over the tensor-parallel group
        (one all-reduce of their concatenation)."""
        if self.ctx.tp_size == 1:
            return
        import torch.distributed as dist
        grads = [self.flat.params[n].main_grad for n in self.tp_partial_grad_names()]
        if not grads:
            return
        flat = torch.cat([g.reshape(-1) for g in grads])
        dist.all_reduce(flat, group=self.ctx.tp_group)
        off = 0
        for g in grads:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()

    @torch.no_grad()
    def sync_bucket_grads(self, bucket: int) -> None:
        """Model-parallel sums of ONE gradient bucket (bucketed gradients: there is no whole-model gradient buffer
        to sum after the backward pass): the tensor-parallel shares of the bucket's ``tp_partial_grad_names``, then
        the context-parallel sum of the whole bucket.  Called by the bucketed optimizer just before it reduces
        the bucket over the data-parallel group."""
        ctx = self.ctx
        tied_pp = (bucket == 0 and ctx.pp_size > 1 and self.cfg.lm_head_name == self.cfg.embed_name
                   and (self.first_stage or self.last_stage) and getattr(ctx, "embed_group", None) is not None)
        if ctx.tp_size == 1 and ctx.cp_size == 1 and ctx.ep_size == 1 and not tied_pp:
            return
        import torch.distributed as dist

        def all_reduce_list(grads, group, scale=1.0):
            if not grads:
                return
            flat = torch.cat([g.reshape(-1) for g in grads])
            dist.all_reduce(flat, group=group)
            if scale != 1.0:
                flat *= scale
            off = 0
            for g in grads:
                g.copy_(flat[off:off + g.numel()].view_as(g))
                off += g.numel()
        if ctx.ep_size > 1:
            # expert-parallel ranks train different micro-batches: everything but the expert weights is a
            # data-parallel replica over that group and takes the mean of the group's gradients
            all_reduce_list([p.main_grad for n, p in self.flat.params.items()
                             if not n.startswith("__packed_moe") and self._bucket_of_entry(n) == bucket],
                            ctx.ep_group, 1.0 / ctx.ep_size)
        if ctx.tp_size > 1:
            grads = [self.flat.params[n].main_grad for n in self.tp_partial_grad_names()
                     if self._bucket_of_entry(n) == bucket]
            if grads:
                flat = torch.cat([g.reshape(-1) for g in grads])
                dist.all_reduce(flat, group=ctx.tp_group)
                off = 0
                for g in grads:
                    g.copy_(flat[off:off + g.numel()].view_as(g))
                    off += g.numel()
        if ctx.cp_size > 1:
            dist.all_reduce(self.flat.bucket_grad(bucket), group=ctx.cp_group)
        if tied_pp:
            # the tied embedding lives on the first and the last pipeline stage: both copies take the sum of the two
            # gradient halves (bucket 0 is reduced once per step, after the last backward pass)
            dist.all_reduce(self.param(self.cfg.embed_name).main_grad, group=ctx.embed_group)

    def trainable_parameters(self) -> List[torch.nn.Parameter]:
        return list(self.flat.params.values())

    # ------------------------------------------------------------------ helpers
    def _rope(self, seq_len: int, device, offset: int = 0):
        key = (seq_len, offset, str(device))
        hit = self._rope_cache.get(key)
        if hit is None:
            hit = ops.rope_tables(seq_len, self.cfg.rotary_dim, self.cfg.rope_theta, device, offset)
            self._rope_cache[key] = hit
        return hit

    def _positions(self, batch: int, seq: int, device) -> torch.Tensor:
        return torch.arange(seq, device=device, dtype=torch.int32).repeat(batch)

    # ------------------------------------------------------------------ tensor-parallel linears
    def _col_linear(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """Column-parallel linear on a replicated input: the input gradient is all-reduced over TP."""
        ctx = self.ctx
        if self._sp_active:
            from ..parallel import tp_sp
            return tp_sp.col_linear(x, w, ctx.tp_sp)
        if ctx.tp_size > 1 and ctx.tp_symm is not None:
            from ..parallel import tp_symm
            if tp_symm.usable(ctx.tp_symm, x, x.reshape(-1, x.shape[-1]).shape[0], x.shape[-1]):
                return tp_symm.column_parallel_linear(x, w, ctx.tp_symm)
        return ops.linear(copy_to_tp(x, ctx.tp_group), w)

    def _row_linear(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """Row-parallel linear on a sharded input: the output is all-reduced over TP."""
        ctx = self.ctx
        if self._sp_active:
            # left reduce-scattered: the result is a handle that only ``tp_sp.norm_gather`` may consume
            from ..parallel import tp_sp
            return tp_sp.row_linear(x, w, ctx.tp_sp)
        if ctx.tp_size > 1 and ctx.tp_symm is not None:
            from ..parallel import tp_symm
            if tp_symm.usable(ctx.tp_symm, x, x.reshape(-1, x.shape[-1]).shape[0], w.shape[0]):
                return tp_symm.row_parallel_linear(x, w, ctx.tp_symm)
        return reduce_from_tp(ops.linear(x, w), ctx.tp_group)

    # ------------------------------------------------------------------ mixers
    def full_attention(self, x: torch.Tensor, i: int, batch: int, seq: int, cache: Optional[dict] = None) -> torch.Tensor:
        cfg, ctx = self.cfg, self.ctx
        p = f"{cfg.layer_root}{i}.self_attn."
        d = cfg.head_dim
        h = cfg.num_attention_heads // ctx.tp_size
        kvh = cfg.num_key_value_heads // ctx.tp_size
        T = x.shape[0]
        qkv = self._col_linear(x, self.fused[f"{i}.qkv"])
        qmul = 1 if cfg.is_qwen3_moe else 2
        q_all, k, v = qkv.split([h * d * qmul, kvh * d, kvh * d], dim=-1)
        if cfg.is_qwen3_moe:
            q, gate = q_all.view(T, h, d), None
        else:
            q, gate = q_all.view(T, h, 2 * d).split([d, d], dim=-1)
        k = k.view(T, kvh, d)
        v = v.view(T, kvh, d)
        cp_off = ctx.cp_rank * seq if ctx.cp_size > 1 else 0     # this shard's first position
        cos, sin = self._rope(seq, x.device, cp_off)
        pos = self._positions(batch, seq, x.device)
        off = cfg.norm_weight_offset
        q = ops.headnorm_rope(q, self.param(p + "q_norm.weight"), cos, sin, pos, cfg.rotary_dim, cfg.rms_norm_eps, off)
        k = ops.headnorm_rope(k, self.param(p + "k_norm.weight"), cos, sin, pos, cfg.rotary_dim, cfg.rms_norm_eps, off)
        if cache is not None:  # prefill of a cached decode: keep the rotated keys and the values
            cache["k"], cache["v"] = k.view(batch, seq, kvh, d), v.reshape(batch, seq, kvh, d)
        zig = False
        if ctx.cp_size > 1 and ctx.cp_zigzag and ctx.cp_symm is None:
            from ..parallel import cp_zigzag as zz
            zig = zz.zigzag_supported(seq, self._cp_original_len or seq * ctx.cp_size, ctx.cp_size) and (
                not q.is_cuda or (seq // 2) % 128 == 0)
        if zig:
            # q | k | v travel to the zig-zag layout as one tensor, the output comes back the same way
            packed = torch.cat([q.reshape(batch, seq, h * d), k.reshape(batch, seq, kvh * d),
                                v.reshape(batch, seq, kvh * d)], dim=-1)
            packed = zz.zigzag_reshard(packed, ctx.cp_group, ctx.cp_rank, ctx.cp_size, True)
            zq, zk, zv = packed.split([h * d, kvh * d, kvh * d], dim=-1)
            o = zz.zigzag_ring_attention(zq.reshape(batch, seq, h, d), zk.reshape(batch, seq, kvh, d),
                                         zv.reshape(batch, seq, kvh, d), ctx.cp_group, ctx.cp_rank, ctx.cp_size,
                                         1.0 / math.sqrt(d))
            o = zz.zigzag_reshard(o.reshape(batch, seq, h * d), ctx.cp_group, ctx.cp_rank, ctx.cp_size, False)
            o = o.reshape(T, h, d)
        elif ctx.cp_size > 1:
            from ..parallel.context_parallel import ring_attention
            o = ring_attention(q.view(batch, seq, h, d).transpose(1, 2), k.view(batch, seq, kvh, d).transpose(1, 2),
                               v.reshape(batch, seq, kvh, d).transpose(1, 2), ctx.cp_group, ctx.cp_rank, ctx.cp_size,
                               self._cp_original_len or seq * ctx.cp_size, 1.0 / math.sqrt(d),
                               symm=ctx.cp_symm, key=i)
            o = o.transpose(1, 2).reshape(T, h, d)
        else:
            o = attn_ops.causal_attention(q, k, v, batch, seq, 1.0 / math.sqrt(d))
        if gate is not None:
            o = ops.siggate(o, gate)
        return self._row_linear(o.reshape(T, h * d), self.param(p + "o_proj.weight"))

    def linear_attention(self, x: torch.Tensor, i: int, batch: int, seq: int,
                         initial_state: Optional[torch.Tensor] = None, return_state: bool = False,
                         cache: Optional[dict] = None):
        cfg, ctx = self.cfg, self.ctx
        p = f"{cfg.layer_root}{i}.linear_attn."
        tp = ctx.tp_size
        kh, vh = cfg.linear_num_key_heads // tp, cfg.linear_num_value_heads // tp
        kd, vd = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        key_dim, value_dim = kh * kd, vh * vd
        conv_dim = 2 * key_dim + value_dim
        T = x.shape[0]
        proj = self._col_linear(x, self.fused[f"{i}.lin_in"])
        mixed, z, b, a = proj.split([conv_dim, value_dim, vh, vh], dim=-1)
        conv_w = self.param(p + "conv1d.weight").view(conv_dim, cfg.linear_conv_kernel_dim)
        if cache is not None:  # the last KW-1 pre-convolution rows seed the decode-time window
            kw = cfg.linear_conv_kernel_dim
            tail = mixed.reshape(batch, seq, conv_dim)[:, max(0, seq - (kw - 1)):]
            if tail.shape[1] < kw - 1:
                tail = F.pad(tail, (0, 0, kw - 1 - tail.shape[1], 0))
            cache["conv"] = tail.clone()
        if ctx.cp_size > 1:
            from ..parallel.context_parallel import conv_halo, recv_initial_state, send_final_state
            halo = cfg.linear_conv_kernel_dim - 1
            ext = conv_halo(mixed.reshape(batch, seq, conv_dim), ctx.cp_group, ctx.cp_rank, ctx.cp_size, halo)
            mixed = ops.conv1d_silu(ext, conv_w)[:, halo:]
            like = torch.zeros(batch, vh, kd, vd, dtype=torch.float32, device=x.device)
            initial_state = recv_initial_state(proj, like, ctx.cp_group, ctx.cp_rank)
        else:
            # one op for "split, then convolve the first group": its backward fills the projection's gradient in
            # place instead of concatenating the groups' gradients
            mixed, z, b, a = ops.conv1d_silu_split(proj.view(batch, seq, proj.shape[-1]), conv_w,
                                                   [conv_dim, value_dim, vh, vh])
        # beta = sigmoid(b), g = -exp(A_log) softplus(a + dt_bias): one kernel each way on the projection's columns
        beta, g = gdn_ops.gdn_gates(b, a, self.param(p + "A_log"), self.param(p + "dt_bias"))
        beta, g = beta.view(batch, seq, vh), g.view(batch, seq, vh)
        # l2norm of q/k and the 1/sqrt(dk) scale on q are applied inside the fused op
        if vh == kh and kd == vd:
            # q | k | v stay packed: the backward kernel writes their gradients into one buffer
            core, state = gdn_ops.gated_delta_rule_packed(mixed, beta, g, initial_state, scale=1.0 / math.sqrt(kd),
                                                          heads=vh)
        else:
            q, k, v = mixed.split([key_dim, key_dim, value_dim], dim=-1)
            q = q.reshape(batch, seq, kh, kd)
            k = k.reshape(batch, seq, kh, kd)
            v = v.reshape(batch, seq, vh, vd)
            if vh // kh > 1:
                q = q.repeat_interleave(vh // kh, dim=2)
                k = k.repeat_interleave(vh // kh, dim=2)
            core, state = gdn_ops.gated_delta_rule_fused(q, k, v, beta, g, initial_state, scale=1.0 / math.sqrt(kd))
        core = core.to(x.dtype).reshape(T, vh, vd)
        if ctx.cp_size > 1:  # hand the state on; the zero token ties the send into the backward pass
            core = core + send_final_state(state, ctx.cp_group, ctx.cp_rank, ctx.cp_size).to(core.dtype)
        # z goes in as the projection's column range: the norm reads it (and writes its gradient) in place
        y = ops.gated_rmsnorm(core, z, self.param(p + "norm.weight"), cfg.rms_norm_eps)
        out = self._row_linear(y.reshape(T, value_dim), self.param(p + "out_proj.weight"))
        if cache is not None:
            cache["state"] = state
        return (out, state) if return_state else out

    def mlp(self, x: torch.Tensor, i: int) -> torch.Tensor:
        cfg, ctx = self.cfg, self.ctx
        if cfg.is_qwen3_moe:
            from .moe import moe_mlp
            return moe_mlp(self, x, i)
        p = f"{cfg.layer_root}{i}.mlp."
        gu = self._col_linear(x, self.fused[f"{i}.gate_up"])
        act = ops.swiglu(gu)
        return self._row_linear(act, self.param(p + "down_proj.weight"))

    # ------------------------------------------------------------------ forward
    def embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        """[B, S] ids -> packed [B*S, H] embeddings (vocab-parallel over TP)."""
        cfg, ctx = self.cfg, self.ctx
        table = self.param(cfg.embed_name)
        lo = ctx.tp_rank * table.shape[0] if ctx.tp_size > 1 else 0
        e = ops.embedding(input_ids.reshape(-1), table, lo)
        if self._sp_active:
            from ..parallel.autograd_collectives import reduce_scatter_rows
            return reduce_scatter_rows(e, ctx.tp_group)          # this rank's token rows of the sum
        return reduce_from_tp(e, ctx.tp_group)

    def _forward_layers_sp(self, x_local: torch.Tensor, batch: int, seq: int) -> torch.Tensor:
        """Sequence-parallel layer stack: ``x_local`` holds this rank's token rows; every residual add + RMSNorm
        runs on those rows only and hands the gathered result to the next column-parallel GEMM; every
        row-parallel GEMM leaves its output reduce-scattered for the next norm.  Returns the final-normed
        hidden states of ALL tokens ``[B*S, H]``."""
        from ..parallel import tp_sp
        cfg, sp = self.cfg, self.ctx.tp_sp
        eps, off = cfg.rms_norm_eps, cfg.norm_weight_offset
        delta, resid, from_parts = x_local, None, False
        for i in range(self.layer_begin, self.layer_end):
            p = f"{cfg.layer_root}{i}."
            n1, resid = tp_sp.norm_gather(delta, resid, self.param(p + "input_layernorm.weight"), eps, off, sp,
                                          from_parts)
            if cfg.layer_types[i] == "full_attention":
                a = self.full_attention(n1, i, batch, seq)
            else:
                a = self.linear_attention(n1, i, batch, seq)
            n2, resid = tp_sp.norm_gather(a, resid, self.param(p + "post_attention_layernorm.weight"), eps, off, sp,
                                          True)
            delta, from_parts = self.mlp(n2, i), True
        out, _ = tp_sp.norm_gather(delta, resid, self.param(cfg.final_norm_name), eps, off, sp, from_parts,
                                   grad_in_tensor=True)
        return out

    def _layer(self, i: int, delta: torch.Tensor, resid: Optional[torch.Tensor], batch: int, seq: int,
               cache: Optional[dict]):
        """Layer ``i`` on the (delta, residual) pair: norm, attention of the layer's kind, norm, MLP."""
        cfg = self.cfg
        eps, off = cfg.rms_norm_eps, cfg.norm_weight_offset
        p = f"{cfg.layer_root}{i}."
        n1, resid = ops.add_rmsnorm(delta, resid, self.param(p + "input_layernorm.weight"), eps, off)
        if cfg.layer_types[i] == "full_attention":
            a = self.full_attention(n1, i, batch, seq, cache=cache)
        else:
            a = self.linear_attention(n1, i, batch, seq, cache=cache)
        n2, resid = ops.add_rmsnorm(a, resid, self.param(p + "post_attention_layernorm.weight"), eps, off)
        return self.mlp(n2, i), resid

    def forward_layers(self, x: torch.Tensor, batch: int, seq: int, final_norm: bool = True,
                       caches: Optional[list] = None) -> torch.Tensor:
        """Run this stage's layers on the packed residual stream ``x`` ``[B*S, H]``."""
        cfg = self.cfg
        eps, off = cfg.rms_norm_eps, cfg.norm_weight_offset
        delta, resid = x, None
        boundary_ok = torch.is_grad_enabled()
        boundary = self.backward_boundary if boundary_ok else None
        for i in range(self.layer_begin, self.layer_end):
            if boundary is not None:       # backward: layer i (bucket 1 + i - begin) is complete when this fires
                delta, resid = boundary(delta, resid, 1 + i - self.layer_begin)
            cache = None
            if caches is not None:
                cache = {}
                caches.append(cache)
            if self.activation_checkpointing and boundary_ok and cache is None:
                # only (delta, resid) stay alive; the layer runs again when the backward pass reaches it.  No
                # random numbers are drawn in a layer, so there is no generator state to carry
                delta, resid = _checkpoint(self._layer, i, delta, resid, batch, seq, None, use_reentrant=False,
                                           preserve_rng_state=False)
            else:
                delta, resid = self._layer(i, delta, resid, batch, seq, cache)
        if boundary is not None:           # fires before the last layer's backward starts
            delta, resid = boundary(delta, resid, self.layer_end - self.layer_begin + 1)
        if self.last_stage and final_norm:
            out, _ = ops.add_rmsnorm(delta, resid, self.param(cfg.final_norm_name), eps, off)
            return out
        return delta if resid is None else delta + resid

    def forward_hidden(self, input_ids: torch.Tensor) -> torch.Tensor:
        """[B, S] ids -> final-normed hidden states ``[B, S, H]`` (single-stage model)."""
        batch, seq = input_ids.shape
        if self.sequence_parallel:
            sp = self.ctx.tp_sp
            if self.activation_checkpointing:
                raise RuntimeError("activation checkpointing is not combined with the sequence-parallel tensor-parallel "
                                   "path (its peer-mapped buffers are handed from layer to layer in launch order)")
            if not (self.first_stage and self.last_stage) or self.cfg.is_qwen3_moe or self.ctx.cp_size > 1:
                raise RuntimeError("the sequence-parallel tensor-parallel path needs a dense single-stage model")
            if not (sp.fits(batch * seq, self.cfg.hidden_size) and input_ids.is_cuda):
                raise RuntimeError(f"sequence-parallel path: {batch} x {seq} tokens do not fit its buffers "
                                   f"(a multiple of {128 * sp.world} and at most {sp.max_rows})")
            self._sp_active = True
            try:
                sp.begin_pass()
                x = self.embed(input_ids)
                return self._forward_layers_sp(x, batch, seq).view(batch, seq, -1)
            finally:
                self._sp_active = False
        x = self.embed(input_ids)
        return self.forward_layers(x, batch, seq).view(batch, seq, -1)

    def lm_head_weight(self) -> torch.nn.Parameter:
        return self.param(self.cfg.lm_head_name)

    def token_logprobs(self, hidden: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Log-probability of ``targets`` under the LM head at each row of ``hidden`` (fp32)."""
        ctx = self.ctx
        w = self.lm_head_weight()
        lo = ctx.tp_rank * w.shape[0] if ctx.tp_size > 1 else 0
        h2 = hidden.reshape(-1, hidden.shape[-1])
        h2 = copy_to_tp(h2, ctx.tp_group)
        lp = ops.lmhead_logprob(h2, w, targets.reshape(-1), lo, ctx.tp_group if ctx.tp_size > 1 else None)
        return lp.view(targets.shape)

    def response_logprobs(self, input_ids: torch.Tensor, prompt_len: int) -> torch.Tensor:
        """Log-probs of the response tokens ``input_ids[:, P:]`` given their prefixes: [B, R] fp32."""
        if self.ctx.cp_size > 1:
            return self._response_logprobs_cp(input_ids, prompt_len)
        hidden = self.forward_hidden(input_ids)
        R = input_ids.shape[1] - prompt_len
        h = hidden[:, prompt_len - 1: prompt_len - 1 + R]
        return self.token_logprobs(h, input_ids[:, prompt_len:])

    def cp_shard_len(self, seq: int) -> int:
        """Tokens of a ``seq``-token sequence that one context-parallel rank holds (the last shard is padded)."""
        from ..parallel.context_parallel import padded_shard_len
        self._cp_original_len = seq
        return padded_shard_len(seq, self.ctx.cp_size)

    def cp_embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Context parallel, first stage: embeds this rank's contiguous shard of ``[B, S]`` ids -> ``[B * s_loc, H]``."""
        from ..parallel.context_parallel import shard_sequence
        self.cp_shard_len(input_ids.shape[1])
        return self.embed(shard_sequence(input_ids, self.ctx.cp_rank, self.ctx.cp_size, dim=1))

    def cp_response_logprobs(self, hidden: torch.Tensor, input_ids: torch.Tensor, prompt_len: int) -> torch.Tensor:
        """Context parallel, last stage: this rank's final-normed hidden rows ``[B * s_loc, H]`` scored against the
        next tokens of its own positions; the per-position log-probs are all-gathered (the backward of the gather
        is a reduce-scatter, so each rank back-propagates only its shard) and cut to the response: ``[B, R]``."""
        from ..parallel.autograd_collectives import all_gather_rows
        ctx = self.ctx
        B, S = input_ids.shape
        s_loc = self.cp_shard_len(S)
        hidden = hidden.view(B, s_loc, -1)
        # position p predicts token p+1; the final padded position predicts nothing (target 0, masked below)
        nxt = torch.nn.functional.pad(input_ids[:, 1:], (0, s_loc * ctx.cp_size - (S - 1)))
        targets = nxt[:, ctx.cp_rank * s_loc:(ctx.cp_rank + 1) * s_loc]
        lp_local = self.token_logprobs(hidden, targets)                       # [B, s_loc]
        lp_full = all_gather_rows(lp_local.t().contiguous(), ctx.cp_group).t()  # [B, cp*s_loc]
        R = S - prompt_len
        return lp_full[:, prompt_len - 1: prompt_len - 1 + R]

    def _response_logprobs_cp(self, input_ids: torch.Tensor, prompt_len: int) -> torch.Tensor:
        """Context parallel: every rank runs its contiguous shard of the sequence and scores its own positions."""
        B, S = input_ids.shape
        x = self.cp_embed(input_ids)
        hidden = self.forward_layers(x, B, self.cp_shard_len(S))
        return self.cp_response_logprobs(hidden, input_ids, prompt_len)

    def forward_logits(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Full fp32 logits ``[B, S, V]`` (debug / rollout sampling; the trainer never builds them)."""
        hidden = self.forward_hidden(input_ids)
        w = self.lm_head_weight()
        logits = hidden.float() @ w.float().t()
        if self.ctx.tp_size > 1:
            from ..parallel.autograd_collectives import all_gather_rows
            logits = all_gather_rows(logits.permute(2, 0, 1).contiguous(), self.ctx.tp_group).permute(1, 2, 0)
        return logits

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.forward_logits(input_ids)
