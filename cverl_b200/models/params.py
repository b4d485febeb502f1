"""Parameter inventory, tensor-parallel sharding rules and the flat buffer.

Every parameter of a pipeline stage lives in ONE flat model-dtype buffer, laid
out in the reference's order (src/model/qwen3_5_text.cc:623-680) and padded to
a multiple of the data-parallel size (src/distributed/optimizer_sharding.cc:
40-48), with a twin fp32 ``main_grad`` buffer that backward kernels accumulate
into.  ZeRO shards, checkpoints and the fused optimizer all address that one
buffer.  Adjacent Hugging Face tensors that one GEMM consumes (q/k/v, the four
linear-attention input projections, gate/up) are additionally exposed as a
single fused view, so the fusion costs no copy and the checkpoint names stay
the Hugging Face ones.

Megatron sharding rules follow src/model/qwen3_5_text.cc:995-1024,1148-1226,
1354-1450 and tools/model/qwen3_5_pp_tp_ppo_trainer.cc:422-493: attention by
heads, linear attention by linear heads (q/k/v sections separately), MLP by the
FFN dimension, embedding by vocabulary rows, experts contiguous by id over EP.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .config import Qwen35TextConfig


@dataclass(frozen=True)
class ParamSpec:
    name: str
    full_shape: Tuple[int, ...]
    # how the tensor is split over TP: None (replicated), ("rows", sections) or ("cols", sections);
    # sections are the sizes of independently sharded row/column blocks of the FULL tensor
    tp: Optional[Tuple[str, Tuple[int, ...]]] = None
    expert: int = -1  # expert index for per-expert MoE tensors

    def local_shape(self, tp_size: int) -> Tuple[int, ...]:
        if self.tp is None or tp_size == 1:
            return self.full_shape
        axis, sections = self.tp
        n = sum(s // tp_size for s in sections)
        if axis == "rows":
            return (n,) + tuple(self.full_shape[1:])
        return (self.full_shape[0], n) + tuple(self.full_shape[2:])


def _check_div(what: str, n: int, tp: int) -> None:
    if n % tp != 0:
        raise ValueError(f"{what}={n} is not divisible by tensor-parallel size {tp}")


def layer_param_specs(cfg: Qwen35TextConfig, i: int) -> List[ParamSpec]:
    p = f"{cfg.layer_root}{i}."
    H, d = cfg.hidden_size, cfg.head_dim
    h, kvh = cfg.num_attention_heads, cfg.num_key_value_heads
    out: List[ParamSpec] = [
        ParamSpec(p + "input_layernorm.weight", (H,)),
        ParamSpec(p + "post_attention_layernorm.weight", (H,)),
    ]
    if cfg.layer_types[i] == "full_attention":
        sa = p + "self_attn."
        qrows = h * d * (1 if cfg.is_qwen3_moe else 2)  # Qwen3.5 q_proj also emits the output gate
        out += [
            ParamSpec(sa + "q_proj.weight", (qrows, H), ("rows", (qrows,))),
            ParamSpec(sa + "k_proj.weight", (kvh * d, H), ("rows", (kvh * d,))),
            ParamSpec(sa + "v_proj.weight", (kvh * d, H), ("rows", (kvh * d,))),
            ParamSpec(sa + "o_proj.weight", (H, h * d), ("cols", (h * d,))),
            ParamSpec(sa + "q_norm.weight", (d,)),
            ParamSpec(sa + "k_norm.weight", (d,)),
        ]
    else:
        la = p + "linear_attn."
        kdim, vdim, vh = cfg.linear_key_dim, cfg.linear_value_dim, cfg.linear_num_value_heads
        out += [
            ParamSpec(la + "in_proj_qkv.weight", (cfg.linear_conv_dim, H), ("rows", (kdim, kdim, vdim))),
            ParamSpec(la + "in_proj_z.weight", (vdim, H), ("rows", (vdim,))),
            ParamSpec(la + "in_proj_b.weight", (vh, H), ("rows", (vh,))),
            ParamSpec(la + "in_proj_a.weight", (vh, H), ("rows", (vh,))),
            ParamSpec(la + "conv1d.weight", (cfg.linear_conv_dim, 1, cfg.linear_conv_kernel_dim),
                      ("rows", (kdim, kdim, vdim))),
            ParamSpec(la + "A_log", (vh,), ("rows", (vh,))),
            ParamSpec(la + "dt_bias", (vh,), ("rows", (vh,))),
            ParamSpec(la + "norm.weight", (cfg.linear_value_head_dim,)),
            ParamSpec(la + "out_proj.weight", (H, vdim), ("cols", (vdim,))),
        ]
    if cfg.is_qwen3_moe:
        out.append(ParamSpec(p + "mlp.gate.weight", (cfg.num_experts, H)))
        I = cfg.moe_intermediate_size
        for e in range(cfg.num_experts):
            ep = f"{p}mlp.experts.{e}."
            out += [
                ParamSpec(ep + "gate_proj.weight", (I, H), ("rows", (I,)), expert=e),
                ParamSpec(ep + "up_proj.weight", (I, H), ("rows", (I,)), expert=e),
                ParamSpec(ep + "down_proj.weight", (H, I), ("cols", (I,)), expert=e),
            ]
    else:
        mp = p + "mlp."
        I = cfg.intermediate_size
        out += [
            ParamSpec(mp + "gate_proj.weight", (I, H), ("rows", (I,))),
            ParamSpec(mp + "up_proj.weight", (I, H), ("rows", (I,))),
            ParamSpec(mp + "down_proj.weight", (H, I), ("cols", (I,))),
        ]
    return out


def model_param_specs(cfg: Qwen35TextConfig, layer_begin: int = 0, layer_end: Optional[int] = None,
                      first_stage: bool = True, last_stage: bool = True) -> List[ParamSpec]:
    """Ordered inventory of the Hugging Face tensors a pipeline stage owns.

    Stage ownership follows tools/model/qwen3_5_pp_tp_ppo_trainer.cc:388-399: the
    embedding on the first stage (and on the last one too when tied), the final
    norm and the LM head on the last stage.
    """
    layer_end = cfg.num_hidden_layers if layer_end is None else layer_end
    V, H = cfg.vocab_size, cfg.hidden_size
    out: List[ParamSpec] = []
    tied = cfg.lm_head_name == cfg.embed_name
    if first_stage or (last_stage and tied):
        out.append(ParamSpec(cfg.embed_name, (V, H), ("rows", (V,))))
    if last_stage:
        out.append(ParamSpec(cfg.final_norm_name, (H,)))
        if not tied:
            out.append(ParamSpec("lm_head.weight", (V, H), ("rows", (V,))))
    for i in range(layer_begin, layer_end):
        out += layer_param_specs(cfg, i)
    return out


def required_weight_names(cfg: Qwen35TextConfig, max_layers: int = -1) -> List[str]:
    n = cfg.num_hidden_layers if max_layers < 0 else min(max_layers, cfg.num_hidden_layers)
    return [s.name for s in model_param_specs(cfg, 0, n)]


def shard_tensor(spec: ParamSpec, full: torch.Tensor, tp_rank: int, tp_size: int) -> torch.Tensor:
    """This rank's Megatron shard of a full Hugging Face tensor."""
    if spec.tp is None or tp_size == 1:
        return full
    axis, sections = spec.tp
    dim = 0 if axis == "rows" else 1
    pieces, begin = [], 0
    for s in sections:
        _check_div(spec.name, s, tp_size)
        step = s // tp_size
        pieces.append(full.narrow(dim, begin + tp_rank * step, step))
        begin += s
    return pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=dim)


def unshard_tensor(spec: ParamSpec, shards: Sequence[torch.Tensor]) -> torch.Tensor:
    """Inverse of :func:`shard_tensor` given every rank's shard in rank order."""
    tp_size = len(shards)
    if spec.tp is None or tp_size == 1:
        return shards[0]
    axis, sections = spec.tp
    dim = 0 if axis == "rows" else 1
    blocks, offset = [], 0
    for s in sections:
        step = s // tp_size
        blocks += [sh.narrow(dim, offset, step) for sh in shards]
        offset += step
    return torch.cat(blocks, dim=dim)


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class FlatParams:
    """One flat parameter buffer (+ fp32 main-grad twin) with named views.

    ``entries`` is an ordered list of ``(name, local_shape)``.  ``numel`` is the
    sum of the entry sizes and ``padded_numel`` rounds it up to a multiple of
    ``pad_multiple`` (the data-parallel size, times the vector width the fused
    optimizer wants).

    ``grad_buckets`` (one non-decreasing bucket id per entry) switches the gradient storage from a
    full-size twin to per-bucket buffers, for an optimizer that reduces a bucket as soon as the
    backward pass has finished with it: every bucket starts on a multiple of ``bucket_align``
    elements, the buckets named in ``pinned_buckets`` own a buffer each (gradients that arrive
    throughout the pass: embedding, head), and the others take turns on ``grad_slots`` buffers
    of the largest bucket's size (bucket b uses slot ``b % grad_slots``).  ``main_grad`` is then
    None; ``bucket_grad(b)`` is bucket b's fp32 buffer and each parameter's ``main_grad`` a view of it.
    """

    def __init__(self, entries: Sequence[Tuple[str, Tuple[int, ...]]], dtype=torch.bfloat16, device="cpu",
                 pad_multiple: int = 1, with_main_grad: bool = True, entry_align: int = 8, allocator=None,
                 grad_buckets: Optional[Sequence[int]] = None, bucket_align: int = 8, grad_slots: int = 2,
                 pinned_buckets: Sequence[int] = ()):
        # Entries start on a 16-byte boundary (8 bf16 elements) so that vector loads and TMA can
        # address every tensor in place.  Every tensor of the shipped model shapes has a multiple
        # of 8 elements, for which this is exactly the gap-free concatenation of the reference.
        self.entries = [(n, tuple(s)) for n, s in entries]
        self.offsets: Dict[str, Tuple[int, int]] = {}
        if grad_buckets is not None:
            if len(grad_buckets) != len(self.entries) or any(b < a for a, b in zip(grad_buckets, grad_buckets[1:])):
                raise ValueError("grad_buckets needs one non-decreasing bucket id per entry")
            pad_multiple = _align(pad_multiple, bucket_align)
        off = 0
        starts: List[Tuple[int, int]] = []              # (bucket id, first element)
        for k, (name, shape) in enumerate(self.entries):
            n = 1
            for s in shape:
                n *= s
            if grad_buckets is not None and (k == 0 or grad_buckets[k] != grad_buckets[k - 1]):
                off = _align(off, bucket_align)
                starts.append((grad_buckets[k], off))
            self.offsets[name] = (off, n)
            off += _align(n, entry_align) if entry_align > 1 else n
        self.numel = off
        self.padded_numel = _align(max(off, 1), pad_multiple)
        # ``allocator(numel, dtype) -> zeroed 1-D tensor`` places the buffers elsewhere, e.g. in
        # peer-mapped memory for the symmetric-memory ZeRO path (parameters first, then gradients)
        alloc = allocator or (lambda n, dt: torch.zeros(n, dtype=dt, device=device))
        self.flat = alloc(self.padded_numel, dtype)
        self.main_grad = None
        self.bucket_ids: List[int] = []
        self.bucket_ranges: Dict[int, Tuple[int, int]] = {}
        self._bucket_buf: Dict[int, torch.Tensor] = {}
        self.grad_slot_of: Dict[int, int] = {}          # rotating buckets only
        self.grad_buffers: List[torch.Tensor] = []      # every gradient allocation, in allocation order
        if grad_buckets is None:
            self.main_grad = alloc(self.padded_numel, torch.float32) if with_main_grad else None
        elif with_main_grad:
            for k, (b, begin) in enumerate(starts):
                end = starts[k + 1][1] if k + 1 < len(starts) else self.padded_numel
                self.bucket_ids.append(b)
                self.bucket_ranges[b] = (begin, end)
            pinned = set(pinned_buckets)
            rotating = [b for b in self.bucket_ids if b not in pinned]
            slot_len = max((self.bucket_ranges[b][1] - self.bucket_ranges[b][0] for b in rotating), default=0)
            n_slots = min(max(grad_slots, 1), len(rotating)) if rotating else 0
            slots = [alloc(slot_len, torch.float32) for _ in range(n_slots)]
            self.grad_buffers += slots
            for b in self.bucket_ids:
                lo, hi = self.bucket_ranges[b]
                if b in pinned:
                    self._bucket_buf[b] = alloc(hi - lo, torch.float32)
                    self.grad_buffers.append(self._bucket_buf[b])
                else:
                    self.grad_slot_of[b] = b % n_slots
                    self._bucket_buf[b] = slots[b % n_slots][:hi - lo]
        self._with_grad = with_main_grad
        self.params: Dict[str, torch.nn.Parameter] = {}
        for name, shape in self.entries:
            self.params[name] = self._make_param(name, *self.offsets[name], shape)

    @property
    def bucketed(self) -> bool:
        return bool(self.bucket_ids)

    def bucket_grad(self, b: int) -> torch.Tensor:
        """Bucket b's fp32 gradient buffer (its slot's first ``end - begin`` elements)."""
        return self._bucket_buf[b]

    def bucket_of_offset(self, off: int) -> int:
        for b in self.bucket_ids:
            lo, hi = self.bucket_ranges[b]
            if lo <= off < hi:
                return b
        raise ValueError(f"offset {off} is outside every gradient bucket")

    def _grad_view(self, off: int, n: int) -> Optional[torch.Tensor]:
        if self.main_grad is not None:
            return self.main_grad[off:off + n]
        if not self.bucket_ids:
            return None
        b = self.bucket_of_offset(off)
        lo, hi = self.bucket_ranges[b]
        if off + n > hi:
            raise ValueError("a parameter view crosses a gradient-bucket boundary")
        return self._bucket_buf[b][off - lo:off - lo + n]

    def _make_param(self, name, off, n, shape) -> torch.nn.Parameter:
        p = torch.nn.Parameter(self.flat[off:off + n].view(shape), requires_grad=True)
        g = self._grad_view(off, n)
        if g is not None:
            p.main_grad = g.view(shape)
        p.flat_name = name
        return p

    def fused_view(self, names: Sequence[str], shape: Tuple[int, ...]) -> torch.nn.Parameter:
        """A parameter spanning adjacent entries (e.g. q|k|v rows) without copying."""
        first, _ = self.offsets[names[0]]
        total, expect = 0, first
        for nme in names:
            off, n = self.offsets[nme]
            if off != expect:
                raise ValueError(f"entries {names} are not adjacent in the flat buffer")
            expect = off + n
            total += n
        return self._make_param("+".join(names), first, total, shape)

    def zero_grad(self) -> None:
        if self.main_grad is not None:
            self.main_grad.zero_()
        for g in self.grad_buffers:
            g.zero_()

    def named_tensors(self):
        for name, shape in self.entries:
            off, n = self.offsets[name]
            yield name, self.flat[off:off + n].view(shape)
