#!/usr/bin/env python
"""Random-init Hugging Face model directories for the reference arm of the benchmarks.

Writes ``config.json`` plus one ``model.safetensors`` with the tensor names the reference's
loader asks for (src/model/qwen3_5_text.cc:528-543,623-680) and the same initial distributions
the framework's own ``Qwen35Model.init_weights`` uses (normal std 0.02 matrices, zero ``1+w``
norm weights, ``A_log = log U(1, 8)``, ``dt_bias = U(-1, 1)``).  Pure ``torch`` + ``json``: it
imports nothing of ``cverl_b200`` so the reference arm stays free of this framework's code.

The safetensors layout is the public one: 8-byte little-endian header length, a JSON header
``{name: {dtype, shape, data_offsets}}``, then the raw tensor bytes.
"""
from __future__ import annotations

import argparse
import json
import struct
from pathlib import Path

import torch

QWEN3_5_0_8B = dict(
    model_type="qwen3_5", vocab_size=248320, hidden_size=1024, num_hidden_layers=24, num_attention_heads=8,
    num_key_value_heads=2, head_dim=256, intermediate_size=3584, linear_key_head_dim=128, linear_value_head_dim=128,
    linear_num_key_heads=16, linear_num_value_heads=16, linear_conv_kernel_dim=4, rms_norm_eps=1e-6,
    rope_theta=1.0e7, partial_rotary_factor=0.25, tie_word_embeddings=True)

QWEN3_30B_A3B = dict(
    model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, num_hidden_layers=48, num_attention_heads=32,
    num_key_value_heads=4, head_dim=128, intermediate_size=6144, moe_intermediate_size=768, num_experts=128,
    num_experts_per_tok=8, norm_topk_prob=True, rms_norm_eps=1e-6, rope_theta=1.0e6, tie_word_embeddings=False)


def tensor_shapes(cfg: dict, layers: int | None = None):
    """(name, shape) in file order for the first ``layers`` layers (all when None)."""
    moe = cfg["model_type"] == "qwen3_moe"
    h, v = cfg["hidden_size"], cfg["vocab_size"]
    nl = cfg["num_hidden_layers"] if layers is None else min(layers, cfg["num_hidden_layers"])
    root = "model." if moe else "model.language_model."
    out = [(root + "embed_tokens.weight", (v, h)), (root + "norm.weight", (h,))]
    if moe and not cfg.get("tie_word_embeddings", False):
        out.append(("lm_head.weight", (v, h)))
    hq, hkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    for i in range(nl):
        p = f"{root}layers.{i}."
        out += [(p + "input_layernorm.weight", (h,)), (p + "post_attention_layernorm.weight", (h,))]
        full = moe or (i + 1) % 4 == 0
        if full:
            q_rows = hq * d if moe else hq * d * 2          # Qwen3.5 packs the output gate beside q
            out += [(p + "self_attn.q_proj.weight", (q_rows, h)), (p + "self_attn.k_proj.weight", (hkv * d, h)),
                    (p + "self_attn.v_proj.weight", (hkv * d, h)), (p + "self_attn.o_proj.weight", (h, hq * d)),
                    (p + "self_attn.q_norm.weight", (d,)), (p + "self_attn.k_norm.weight", (d,))]
        else:
            kd, vd = cfg["linear_key_head_dim"], cfg["linear_value_head_dim"]
            hk, hv = cfg["linear_num_key_heads"], cfg["linear_num_value_heads"]
            conv = 2 * hk * kd + hv * vd
            out += [(p + "linear_attn.in_proj_qkv.weight", (conv, h)), (p + "linear_attn.in_proj_z.weight", (hv * vd, h)),
                    (p + "linear_attn.in_proj_b.weight", (hv, h)), (p + "linear_attn.in_proj_a.weight", (hv, h)),
                    (p + "linear_attn.conv1d.weight", (conv, 1, cfg["linear_conv_kernel_dim"])),
                    (p + "linear_attn.A_log", (hv,)), (p + "linear_attn.dt_bias", (hv,)),
                    (p + "linear_attn.norm.weight", (vd,)), (p + "linear_attn.out_proj.weight", (h, hv * vd))]
        if moe:
            out.append((p + "mlp.gate.weight", (cfg["num_experts"], h)))
            mi = cfg["moe_intermediate_size"]
            for e in range(cfg["num_experts"]):
                ep = f"{p}mlp.experts.{e}."
                out += [(ep + "gate_proj.weight", (mi, h)), (ep + "up_proj.weight", (mi, h)),
                        (ep + "down_proj.weight", (h, mi))]
        else:
            inter = cfg["intermediate_size"]
            out += [(p + "mlp.gate_proj.weight", (inter, h)), (p + "mlp.up_proj.weight", (inter, h)),
                    (p + "mlp.down_proj.weight", (h, inter))]
    return out


def init_tensor(name: str, shape, moe: bool, gen: torch.Generator) -> torch.Tensor:
    if name.endswith("A_log"):
        return torch.log(torch.empty(shape).uniform_(1.0, 8.0, generator=gen))
    if name.endswith("dt_bias"):
        return torch.empty(shape).uniform_(-1.0, 1.0, generator=gen)
    if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
        gated = name.endswith("linear_attn.norm.weight")
        return torch.full(shape, 1.0 if (moe or gated) else 0.0)
    if name.endswith("conv1d.weight"):
        return torch.empty(shape).uniform_(-0.5, 0.5, generator=gen)
    return torch.empty(shape).normal_(0.0, 0.02, generator=gen)


def write_model_dir(cfg: dict, out_dir, layers: int | None = None, seed: int = 1234) -> Path:
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text(json.dumps(cfg, indent=1))
    shapes = tensor_shapes(cfg, layers)
    header, offset = {"__metadata__": {"format": "pt"}}, 0
    for name, shape in shapes:
        n = 2
        for s in shape:
            n *= s
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - (8 + len(blob)) % 8) % 8)
    gen = torch.Generator(device="cpu").manual_seed(seed)
    moe = cfg["model_type"] == "qwen3_moe"
    tmp = out / "model.safetensors.tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, shape in shapes:
            t = init_tensor(name, shape, moe, gen).to(torch.bfloat16).contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes())
    tmp.rename(out / "model.safetensors")
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("out_dir")
    ap.add_argument("--model", default="qwen3_5_0_8b", choices=["qwen3_5_0_8b", "qwen3_30b_a3b"])
    ap.add_argument("--layers", type=int, default=None)
    args = ap.parse_args()
    cfg = QWEN3_5_0_8B if args.model == "qwen3_5_0_8b" else QWEN3_30B_A3B
    print(write_model_dir(cfg, args.out_dir, args.layers))


if __name__ == "__main__":
    main()
