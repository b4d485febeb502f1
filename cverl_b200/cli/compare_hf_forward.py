"""Forward parity against Hugging Face Transformers on the CPU, in fp32.

``python -m cverl_b200.cli.compare_hf_forward --random qwen3_5 [--tokens 1,2,3,...] [--logits]``
``python -m cverl_b200.cli.compare_hf_forward --model-dir DIR [--layers N] [--logits]``

``--random`` builds a small randomly initialised Transformers model (``Qwen3_5ForCausalLM`` or
``Qwen3MoeForCausalLM``), loads the very same tensors into this package's model under the reference's tensor names
and compares final hidden states (or logits): maximum / mean absolute error, the error relative to the largest
reference value, ``allclose`` at the given tolerances and, for logits, the top-5 ids of the last position.
``--model-dir`` does the same for a checkpoint directory that Transformers can load.  Exit code 0 when allclose.
The reference's tool runs its C++ forward executable against Transformers the same way
(tools/model/compare_qwen3_5_forward.py).
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from ..models.config import Qwen35TextConfig
from ..models.qwen3_5 import Qwen35Model

TINY = dict(vocab_size=512, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
            head_dim=32, intermediate_size=128)


def _random_pair(kind: str, seed: int):
    """(Transformers model, this package's model) holding identical random weights."""
    torch.manual_seed(seed)
    if kind == "qwen3_5":
        from transformers.models.qwen3_5 import Qwen3_5ForCausalLM, Qwen3_5TextConfig
        hf_cfg = Qwen3_5TextConfig(**TINY, linear_key_head_dim=16, linear_value_head_dim=16, linear_num_key_heads=2,
                                   linear_num_value_heads=4, tie_word_embeddings=True)
        hf = Qwen3_5ForCausalLM(hf_cfg)
        rope = getattr(hf_cfg, "rope_parameters", None) or {}
        cfg = Qwen35TextConfig(**TINY, linear_key_head_dim=16, linear_value_head_dim=16, linear_num_key_heads=2,
                               linear_num_value_heads=4, rms_norm_eps=hf_cfg.rms_norm_eps,
                               rope_theta=float(rope.get("rope_theta", getattr(hf_cfg, "rope_theta", 1e4))),
                               partial_rotary_factor=float(rope.get("partial_rotary_factor", 0.25)),
                               tie_word_embeddings=True, layer_types=list(hf_cfg.layer_types))
        rename = lambda n: n.replace("model.", "model.language_model.", 1) if n.startswith("model.") else n
    else:
        from transformers.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeForCausalLM
        hf_cfg = Qwen3MoeConfig(**TINY, moe_intermediate_size=48, num_experts=8, num_experts_per_tok=2,
                                norm_topk_prob=True, tie_word_embeddings=False, decoder_sparse_step=1,
                                mlp_only_layers=[], output_router_logits=False)
        hf = Qwen3MoeForCausalLM(hf_cfg)
        rope = getattr(hf_cfg, "rope_parameters", None) or {}
        cfg = Qwen35TextConfig(model_type="qwen3_moe", **TINY, moe_intermediate_size=48, num_experts=8,
                               num_experts_per_tok=2, norm_topk_prob=True, tie_word_embeddings=False,
                               rms_norm_eps=hf_cfg.rms_norm_eps,
                               rope_theta=float(rope.get("rope_theta", getattr(hf_cfg, "rope_theta", 1e4))))
        rename = lambda n: n
    # random, non-trivial values everywhere (Transformers initialises norms to ones and gates to constants)
    with torch.no_grad():
        for name, p in hf.named_parameters():
            if name.endswith("A_log"):
                p.copy_(torch.log(torch.empty_like(p).uniform_(1.0, 8.0)))
            elif p.dim() == 1:
                p.copy_(torch.empty_like(p).uniform_(-0.5, 0.5) + (0.0 if "norm" in name and kind == "qwen3_5"
                                                                     and "linear_attn.norm" not in name else 1.0))
            else:
                p.normal_(0.0, 0.05)
    hf = hf.float().eval()
    ours = Qwen35Model(cfg, dtype=torch.float32, device="cpu", with_main_grad=False)
    state = {rename(k): v.detach() for k, v in hf.state_dict().items()}
    if kind == "qwen3_moe" and not any(".mlp.experts.0." in k for k in state):
        # Transformers keeps the experts packed as [E, 2I, H] / [E, H, I]: unpack to the per-expert names
        for k in [k for k in list(state) if k.endswith("mlp.experts.gate_up_proj") or k.endswith("mlp.experts.down_proj")]:
            t = state.pop(k)
            root = k.rsplit(".", 1)[0]
            for e in range(t.shape[0]):
                if k.endswith("gate_up_proj"):
                    gu = t[e] if t.shape[1] == 2 * cfg.moe_intermediate_size else t[e].t()
                    state[f"{root}.{e}.gate_proj.weight"] = gu[:cfg.moe_intermediate_size].contiguous()
                    state[f"{root}.{e}.up_proj.weight"] = gu[cfg.moe_intermediate_size:].contiguous()
                else:
                    dn = t[e] if t.shape[0 + 1] == cfg.hidden_size else t[e].t()
                    state[f"{root}.{e}.down_proj.weight"] = dn.contiguous()
    missing = [s.name for s in ours.specs if s.name not in state]
    if missing:
        raise RuntimeError(f"Transformers state dict lacks {missing[:4]} ...")
    for s in ours.specs:
        ours.load_full_tensor(s.name, state[s.name].float())
    return hf, ours


def _from_dir(model_dir: str, layers):
    from transformers import AutoModelForCausalLM
    from ..models.hf_io import HfModelLoader, load_model_weights
    hf = AutoModelForCausalLM.from_pretrained(model_dir, torch_dtype=torch.float32).eval()
    loader = HfModelLoader(model_dir).load_metadata()
    cfg = loader.config()
    if layers:
        cfg = Qwen35TextConfig(**{**{k: getattr(cfg, k) for k in cfg.__dataclass_fields__},
                                  "num_hidden_layers": layers, "layer_types": cfg.layer_types[:layers]})
        hf.config.num_hidden_layers = layers
        inner = hf.model.language_model if hasattr(hf.model, "language_model") else hf.model
        inner.layers = inner.layers[:layers]
    ours = Qwen35Model(cfg, dtype=torch.float32, device="cpu", with_main_grad=False)
    load_model_weights(ours, loader)
    return hf, ours


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("model_dir_positional", nargs="?", default="", help="model directory (the reference's argv[1])")
    ap.add_argument("--random", choices=["qwen3_5", "qwen3_moe"])
    ap.add_argument("--model-dir", default="")
    ap.add_argument("--tokens", default="1,7,3,250,9,42,100,5,17,8,300,2")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--logits", action="store_true")
    ap.add_argument("--rtol", type=float, default=1e-3)
    ap.add_argument("--atol", type=float, default=1e-3)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    a.model_dir = a.model_dir or a.model_dir_positional
    if not a.random and not a.model_dir:
        ap.error("give a model directory or --random")
    tokens = [int(t) for t in a.tokens.split(",") if t]
    if not tokens:
        raise SystemExit("--tokens must contain at least one id")
    try:
        hf, ours = _random_pair(a.random, a.seed) if a.random else _from_dir(a.model_dir, a.layers)
    except ImportError as exc:
        print(json.dumps({"unavailable": f"transformers cannot provide the model: {exc}"}))
        return 3
    ids = torch.tensor([tokens], dtype=torch.long)
    with torch.no_grad():
        out = hf(input_ids=ids, output_hidden_states=not a.logits)
        ref = out.logits.float() if a.logits else out.hidden_states[-1].float()
        mine = (ours.forward_logits(ids) if a.logits else ours.forward_hidden(ids)).float()
    diff = (mine - ref).abs()
    ok = bool(torch.allclose(mine, ref, rtol=a.rtol, atol=a.atol))
    report = {"tokens": tokens, "logits": a.logits, "shape": list(mine.shape), "max_abs": diff.max().item(),
              "mean_abs": diff.mean().item(), "ref_abs_max": ref.abs().max().item(),
              "rel_max": diff.max().item() / max(ref.abs().max().item(), 1e-12), "allclose": ok}
    if a.logits:
        report["ours_top5"] = mine[0, -1].topk(5).indices.tolist()
        report["hf_top5"] = ref[0, -1].topk(5).indices.tolist()
    print(json.dumps(report, indent=2))
    return 0 if ok else 2


if __name__ == "__main__":
    sys.exit(main())
