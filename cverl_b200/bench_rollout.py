"""Rollout (generation) throughput of the cached native decode, in tokens per second.

``python -m cverl_b200.bench_rollout [--batch 128] [--prompt-len 256] [--new-tokens 1024] [--baseline-tokens 8]``

Qwen3.5-0.8B shape, random-init bf16 weights, uniform random prompt ids.  Timed with CUDA events after a warm-up
generation: the prompt prefill, then ``new-tokens`` decode steps replayed from one CUDA graph (tcgen05 GEMMs,
``cvb_decode_attention``, ``cvb_gdn_decode_step``), greedy sampling on the device.  ``--baseline-tokens N`` also
times ``PolicyRolloutWorker`` - the reference's algorithm, which re-runs the full forward over prompt + prefix
for every token (src/rollout/policy_worker.cc:99-102) - for N tokens on the same model and reports its
tokens/s at that (short, therefore favourable) prefix length.  One JSON line.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--new-tokens", type=int, default=1024)
    ap.add_argument("--baseline-tokens", type=int, default=4)
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer layers")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    from . import _native as nv
    from .models.config import Qwen35TextConfig
    from .models.decode import GraphedDecoder, prefill
    from .models.qwen3_5 import Qwen35Model
    dev = torch.device("cuda", 0)
    cfg = Qwen35TextConfig.qwen3_5_0_8b() if not a.layers else Qwen35TextConfig(num_hidden_layers=a.layers)
    model = Qwen35Model(cfg, dtype=torch.bfloat16, device=dev, with_main_grad=False)
    model.init_weights(seed=1)
    g = torch.Generator(device=dev).manual_seed(0)
    prompts = torch.randint(1, cfg.vocab_size, (a.batch, a.prompt_len), device=dev, generator=g)

    def generate(n):
        with torch.no_grad():
            state, logits = prefill(model, prompts, max_len=a.prompt_len + n)
            dec = GraphedDecoder(model, state, a.batch)
            tok = logits.argmax(-1)
            for _ in range(n - 1):
                tok = dec.step(tok).argmax(-1)
        return tok

    generate(8)                                     # warm-up: lazy initialisation, graph pools
    torch.cuda.synchronize()
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    e0.record()
    with torch.no_grad():
        state, logits = prefill(model, prompts, max_len=a.prompt_len + a.new_tokens)
        dec = GraphedDecoder(model, state, a.batch)
    e1.record()
    with torch.no_grad():
        tok = logits.argmax(-1)
        for _ in range(a.new_tokens - 1):
            tok = dec.step(tok).argmax(-1)
    e2.record()
    torch.cuda.synchronize()
    nv.check_status(dev)
    setup_ms, decode_ms = e0.elapsed_time(e1), e1.elapsed_time(e2)
    out = {"metric": "rollout tokens/s (cached native decode, one B200)", "batch": a.batch,
           "prompt_len": a.prompt_len, "new_tokens": a.new_tokens, "prefill_and_capture_ms": setup_ms,
           "decode_ms": decode_ms, "ms_per_token_step": decode_ms / max(1, a.new_tokens - 1),
           "decode_tokens_per_s": a.batch * (a.new_tokens - 1) / (decode_ms / 1e3),
           "end_to_end_tokens_per_s": a.batch * a.new_tokens / ((setup_ms + decode_ms) / 1e3), "dtype": "bf16",
           "data": "uniform random prompt ids, random-init weights, greedy sampling"}
    if a.baseline_tokens > 0:
        from .models.policy import Qwen3_5CausalLmPolicy
        from .rollout.worker import GenerationConfig, PolicyRolloutWorker, TokenBatch
        policy = Qwen3_5CausalLmPolicy(cfg, torch.bfloat16, dev, pad_id=0)
        policy.model.flat.flat.copy_(model.flat.flat)
        worker = PolicyRolloutWorker(policy)
        cfg_gen = GenerationConfig(max_new_tokens=a.baseline_tokens, temperature=0.0, eos_token_id=-1, seed=0)
        batch = TokenBatch(prompts, torch.ones_like(prompts), torch.full((a.batch,), a.prompt_len, device=dev))
        worker.generate(TokenBatch(prompts[:, :128], torch.ones_like(prompts[:, :128]),
                                   torch.full((a.batch,), 128, device=dev)),
                        GenerationConfig(max_new_tokens=2, temperature=0.0, eos_token_id=-1, seed=0))
        torch.cuda.synchronize()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        worker.generate(batch, cfg_gen)
        b1.record()
        torch.cuda.synchronize()
        ms = b0.elapsed_time(b1)
        out["recompute_worker"] = {"tokens": a.baseline_tokens, "ms": ms,
                                   "tokens_per_s": a.batch * a.baseline_tokens / (ms / 1e3),
                                   "note": "full forward over prompt + prefix per token, prefix <= "
                                           f"{a.prompt_len + a.baseline_tokens} tokens"}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
