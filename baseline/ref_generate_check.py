"""Greedy generation: the reference's rollout worker against this package's cached decode.

    python baseline/ref_generate_check.py [--keep DIR] [--new-tokens 12]

``baseline/ref_generate_check.cc`` runs the reference's ``PolicyRolloutWorker`` (which runs the full forward again for
every new token) over its ``Qwen3_5CausalLmPolicy`` on model directories written by this package, greedy
(temperature 0), once without an EOS and once with the third generated token of the first row as EOS and a host
check every two steps.  ``CachedQwenRolloutWorker`` (prefill + one cached step per token: KV cache, convolution
tail, recurrent state) generates for the same prompts; tokens, lengths and log-probabilities are compared.  One JSON
line per case; exit code 0 when all agree, 3 when the reference library is not built.
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
PROMPTS = "5,6,7,8,9,42;100,3,17,250,11,2;77,1,300,64,8,19"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--keep", default="")
    ap.add_argument("--new-tokens", type=int, default=12)
    a = ap.parse_args(argv)
    import torch

    from cverl_b200.models.config import Qwen35TextConfig
    from cverl_b200.models.hf_io import HfModelLoader, load_model_weights, synthesize_model_dir
    from cverl_b200.models.qwen3_5 import Qwen35Model
    from cverl_b200.rollout.worker import CachedQwenRolloutWorker, GenerationConfig, TokenBatch
    import ref_common
    try:
        exe = ref_common.link_driver(HERE / "ref_generate_check.cc", "ref_generate_check")
    except ref_common.Unavailable as exc:
        print(json.dumps({"unavailable": str(exc)}))
        return 3
    with tempfile.TemporaryDirectory(prefix="cverl_ref_") as tmp:
        work = Path(a.keep) if a.keep else Path(tmp)
        work.mkdir(parents=True, exist_ok=True)
        ids = torch.tensor([[int(t) for t in row.split(",")] for row in PROMPTS.split(";")])
        ok = True
        for moe in (False, True):
            d = synthesize_model_dir(Qwen35TextConfig.tiny(moe=moe), work / f"model_{int(moe)}", seed=23, dtype=torch.float32)
            loader = HfModelLoader(d).load_metadata()
            model = Qwen35Model(loader.config(), dtype=torch.float32)
            load_model_weights(model, loader)
            worker = CachedQwenRolloutWorker(model)
            eos = -1
            for case in ("no_eos", "eos"):
                interval = 0 if case == "no_eos" else 2
                r = subprocess.run([str(exe), str(d), PROMPTS, str(a.new_tokens), str(eos), str(interval)],
                                   capture_output=True, text=True)
                row = {"model": "qwen3_moe" if moe else "qwen3_5", "case": case, "eos": eos}
                if r.returncode != 0:
                    row.update(agree=False, error=r.stderr[-300:])
                    ok = False
                    print(json.dumps(row))
                    continue
                ref = json.loads(r.stdout)
                want = torch.tensor(ref["token_ids"]).reshape(ref["shape"])
                want_lp = torch.tensor(ref["logprobs"]).reshape(ref["shape"])
                got = worker.generate(TokenBatch(ids), GenerationConfig(max_new_tokens=a.new_tokens, temperature=0.0,
                                                                        eos_token_id=eos, eos_check_interval=interval))
                n = min(want.shape[1], got.token_ids.shape[1])
                same_tokens = bool(torch.equal(want[:, :n], got.token_ids[:, :n]))
                lp_diff = float((want_lp[:, :n] - got.logprobs[:, :n]).abs().max())
                same_len = ref.get("lengths") is None or ref["lengths"] == got.lengths.tolist()
                agree = same_tokens and same_len and lp_diff <= 2e-5
                ok = ok and agree
                row.update(tokens_equal=same_tokens, lengths_equal=same_len, largest_logprob_difference=lp_diff,
                           distinct_tokens=int(want.unique().numel()), agree=agree)
                print(json.dumps(row))
                if case == "no_eos":
                    eos = int(want[0, 2])
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
