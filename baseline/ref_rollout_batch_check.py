"""The rollout-batch builder against the reference's own function, case by case.

    python baseline/ref_rollout_batch_check.py [--keep DIR] [--cases 40]

``baseline/ref_rollout_batch_check.cc`` feeds JSON cases to the reference's ``build_gsm8k_rollout_batch`` (from the
reference library built by ``baseline/build_ref.py``) with its byte tokenizer and with its BPE tokenizer on
``tests/fixtures/synthetic_tokenizer.json``; the same cases go through this package's builder - the multi-threaded
native one and the Python statement of the rules - and all six tensors are compared: prompts shorter and longer
than the limit, responses as text (with and without the EOS option) and as token ids, empty responses, empty id
lists, both reward methods.  One JSON line per tokenizer; exit code 0 when everything agrees, 3 when the reference
library is not built.
"""
from __future__ import annotations

import argparse
import json
import random
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
FIELDS = ["prompt_ids", "response_ids", "response_mask", "group_ids", "rewards", "token_rewards"]


def make_case(rng: random.Random, vocab_limit: int):
    words = ["the", "answer", "is", "####", "12", "4", "-3", "1,000", "hello", "world", "\n", "so", "x", "2+2", "?", "é"]

    def text(lo, hi):
        return " ".join(rng.choice(words) for _ in range(rng.randrange(lo, hi)))
    prompts = [text(0, 12) for _ in range(rng.randrange(1, 5))]
    answers = [rng.choice(["#### 4", "12", "1,000", "-3", "nothing"]) for _ in prompts]
    samples = []
    for _ in range(rng.randrange(1, 7)):
        ids = [rng.randrange(4, vocab_limit) for _ in range(rng.randrange(0, 30))] if rng.random() < 0.4 else []
        samples.append({"prompt_index": rng.randrange(len(prompts)), "text": text(0, 14), "token_ids": ids})
    return {"prompts": prompts, "answers": answers, "samples": samples, "max_prompt_tokens": rng.choice([4, 8, 64]),
            "max_response_tokens": rng.choice([4, 16, 64]), "method": rng.choice(["strict", "flexible"]),
            "add_eos": rng.random() < 0.7}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--keep", default="")
    ap.add_argument("--cases", type=int, default=40)
    a = ap.parse_args(argv)
    import torch

    from cverl_b200.reward import Gsm8kRewardOptions
    from cverl_b200.rollout.rollout_batch import RolloutSample, build_gsm8k_rollout_batch
    from cverl_b200.text import ByteTokenizer, HfBpeTokenizer
    import ref_common
    fixture = HERE.parent / "tests" / "fixtures" / "synthetic_tokenizer.json"
    try:
        exe = ref_common.link_driver(HERE / "ref_rollout_batch_check.cc", "ref_rollout_batch_check")
    except ref_common.Unavailable as exc:
        print(json.dumps({"unavailable": str(exc)}))
        return 3
    with tempfile.TemporaryDirectory(prefix="cverl_ref_") as tmp:
        work = Path(a.keep) if a.keep else Path(tmp)
        work.mkdir(parents=True, exist_ok=True)
        ok = True
        for kind in ("byte", "bpe"):
            tok = ByteTokenizer() if kind == "byte" else HfBpeTokenizer(str(fixture))
            rng = random.Random(5 if kind == "byte" else 6)
            mismatches = []
            for c in range(a.cases):
                case = make_case(rng, min(tok.vocab_size, 250))
                case_file = work / "case.json"
                case_file.write_text(json.dumps(case))
                r = subprocess.run([str(exe), str(case_file), *([str(fixture)] if kind == "bpe" else [])],
                                   capture_output=True, text=True)
                if r.returncode != 0:
                    mismatches.append({"case": c, "error": r.stderr[-200:]})
                    continue
                ref = json.loads(r.stdout)
                samples = [RolloutSample(s["prompt_index"], s["text"], s["token_ids"] or None) for s in case["samples"]]
                opts = Gsm8kRewardOptions(method=case["method"])
                for threads in (-1, 3):
                    got = build_gsm8k_rollout_batch(tok, case["prompts"], case["answers"], samples, case["max_prompt_tokens"],
                                                    case["max_response_tokens"], opts, threads=threads,
                                                    add_eos=case["add_eos"])
                    mine = {"prompt_ids": got.prompt_ids, "response_ids": got.response_ids,
                            "response_mask": got.response_mask, "group_ids": got.group_ids, "rewards": got.rewards,
                            "token_rewards": got.token_rewards}
                    for f in FIELDS:
                        want = torch.tensor(ref[f]).reshape(mine[f].shape).to(mine[f].dtype)
                        if not torch.equal(want, mine[f]):
                            mismatches.append({"case": c, "field": f, "builder": "python" if threads < 0 else "native"})
            ok = ok and not mismatches
            print(json.dumps({"tokenizer": kind, "cases": a.cases, "mismatches": mismatches[:5], "agree": not mismatches}))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
