"""The JSONL reader against the reference's own ``load_prompt_answer_jsonl``, on random files.

    python baseline/ref_jsonl_check.py [--keep DIR] [--files 100]

``baseline/ref_jsonl_check.cc`` loads a file with the reference's function (from the reference library built by
``baseline/build_ref.py``).  Random files - strings with escapes and non-ASCII text (raw and as \\u escapes), numbers,
booleans and nulls in the two fields, other fields holding nested values, blank lines, rows that lack a field,
every kind of ``max_examples`` - go through both readers; the rows, or the fact that the file is refused, must agree.
One JSON line; exit code 0 when all agree, 3 when the reference library is not built.
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


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--keep", default="")
    ap.add_argument("--files", type=int, default=100)
    a = ap.parse_args(argv)
    import torch

    from cverl_b200.data import load_prompt_answer_jsonl
    import ref_common
    try:
        exe = ref_common.link_driver(HERE / "ref_jsonl_check.cc", "ref_jsonl_check")
    except ref_common.Unavailable as exc:
        print(json.dumps({"unavailable": str(exc)}))
        return 3
    with tempfile.TemporaryDirectory(prefix="cverl_ref_") as tmp:
        work = Path(a.keep) if a.keep else Path(tmp)
        work.mkdir(parents=True, exist_ok=True)
        rng = random.Random(4)
        alphabet = ["a", "Z", " ", '"', "\\", "/", "\n", "\t", "é", "数", "\U0001F642", "{", "}", ":", ","]

        def text():
            return "".join(rng.choice(alphabet) for _ in range(rng.randrange(0, 10)))
        problems, refused = [], 0
        for k in range(a.files):
            rows = []
            for _ in range(rng.randrange(1, 5)):
                row = {"junk": rng.choice([1, [1, {"a": "b"}], None, "x"]),
                       "prompt": rng.choice([text(), text(), 7, 2.5, True, None, 1e10, -3]),
                       "answer": rng.choice([text(), text(), 42, 0.125, False, 12345678901234])}
                if rng.random() < 0.08:
                    row.pop("answer")
                rows.append(row)
            path = work / "case.jsonl"
            sep = "\n\n" if rng.random() < 0.3 else "\n"
            path.write_text(sep.join(json.dumps(r, ensure_ascii=rng.random() < 0.5) for r in rows) + "\n", encoding="utf-8")
            limit = rng.choice([-1, -1, 0, 1, 2])
            r = subprocess.run([str(exe), str(path), "prompt", "answer", str(limit)], capture_output=True, text=True)
            ref = json.loads(r.stdout)
            try:
                mine = [[e.prompt, e.answer] for e in load_prompt_answer_jsonl(path, "prompt", "answer", limit)]
            except (ValueError, RuntimeError) as exc:
                mine = {"error": str(exc)}
            both_refuse = isinstance(ref, dict) and isinstance(mine, dict)
            refused += int(both_refuse)
            if not (both_refuse or ref == mine):
                problems.append({"file": k, "limit": limit, "reference": str(ref)[:200], "ours": str(mine)[:200]})
        ok = not problems
        print(json.dumps({"files": a.files, "refused_by_both": refused, "problems": problems[:5], "agree": ok}))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
