"""Host-side text throughput: the BPE tokenizer and the rollout-batch builder.

    python -m cverl_b200.bench_tokenizer [--tokenizer-json F] [--corpus F] [--doc-bytes 4000] [--max-mb 8]

Without ``--tokenizer-json`` a 16,000-entry byte-level BPE vocabulary with the Qwen pre-tokenizer pattern is trained
(Hugging Face ``tokenizers``) on ``--corpus`` (default: the Python standard library's sources, the one sizeable body
of text every installation has).  Arms, all on the same documents and checked to give the same ids:

* this package's tokenizer: one ``encode`` call per document from Python; ``encode_batch_flat`` on 1 .. N threads;
* Hugging Face ``tokenizers`` (Rust): ``encode`` per document and ``encode_batch``, when importable;
* the reference's C++ ``HfBpeTokenizer`` (src/text/hf_bpe_tokenizer.cc), when its objects have been built by
  ``baseline/build_ref.py``: a small driver (``baseline/ref_tokenizer_bench.cc``) is linked against them and run.

Then the GRPO batch builder (128 prompts x 8 samples, 256 + 1024 tokens): the Python loop against the native
multi-threaded builder.  Prints one JSON document.  Nothing here touches a GPU.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import random
import subprocess
import sys
import sysconfig
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def default_corpus(path: Path, max_bytes: int) -> None:
    files = sorted(glob.glob(sysconfig.get_paths()["stdlib"] + "/*.py"))
    n = 0
    with open(path, "w", encoding="utf-8") as f:
        for p in files:
            try:
                text = open(p, encoding="utf-8").read()
            except (OSError, UnicodeDecodeError):
                continue
            f.write(text.replace("\f", " "))
            n += len(text)
            if n >= max_bytes:
                break


def best_of(fn, repeats: int):
    best, out = 1e30, None
    for _ in range(repeats):
        t0 = time.perf_counter()
        out = fn()
        best = min(best, time.perf_counter() - t0)
    return best, out


def reference_arm(tokenizer_json: Path, docs, work: Path, repeats: int):
    """Links and runs the driver against the reference's compiled tokenizer objects; None when they are absent."""
    obj = ROOT / "baseline" / "_ref" / "obj" / "src__text__hf_bpe_tokenizer.cc.o"
    driver = ROOT / "baseline" / "ref_tokenizer_bench.cc"
    if not obj.exists() or not driver.exists():
        return None
    sys.path.insert(0, str(ROOT / "baseline"))
    try:
        import build_ref
        paths = build_ref.find_paths()
        src = build_ref.default_source_dir()
    except Exception as exc:  # noqa: BLE001 - the arm is optional
        return {"unavailable": f"{type(exc).__name__}: {exc}"}
    finally:
        sys.path.pop(0)
    exe = work / "ref_tokenizer_bench"
    cmd = [os.environ.get("CXX", "g++"), "-std=c++17", "-O2", f"-D_GLIBCXX_USE_CXX11_ABI={paths['cxx11_abi']}",
           "-I", str(src / "include"), str(driver), str(obj), str(paths["pcre"]), "-o", str(exe)]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        return {"unavailable": "link failed: " + p.stderr[-300:]}
    doc_file = work / "docs.txt"
    doc_file.write_text("\f".join(docs), encoding="utf-8")
    p = subprocess.run([str(exe), str(tokenizer_json), str(doc_file), str(repeats)], capture_output=True, text=True)
    if p.returncode != 0:
        return {"unavailable": "run failed: " + p.stderr[-300:]}
    return json.loads(p.stdout.strip().splitlines()[-1])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--tokenizer-json", type=Path, default=None)
    ap.add_argument("--corpus", type=Path, default=None)
    ap.add_argument("--vocab-size", type=int, default=16000)
    ap.add_argument("--doc-bytes", type=int, default=4000)
    ap.add_argument("--max-mb", type=float, default=8.0)
    ap.add_argument("--threads", type=int, nargs="*", default=[1, 2, 4, 8])
    ap.add_argument("--repeats", type=int, default=3)
    args = ap.parse_args(argv)
    from .rollout.rollout_batch import RolloutSample, build_gsm8k_rollout_batch
    from .text import HfBpeTokenizer
    result = {"cpus": os.cpu_count()}
    with tempfile.TemporaryDirectory(prefix="cverl_tok_") as tmp:
        work = Path(tmp)
        corpus = args.corpus
        if corpus is None:
            corpus = work / "corpus.txt"
            default_corpus(corpus, int(args.max_mb * 1e6))
        tj = args.tokenizer_json
        if tj is None:
            from .cli.dump_tokenizer_fixtures import train_tokenizer
            train_tokenizer(corpus, args.vocab_size, work)
            tj = work / "tokenizer.json"
        text = corpus.read_text(encoding="utf-8", errors="replace").replace("\f", " ")[:int(args.max_mb * 1e6)]
        docs = [text[i:i + args.doc_bytes] for i in range(0, len(text), args.doc_bytes)]
        nbytes = sum(len(d.encode("utf-8")) for d in docs)
        result.update(docs=len(docs), bytes=nbytes, doc_bytes=args.doc_bytes)
        ours = HfBpeTokenizer(str(tj))
        result["pcre2"], result["jit"], result["id_merges"] = ours.uses_pcre2, ours.uses_jit, ours.uses_id_merges
        arms = {}
        cold = HfBpeTokenizer(str(tj))
        t0 = time.perf_counter()
        ids_flat, offsets = cold.encode_batch_flat(docs, 1)
        arms["ours_1_thread_cold_cache"] = nbytes / (time.perf_counter() - t0) / 1e6
        s, per_doc = best_of(lambda: [ours.encode(d) for d in docs], args.repeats)
        arms["ours_python_call_per_doc"] = nbytes / s / 1e6
        for th in args.threads:
            s, _ = best_of(lambda th=th: ours.encode_batch_flat(docs, th), args.repeats)
            arms[f"ours_batch_{th}_threads"] = nbytes / s / 1e6
        result["tokens"] = int(len(ids_flat))
        same = all(ids_flat[offsets[i]:offsets[i + 1]].tolist() == per_doc[i] for i in range(len(docs)))
        try:
            from tokenizers import Tokenizer as HfTokenizer
            hf = HfTokenizer.from_file(str(tj))
            s, hf_ids = best_of(lambda: [hf.encode(d, add_special_tokens=False).ids for d in docs], args.repeats)
            arms["hf_tokenizers_per_doc"] = nbytes / s / 1e6
            s, _ = best_of(lambda: hf.encode_batch(docs, add_special_tokens=False), args.repeats)
            arms["hf_tokenizers_encode_batch"] = nbytes / s / 1e6
            same = same and hf_ids == per_doc
        except ImportError:
            arms["hf_tokenizers_per_doc"] = None
        ref = reference_arm(Path(tj), docs, work, args.repeats)
        if ref is not None and "mb_per_s" in ref:
            arms["reference_cpp_per_doc"] = ref["mb_per_s"]
            checksum = 0                      # the driver's running hash of every id, in document order
            for t in ids_flat.tolist():
                checksum = (checksum * 1000003 + t) & 0xFFFFFFFFFFFFFFFF
            same = same and ref["tokens"] == len(ids_flat) and ref["checksum"] == checksum
        elif ref is not None:
            result["reference"] = ref
        result["encode_mb_per_s"] = {k: (round(v, 2) if v is not None else None) for k, v in arms.items()}
        result["all_arms_same_ids"] = bool(same)
        # the GRPO batch builder
        rng = random.Random(0)
        prompts = [text[i * 3000:i * 3000 + 1200] for i in range(128)]
        answers = [str(i % 50) for i in range(128)]
        samples = []
        for p in range(128):
            for k in range(8):
                off = rng.randrange(0, max(len(text) - 5000, 1))
                resp = text[off:off + rng.randrange(10, 4000)] + (f"\n#### {p % 50}" if k % 3 == 0 else "")
                samples.append(RolloutSample(p, resp))
        s_py, ref_batch = best_of(lambda: build_gsm8k_rollout_batch(ours, prompts, answers, samples, 256, 1024,
                                                                    threads=-1), 1)
        builder = {"samples": len(samples), "python_loop_ms": round(1e3 * s_py, 2)}
        for th in args.threads:
            s, got = best_of(lambda th=th: build_gsm8k_rollout_batch(ours, prompts, answers, samples, 256, 1024,
                                                                     threads=th), args.repeats)
            builder[f"native_{th}_threads_ms"] = round(1e3 * s, 2)
            import torch
            builder["same_tensors"] = builder.get("same_tensors", True) and all(
                torch.equal(getattr(ref_batch, f), getattr(got, f)) for f in ref_batch.__dataclass_fields__)
        result["rollout_batch_builder"] = builder
    print(json.dumps(result, indent=1))
    return 0 if result["all_arms_same_ids"] and result["rollout_batch_builder"]["same_tensors"] else 1


if __name__ == "__main__":
    sys.exit(main())
