"""Golden tokenizer fixtures from Hugging Face ``tokenizers``, for testing ``HfBpeTokenizer``.

``python -m cverl_b200.cli.dump_tokenizer_fixtures real --tokenizer-json TOKENIZER.json --out fixtures.json``
``python -m cverl_b200.cli.dump_tokenizer_fixtures train --corpus FILE --vocab-size 600 --out-dir DIR``

``real`` encodes a list of probe strings (built in, or one per line of ``--probes-file``) with the tokenizer the
JSON file describes and writes ``[{"text", "ids", "decoded"}]``.  ``train`` first trains a small byte-level BPE
tokenizer with the Qwen pre-tokenizer pattern on a text file, saves its ``tokenizer.json`` into ``--out-dir`` and
dumps the fixtures beside it - a way to get a tokenizer with real merges when no model download is possible.
The reference's tool does the same with a hand-built synthetic vocabulary
(tools/text/dump_hf_tokenizer_fixtures.py).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

QWEN_PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+"
                r"|\s+(?!\S)|\s+")

PROBES = [
    "Hello world", "hello world", " hello", "abc", "an apple", "Q: What is 2+2?\nA: 4", "1234567890",
    "<|endoftext|>", "a<|im_start|>user\nhi<|im_end|>", "  two  spaces  ", "naïve café — ünïcödé",
    "tabs\tand\nnewlines\r\n\r\n", "it's we're I'll don't THEY'VE", "数学 123 测试", "emoji 🙂 ok", "",
    "x = [i**2 for i in range(10)]  # squares", "The answer is #### 42.", "   ", "\n", "a" * 40,
]


def dump(tokenizer, probes, out_path: Path) -> int:
    rows = []
    for text in probes:
        ids = tokenizer.encode(text, add_special_tokens=False).ids
        rows.append({"text": text, "ids": ids, "decoded": tokenizer.decode(ids, skip_special_tokens=False)})
    out_path.parent.mkdir(parents=True, exist_ok=True)
    out_path.write_text(json.dumps(rows, ensure_ascii=False))
    return len(rows)


def train_tokenizer(corpus: Path, vocab_size: int, out_dir: Path):
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.Sequence([
        pre_tokenizers.Split(Regex(QWEN_PATTERN), behavior="isolated", invert=False),
        pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=vocab_size, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(),
                                  special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"], show_progress=False)
    tok.train([str(corpus)], trainer)
    out_dir.mkdir(parents=True, exist_ok=True)
    tok.save(str(out_dir / "tokenizer.json"))
    return tok


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--probes-file", type=Path, default=None, help="one probe string per line")
    sub = ap.add_subparsers(dest="cmd", required=True)
    real = sub.add_parser("real")
    real.add_argument("--tokenizer-json", type=Path, required=True)
    real.add_argument("--out", type=Path, required=True)
    train = sub.add_parser("train")
    train.add_argument("--corpus", type=Path, required=True)
    train.add_argument("--vocab-size", type=int, default=600)
    train.add_argument("--out-dir", type=Path, required=True)
    a = ap.parse_args(argv)
    try:
        from tokenizers import Tokenizer
    except ImportError:
        print("the 'tokenizers' package is required", file=sys.stderr)
        return 3
    probes = PROBES if a.probes_file is None else a.probes_file.read_text().splitlines()
    if a.cmd == "real":
        n = dump(Tokenizer.from_file(str(a.tokenizer_json)), probes, a.out)
        print(f"wrote {n} fixtures to {a.out}")
    else:
        tok = train_tokenizer(a.corpus, a.vocab_size, a.out_dir)
        n = dump(tok, probes, a.out_dir / "fixtures.json")
        print(f"trained {tok.get_vocab_size()} tokens; wrote {n} fixtures to {a.out_dir / 'fixtures.json'}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
