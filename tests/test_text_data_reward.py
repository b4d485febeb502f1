"""Tokenizers, GSM8K reward and the JSONL reader (all served by libcverl.so)."""
import json
from pathlib import Path

import pytest

from cverl_b200.data import load_prompt_answer_jsonl
from cverl_b200.reward import (Gsm8kRewardOptions, compute_gsm8k_reward, compute_gsm8k_rewards,
                               extract_gsm8k_answer, normalize_gsm8k_ground_truth)
from cverl_b200.text import ByteTokenizer, EncodeOptions, HfBpeTokenizer

FIX = Path(__file__).parent / "fixtures"


def test_byte_tokenizer_roundtrip_and_options():
    t = ByteTokenizer()
    assert (t.vocab_size, t.pad_id, t.bos_id, t.eos_id, t.unk_id) == (260, 0, 1, 2, 3)
    ids = t.encode("héllo", EncodeOptions(add_bos=True, add_eos=True))
    assert ids[0] == 1 and ids[-1] == 2 and len(ids) == 2 + len("héllo".encode())
    assert t.decode(ids) == "héllo"
    assert t.decode(ids, skip_special=False) == "<bos>héllo<eos>"
    # the terminator is appended only where the limit leaves room (the reference's rule, checked against its own
    # tokenizer by baseline/ref_rollout_batch_check.py): a cut-off text ends on its last kept byte
    cut = t.encode("abcdefgh", EncodeOptions(add_eos=True, max_tokens=4))
    assert cut == [4 + ord(c) for c in "abcd"]
    assert t.encode("abc", EncodeOptions(add_eos=True, max_tokens=4)) == [4 + ord(c) for c in "abc"] + [2]
    assert t.encode("abcd", EncodeOptions(add_bos=True, add_eos=True, max_tokens=4)) == [1] + [4 + ord(c) for c in "abc"]


def test_hf_bpe_matches_fixture_ids():
    tok = HfBpeTokenizer(FIX / "synthetic_tokenizer.json")
    cases = json.loads((FIX / "synthetic_tokenizer_cases.json").read_text())
    # the reference's discovery rule: the first special token with a usual spelling, in file order
    assert (tok.pad_id, tok.bos_id, tok.eos_id, tok.unk_id) == (0, 1, 0, -1)
    for c in cases:
        ids = tok.encode(c["text"])
        if tok.uses_pcre2 or c["text"].isascii():
            assert ids == c["ids"], c["text"]
        assert tok.decode(ids, skip_special=False) == c["text"]
    assert tok.decode(tok.encode("a<|endoftext|>b"), skip_special=True) == "ab"
    assert tok.encode("x", EncodeOptions(add_eos=True))[-1] == tok.eos_id


def test_gsm8k_reward_rules():
    assert extract_gsm8k_answer("work... #### 5 more #### -7.5") == "-7.5"
    assert extract_gsm8k_answer("no marker 12") is None
    assert extract_gsm8k_answer("no marker 12 and 7.", Gsm8kRewardOptions(method="flexible")) == "7."
    assert normalize_gsm8k_ground_truth("long explanation #### 1,234") == "1234"
    assert normalize_gsm8k_ground_truth(" $1,000 ") == "1000"
    assert compute_gsm8k_reward("the answer is #### 1,234", "1234") == 1.0
    assert compute_gsm8k_reward("the answer is #### 12", "13", Gsm8kRewardOptions(format_score=0.1)) == 0.1
    assert compute_gsm8k_reward("nothing here", "13", Gsm8kRewardOptions(no_answer_score=-1.0)) == -1.0
    # only the last 300 characters are searched
    assert compute_gsm8k_reward("#### 13" + " " * 400, "13") == 0.0
    assert compute_gsm8k_rewards(["#### 1", "#### 2"], ["1", "3"]) == [1.0, 0.0]
    with pytest.raises(ValueError):
        compute_gsm8k_rewards(["a"], [])


def test_jsonl_reader(tmp_path):
    p = tmp_path / "d.jsonl"
    p.write_text('{"question":"a\\n\\u00e9","answer":42}\n\n{"answer":"x","question":"b","z":[1,{"q":"}"}]}\n'
                 '{"question":"c","answer":true}\n')
    rows = load_prompt_answer_jsonl(p, "question", "answer")
    assert [(r.prompt, r.answer) for r in rows] == [("a\né", "42"), ("b", "x"), ("c", "true")]
    assert len(load_prompt_answer_jsonl(p, "question", "answer", max_examples=2)) == 2
    with pytest.raises(ValueError):
        load_prompt_answer_jsonl(p, "missing", "answer")
    with pytest.raises(ValueError):
        load_prompt_answer_jsonl(tmp_path / "nope.jsonl")


def test_bpe_batch_encoding_on_threads_equals_single_calls():
    from cverl_b200.text import EncodeOptions
    tok = HfBpeTokenizer(str(FIX / "synthetic_tokenizer.json"))
    texts = ["hello world", "", "abc abc abc", "<|endoftext|>tail", "naïve café 数学 🙂", "x" * 300] * 7
    single = [tok.encode(t) for t in texts]
    for threads in (1, 4):
        ids, offsets = tok.encode_batch_flat(texts, threads)
        assert offsets[0] == 0 and offsets[-1] == len(ids) == sum(map(len, single))
        assert [ids[offsets[i]:offsets[i + 1]].tolist() for i in range(len(texts))] == single
    opts = EncodeOptions(add_bos=True, add_eos=True, max_tokens=5)
    assert tok.encode_batch(texts[:4], opts, threads=2) == [tok.encode(t, opts) for t in texts[:4]]
    ids, offsets = tok.encode_batch_flat([], 3)
    assert len(ids) == 0 and offsets.tolist() == [0]
    assert isinstance(tok.uses_jit, bool) and isinstance(tok.uses_id_merges, bool)


def test_tokenizer_benchmark_runs_and_all_arms_agree(capsys):
    import json
    from cverl_b200 import bench_tokenizer
    assert bench_tokenizer.main(["--max-mb", "0.25", "--vocab-size", "1500", "--threads", "1", "2", "--repeats", "1"]) == 0
    doc = json.loads(capsys.readouterr().out)
    assert doc["all_arms_same_ids"] and doc["rollout_batch_builder"]["same_tensors"]
    assert doc["encode_mb_per_s"]["ours_batch_1_threads"] > 0 and doc["tokens"] > 1000
