"""Parity against outside oracles on the CPU: the model forward against Hugging Face Transformers, the BPE
tokenizer against Hugging Face ``tokenizers`` on a freshly trained vocabulary, and the small demo programs."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("kind", ["qwen3_5", "qwen3_moe"])
def test_forward_matches_transformers(kind, capsys):
    pytest.importorskip("transformers")
    from cverl_b200.cli import compare_hf_forward
    rc = compare_hf_forward.main(["--random", kind, "--rtol", "1e-4", "--atol", "1e-4"])
    report = json.loads(capsys.readouterr().out)
    if rc == 3:
        pytest.skip(report["unavailable"])
    assert rc == 0 and report["allclose"] and report["max_abs"] < 1e-4, report
    rc = compare_hf_forward.main(["--random", kind, "--logits", "--rtol", "1e-4", "--atol", "1e-4", "--seed", "3"])
    report = json.loads(capsys.readouterr().out)
    assert rc == 0 and report["ours_top5"] == report["hf_top5"], report


def test_bpe_tokenizer_matches_hf_tokenizers_on_a_trained_vocabulary(tmp_path):
    """A byte-level BPE tokenizer with a few hundred real merges, the Qwen pre-tokenizer pattern and special tokens,
    trained here on the repository's own prose: every probe and every line of the corpus must encode to the ids
    Hugging Face ``tokenizers`` gives, and decode back."""
    pytest.importorskip("tokenizers")
    from tokenizers import Tokenizer
    from cverl_b200.cli import dump_tokenizer_fixtures as dump
    from cverl_b200.text import HfBpeTokenizer
    corpus = tmp_path / "corpus.txt"
    corpus.write_text((ROOT / "README.md").read_text() + "\n" + (ROOT / "cverl_b200" / "ops" / "rl.py").read_text())
    assert dump.main(["train", "--corpus", str(corpus), "--vocab-size", "700", "--out-dir", str(tmp_path / "tok")]) == 0
    fixtures = json.loads((tmp_path / "tok" / "fixtures.json").read_text())
    mine = HfBpeTokenizer(str(tmp_path / "tok" / "tokenizer.json"))
    hf = Tokenizer.from_file(str(tmp_path / "tok" / "tokenizer.json"))
    assert mine.vocab_size == hf.get_vocab_size() and len(fixtures) == len(dump.PROBES)
    for row in fixtures:
        assert mine.encode(row["text"]) == row["ids"], row["text"]
        assert mine.decode(row["ids"], skip_special=False) == row["decoded"], row["text"]
    lines = [ln for ln in corpus.read_text().splitlines() if ln.strip()][:300]
    for ln in lines:
        assert mine.encode(ln) == hf.encode(ln, add_special_tokens=False).ids, ln
    # the fixture file of a real tokenizer (e.g. Qwen3.5's) replays the same way when one is present
    real = os.environ.get("CVERL_QWEN_MODEL_DIR")
    if real and (Path(real) / "tokenizer.json").exists():
        out = tmp_path / "real.json"
        assert dump.main(["real", "--tokenizer-json", str(Path(real) / "tokenizer.json"), "--out", str(out)]) == 0
        big = HfBpeTokenizer(str(Path(real) / "tokenizer.json"))
        for row in json.loads(out.read_text()):
            assert big.encode(row["text"]) == row["ids"], row["text"]


@pytest.fixture(scope="module")
def tiny_dir(tmp_path_factory):
    from cverl_b200.models.config import Qwen35TextConfig
    from cverl_b200.models.hf_io import synthesize_model_dir
    d = tmp_path_factory.mktemp("tiny_model_demo")
    synthesize_model_dir(Qwen35TextConfig.tiny(), d, seed=3, dtype=torch.float32)
    return d


def _run(*args):
    return subprocess.run([sys.executable, "-m", *args], cwd=ROOT, env=dict(os.environ, PYTHONPATH=str(ROOT)),
                          capture_output=True, text=True, timeout=240)


def test_demo_programs(tmp_path, tiny_dir):
    p = _run("cverl_b200.cli.minimal_ppo_step")
    assert p.returncode == 0 and "param_delta=" in p.stdout, p.stderr[-1000:]
    prefix = str(tmp_path / "toy")
    p = _run("cverl_b200.cli.toy_grpo_trainer", "3", "4", "4", "--save-prefix", prefix)
    assert p.returncode == 0 and p.stdout.splitlines()[0] == "step,loss,avg_reward,success_rate,ppo_kl,clipfrac"
    assert len(p.stdout.splitlines()) == 4 and Path(prefix + ".model.pt").exists()
    p = _run("cverl_b200.cli.toy_grpo_trainer", "1", "4", "4", "--load-prefix", prefix)
    assert p.returncode == 0
    p = _run("cverl_b200.cli.hf_embedding_grpo_trainer", str(tiny_dir), "--steps", "3", "--vocab-subset", "32")
    assert p.returncode == 0, p.stderr[-1500:]
    rows = p.stdout.splitlines()
    assert rows[2].startswith("embedding_subset=[32,") and rows[3].startswith("step,loss") and len(rows) == 7
    data = tmp_path / "d.jsonl"
    data.write_text("\n".join(json.dumps({"prompt": f"What is {i}+1?", "answer": f"#### {i + 1}"}) for i in range(9)))
    p = _run("cverl_b200.cli.gsm8k_grpo_bench", "--dataset", str(data), "--steps", "6", "--lr", "0.01")
    assert p.returncode == 0, p.stderr[-1500:]
    kv = dict(ln.split(",", 1) for ln in p.stdout.splitlines())
    assert kv["backend"] == "cverl_b200" and float(kv["train_tokens_per_second"]) > 0 and kv["dataset_rows"] == "9"
    assert float(kv["train_tokens_per_second"]) == pytest.approx(
        6 * 8 * 4 * 16 * 2 / float(kv["seconds"]), rel=1e-3)


def test_mnist_demo_reads_idx_files_and_learns(tmp_path, capsys):
    """The small supervised demo: raw IDX files (big-endian headers) in, falling loss and the reference's CSV columns
    out; a damaged header is refused."""
    import struct
    from cverl_b200.cli import mnist_demo
    x, y = mnist_demo.synthetic_split(2048, 3)
    xt, yt = mnist_demo.synthetic_split(128, 4)
    for stem, (xs, ys) in {"train": (x, y), "t10k": (xt, yt)}.items():
        (tmp_path / f"{stem}-images-idx3-ubyte").write_bytes(
            struct.pack(">iiii", 2051, xs.shape[0], 28, 28) + (xs * 255).to(torch.uint8).numpy().tobytes())
        (tmp_path / f"{stem}-labels-idx1-ubyte").write_bytes(
            struct.pack(">ii", 2049, ys.shape[0]) + ys.to(torch.uint8).numpy().tobytes())
    xr, yr = mnist_demo.load_split(tmp_path, True)
    assert xr.shape == (2048, 1, 28, 28) and torch.equal(yr, y) and float((xr - (x * 255).to(torch.uint8) / 255).abs().max()) < 1e-6
    csv = tmp_path / "m.csv"
    rc = mnist_demo.main(["--data-dir", str(tmp_path), "--device", "cpu", "--batch-size", "64", "--epochs", "2",
                          "--lr", "3e-3", "--metrics-csv", str(csv)])
    out = capsys.readouterr().out
    assert rc == 0 and "mnist_demo finished" in out
    rows = csv.read_text().splitlines()
    assert rows[0] == mnist_demo.COLUMNS and len(rows) == 1 + 2 * 32 + 2
    assert float(rows[-1].split(",")[-1]) > 0.5                      # test accuracy after two epochs
    (tmp_path / "train-labels-idx1-ubyte").write_bytes(struct.pack(">ii", 1234, 2048) + bytes(2048))
    with pytest.raises(ValueError):
        mnist_demo.load_split(tmp_path, True)


def test_cifar10_export_and_resnet_bench(tmp_path, capsys):
    """Parquet of PNG records -> normalised flat tensors + metadata; the ResNet training-step benchmark maps them."""
    import io
    import numpy as np
    import pyarrow as pa
    import pyarrow.parquet as pq
    from PIL import Image
    from cverl_b200.cli import export_cifar10_tensors as ex, resnet_cifar10_bench as rb
    rng = np.random.default_rng(0)
    raw = rng.integers(0, 256, (24, 32, 32, 3), dtype=np.uint8)
    recs = []
    for img in raw:
        buf = io.BytesIO()
        Image.fromarray(img).save(buf, format="PNG")
        recs.append({"bytes": buf.getvalue(), "path": None})
    labels = [int(i % 10) for i in range(24)]
    pq.write_table(pa.table({"img": recs, "label": labels}), tmp_path / "train.parquet")
    meta = ex.export(str(tmp_path / "train.parquet"), str(tmp_path / "out"))
    assert meta["shape"] == [24, 3, 32, 32] and meta["normalized"]
    x, y = rb.load_tensors(tmp_path / "out")
    want = (raw[5].astype(np.float32).transpose(2, 0, 1) / 255.0 - np.asarray(ex.MEAN, np.float32).reshape(3, 1, 1)) \
        / np.asarray(ex.STD, np.float32).reshape(3, 1, 1)
    assert np.allclose(x[5].numpy(), want, atol=1e-6) and y.tolist() == labels
    rc = rb.main(["--data-dir", str(tmp_path / "out"), "--device", "cpu", "--depth", "14", "--width", "8",
                  "--batch-size", "8", "--steps", "2", "--warmup", "1", "--dtype", "float32"])
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and line["images_per_s"] > 0 and line["benchmark"] == "resnet14_cifar10_train_step"
    assert len(rb.BLOCKS[152]) == 4 and sum(rb.BLOCKS[152]) == 50      # 3 * 50 + 2 = 152 layers


def test_demo_launcher_scripts(tmp_path):
    """examples/run_mnist_demo.sh and run_resnet_cifar10_bench.sh map their environment onto the two tools."""
    import os
    import subprocess
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    env = dict(os.environ, PYTHONPATH=str(root), OMP_NUM_THREADS="2", DEVICE="cpu")
    p = subprocess.run(["bash", str(root / "examples" / "run_mnist_demo.sh"), "", "--max-train-batches", "4",
                        "--max-test-batches", "1"], cwd=root, env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "mnist_demo finished" in p.stdout, p.stdout[-800:] + p.stderr[-1500:]
    p = subprocess.run(["bash", str(root / "examples" / "run_resnet_cifar10_bench.sh"), "--width", "8"], cwd=root,
                       env=dict(env, DEPTH="14", STEPS="2", WARMUP="1", BATCH_SIZE="8", DTYPE="float32"),
                       capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "images_per_s" in p.stdout, p.stdout[-800:] + p.stderr[-1500:]


def test_forward_matches_the_reference_itself():
    """``baseline/ref_forward_check.py``: the reference's own forward tool (its source as it is, linked against the
    reference library) and this package's model agree on hidden states and logits of a Qwen3.5 hybrid and a
    Qwen3-MoE model directory written here (fp32, CPU).  Skipped where the reference library has not been built."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    p = subprocess.run([sys.executable, str(root / "baseline" / "ref_forward_check.py")], capture_output=True, text=True,
                       timeout=1200, cwd=root)
    if p.returncode == 3:
        import pytest
        pytest.skip(p.stdout.strip()[-300:])
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-1500:]
    rows = [json.loads(ln) for ln in p.stdout.strip().splitlines() if ln.startswith("{")]
    assert len(rows) == 4 and all(r["agree"] and r["argmax_equal"] and r["max_abs"] < 2e-5 for r in rows)
    assert {(r["model"], r["output"]) for r in rows} == {("qwen3_5", "hidden"), ("qwen3_5", "logits"),
                                                         ("qwen3_moe", "hidden"), ("qwen3_moe", "logits")}


def test_gradients_match_the_reference_itself():
    """``baseline/ref_backward_check.py``: the reference's policy class (linked from the reference library) and this
    package's model back-propagate the same weighted log-likelihood on model directories written here; the loss and
    every parameter gradient agree (Qwen3.5 hybrid: 55 tensors; Qwen3-MoE: every expert that received a token)."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    p = subprocess.run([sys.executable, str(root / "baseline" / "ref_backward_check.py")], capture_output=True, text=True,
                       timeout=1200, cwd=root)
    if p.returncode == 3:
        import pytest
        pytest.skip(p.stdout.strip()[-300:])
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-1500:]
    rows = [json.loads(ln) for ln in p.stdout.strip().splitlines() if ln.startswith("{")]
    assert [r["model"] for r in rows] == ["qwen3_5", "qwen3_moe"] and all(r["agree"] for r in rows)
    assert rows[0]["gradients_compared"] == 55 and rows[1]["gradients_compared"] > 60
    assert all(r["worst_relative_difference"] < 1e-3 for r in rows)


def test_optimizers_match_the_reference_itself():
    """``baseline/ref_optimizer_check.py``: five AdamW steps of the reference's ``FlatAdamW`` and ``Fp32MasterAdamW``
    (with and without fp32 master weights) against this package's: parameters and moments agree to the last bits."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    p = subprocess.run([sys.executable, str(root / "baseline" / "ref_optimizer_check.py")], capture_output=True, text=True,
                       timeout=1200, cwd=root)
    if p.returncode == 3:
        import pytest
        pytest.skip(p.stdout.strip()[-300:])
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-1500:]
    row = json.loads([ln for ln in p.stdout.strip().splitlines() if ln.startswith("{")][-1])
    assert row["agree"] and row["tensors_compared"] == 12 and row["largest_difference"] <= 2e-6


def test_rollout_batch_builder_matches_the_reference_itself():
    """``baseline/ref_rollout_batch_check.py``: random cases through the reference's own ``build_gsm8k_rollout_batch``
    (byte tokenizer and BPE tokenizer) and through this package's two builders give the same six tensors."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    p = subprocess.run([sys.executable, str(root / "baseline" / "ref_rollout_batch_check.py"), "--cases", "12"],
                       capture_output=True, text=True, timeout=1200, cwd=root)
    if p.returncode == 3:
        import pytest
        pytest.skip(p.stdout.strip()[-300:])
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-1500:]
    rows = [json.loads(ln) for ln in p.stdout.strip().splitlines() if ln.startswith("{")]
    assert [r["tokenizer"] for r in rows] == ["byte", "bpe"] and all(r["agree"] and not r["mismatches"] for r in rows)


def test_cached_decode_matches_the_reference_rollout_worker():
    """``baseline/ref_generate_check.py``: greedy generation by the reference's ``PolicyRolloutWorker`` (full forward per
    token) and by this package's cached decode give the same tokens, lengths and log-probabilities on a Qwen3.5
    hybrid and a Qwen3-MoE model, without and with an EOS token."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    p = subprocess.run([sys.executable, str(root / "baseline" / "ref_generate_check.py")], capture_output=True, text=True,
                       timeout=1200, cwd=root)
    if p.returncode == 3:
        import pytest
        pytest.skip(p.stdout.strip()[-300:])
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-1500:]
    rows = [json.loads(ln) for ln in p.stdout.strip().splitlines() if ln.startswith("{")]
    assert len(rows) == 4 and all(r["agree"] and r["tokens_equal"] and r["lengths_equal"] for r in rows)
    assert max(r["largest_logprob_difference"] for r in rows) < 2e-5


def test_planner_matches_the_reference_itself():
    """``baseline/ref_topology_check.py``: random valid and invalid layouts through the reference's own ``Topology`` and
    pipeline schedule and through this package's planner: same verdicts, coordinates, groups, neighbours, layer
    ranges, 1F1B action lists, live-activation peaks and NCCL environment."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    p = subprocess.run([sys.executable, str(root / "baseline" / "ref_topology_check.py"), "--layouts", "40"],
                       capture_output=True, text=True, timeout=1200, cwd=root)
    if p.returncode == 3:
        import pytest
        pytest.skip(p.stdout.strip()[-300:])
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-1500:]
    row = json.loads([ln for ln in p.stdout.strip().splitlines() if ln.startswith("{")][-1])
    assert row["agree"] and row["valid"] > 10 and row["invalid"] > 10 and not row["problems"]


def test_c_abi_matches_the_reference_library_on_random_inputs():
    """The ten ``cverl_*_f32_cpu`` entry points of this package's ``libcverl.so`` and of the reference's library
    (built by ``baseline/build_ref.py``; skipped where it is absent) on random shapes, masks with empty rows, all
    KL kinds, every aggregation mode, plain and dual clipping, single-member groups - same values, and the same
    refusal of mismatched shapes."""
    import random
    from pathlib import Path

    import pytest
    import torch
    from cverl_b200.ops import rl
    lib = Path(__file__).resolve().parents[1] / "baseline" / "_ref" / "lib" / "libcverl_ref.so"
    if not lib.exists():
        pytest.skip("reference library not built (python baseline/build_ref.py)")
    ref, ours = rl._CAbi(str(lib)), rl.c_abi
    rng = random.Random(3)
    torch.manual_seed(3)

    def close(a, b, tol=2e-5):
        a, b = torch.as_tensor(a, dtype=torch.float32), torch.as_tensor(b, dtype=torch.float32)
        assert torch.allclose(a, b, rtol=tol, atol=tol, equal_nan=True), (a.flatten()[:4], b.flatten()[:4])
    for _ in range(120):
        rows, cols = rng.randrange(1, 7), rng.randrange(1, 9)
        v = torch.randn(rows, cols) * rng.choice([1, 5, 0.01])
        w = torch.randn(rows, cols)
        m = (torch.rand(rows, cols) < rng.choice([0.3, 0.8, 1.0])).float()
        if rng.random() < 0.2:
            m[rng.randrange(rows)] = 0
        close(ref.masked_sum(v, m), ours.masked_sum(v, m))
        close(ref.masked_mean(v, m), ours.masked_mean(v, m))
        if m.sum() > 1:
            for shift in (True, False):
                close(ref.masked_whiten(v, m, shift), ours.masked_whiten(v, m, shift), 1e-4)
            a1, r1 = ref.gae(v, w, m, 0.99, 0.95)
            a2, r2 = ours.gae(v, w, m, 0.99, 0.95)
            close(a1, a2, 2e-4)
            close(r1, r2, 2e-4)
        for kind in ("k1", "abs", "k2", "k3"):
            close(ref.kl_penalty(v, w, kind), ours.kl_penalty(v, w, kind), 1e-4)
            close(ref.kl_penalty(v, w, kind, backward=True), ours.kl_penalty(v, w, kind, backward=True), 1e-4)
        gid = torch.tensor([rng.randrange(0, 3) for _ in range(rows)])
        for norm in (True, False):
            close(ref.grpo(v, m, gid, 1e-6, norm)[0], ours.grpo(v, m, gid, 1e-6, norm)[0], 2e-4)
        if m.sum() == 0:
            continue
        old = torch.randn(rows, cols) * 0.3 - 2
        lp = old + torch.randn(rows, cols) * rng.choice([0.05, 0.5, 30.0])
        adv = torch.randn(rows, cols)
        for agg in (0, 1, 2):
            for clip, lo, hi, c in ((0.2, -1.0, -1.0, 3.0), (0.2, 0.1, 0.3, 1.5)):
                close(ref.ppo_loss(old, lp, adv, m, clip, lo, hi, c, agg), ours.ppo_loss(old, lp, adv, m, clip, lo, hi, c, agg), 2e-4)
                close(ref.ppo_loss_backward(old, lp, adv, m, clip, lo, hi, c, agg),
                      ours.ppo_loss_backward(old, lp, adv, m, clip, lo, hi, c, agg), 2e-4)
    bad_mask = torch.ones(2, 3)
    for side in (ref, ours):
        with pytest.raises(ValueError):
            side.masked_sum(torch.ones(2, 4), bad_mask)
        with pytest.raises(ValueError):
            side.ppo_loss(torch.ones(2, 4), torch.ones(2, 4), torch.ones(2, 4), bad_mask)
        with pytest.raises(ValueError):
            side.ppo_loss(torch.ones(2, 3), torch.ones(2, 3), torch.ones(2, 3), bad_mask, c=1.0)   # dual clip needs c > 1


def test_jsonl_reader_matches_the_reference_itself():
    """``baseline/ref_jsonl_check.py``: random JSONL files through the reference's own ``load_prompt_answer_jsonl`` and
    through this package's reader: same rows (numbers and booleans as their JSON text, null as the empty string,
    ``max_examples`` 0 = no row, negative = all), same refusals."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    p = subprocess.run([sys.executable, str(root / "baseline" / "ref_jsonl_check.py"), "--files", "30"],
                       capture_output=True, text=True, timeout=1200, cwd=root)
    if p.returncode == 3:
        import pytest
        pytest.skip(p.stdout.strip()[-300:])
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-1500:]
    row = json.loads([ln for ln in p.stdout.strip().splitlines() if ln.startswith("{")][-1])
    assert row["agree"] and not row["problems"] and row["refused_by_both"] > 0


def test_weight_manifest_matches_the_reference_tool():
    """``baseline/ref_manifest_check.py``: the reference's own manifest tool (compiled as it is) and this package's print
    the same JSON document for model directories written here - names in the same order, dtypes, shapes, packing."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    p = subprocess.run([sys.executable, str(root / "baseline" / "ref_manifest_check.py")], capture_output=True, text=True,
                       timeout=1200, cwd=root)
    if p.returncode == 3:
        import pytest
        pytest.skip(p.stdout.strip()[-300:])
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-1500:]
    rows = [json.loads(ln) for ln in p.stdout.strip().splitlines() if ln.startswith("{")]
    assert len(rows) == 4 and all(r["agree"] and r["names"] > 10 for r in rows)
