"""A Hugging Face dataset split on disk as prompt / answer JSONL."""
import sys

import pytest



def test_hf_dataset_split_to_prompt_answer_jsonl(tmp_path, capsys):
    """A dataset snapshot on disk in the Hub's parquet layout (``<config>/<split>-0000i-of-0000n.parquet``) becomes
    a prompt / answer JSONL that the native reader loads; ``None`` fields become empty strings, ``max_examples``
    truncates, a missing field is an error that lists the keys."""
    import pyarrow as pa
    import pyarrow.parquet as pq
    from cverl_b200.cli import hf_dataset_download
    from cverl_b200.data import download_hf_dataset, load_prompt_answer_jsonl
    snap = tmp_path / "snap" / "main"
    snap.mkdir(parents=True)
    pq.write_table(pa.table({"question": ["What is 1+1?", "Ünïcode?"], "answer": ["#### 2", None]}),
                   snap / "train-00000-of-00002.parquet")
    pq.write_table(pa.table({"question": ["Third?"], "answer": ["#### 3"]}), snap / "train-00001-of-00002.parquet")
    pq.write_table(pa.table({"question": ["test q"], "answer": ["t"]}), snap / "test-00000-of-00001.parquet")
    out = tmp_path / "out" / "train.jsonl"
    res = download_hf_dataset(str(tmp_path / "snap"), out, name="main", split="train")
    assert res.rows == 3 and res.output_file == out
    rows = load_prompt_answer_jsonl(out)
    assert [r.prompt for r in rows] == ["What is 1+1?", "Ünïcode?", "Third?"] and rows[1].answer == ""
    assert hf_dataset_download.main(["--dataset", str(tmp_path / "snap"), "--name", "main", "--split", "test",
                                     "--output-file", str(tmp_path / "t.jsonl"), "--max-examples", "1"]) == 0
    printed = capsys.readouterr().out
    assert f"CVERL_HF_DATASET_FILE={tmp_path / 't.jsonl'}" in printed and "CVERL_HF_DATASET_ROWS=1" in printed
    with pytest.raises(KeyError, match="available keys"):
        download_hf_dataset(str(tmp_path / "snap"), tmp_path / "x.jsonl", name="main", prompt_field="prompt")
    with pytest.raises(FileNotFoundError):
        download_hf_dataset(str(tmp_path / "snap"), tmp_path / "x.jsonl", name="main", split="validation")


def test_hf_download_cli_options_and_offline_behaviour(tmp_path, capsys, monkeypatch):
    """The snapshot CLI: a directory that already holds a model is returned without touching the hub; the options
    of the reference's wrapper reach ``snapshot_download``; a dry run prints the repository's commit and file count."""
    import types
    from cverl_b200.cli import hf_download
    local = tmp_path / "m"
    local.mkdir()
    (local / "config.json").write_text("{}")
    (local / "model.safetensors").write_bytes(b"")
    assert hf_download.main(["model", "org/name", "--local-dir", str(local)]) == 0
    assert f"CVERL_HF_LOCAL_DIR={local}" in capsys.readouterr().out
    calls = {}
    fake = types.ModuleType("huggingface_hub")
    fake.snapshot_download = lambda **kw: calls.update(kw) or str(tmp_path / "snap")
    fake.model_info = lambda repo, revision=None, token=None: types.SimpleNamespace(sha="abc123", siblings=[1, 2, 3])
    monkeypatch.setitem(sys.modules, "huggingface_hub", fake)
    assert hf_download.main(["model", "org/name", "--local-dir", str(tmp_path / "new"), "--revision", "v1",
                             "--allow-pattern", "*.json", "--allow-pattern", "*.safetensors", "--ignore-pattern", "*.bin",
                             "--local-files-only", "--token", "t"]) == 0
    assert calls["revision"] == "v1" and calls["allow_patterns"] == ["*.json", "*.safetensors"]
    assert calls["ignore_patterns"] == ["*.bin"] and calls["local_files_only"] is True and calls["token"] == "t"
    capsys.readouterr()
    assert hf_download.main(["model", "org/name", "--dry-run"]) == 0
    out = capsys.readouterr().out
    assert "CVERL_HF_SHA=abc123" in out and "CVERL_HF_FILE_COUNT=3" in out
    # the reference's form: --repo-id instead of a sub-command
    calls.clear()
    assert hf_download.main(["--local-dir", str(tmp_path / "n2"), "--repo-id", "org/other", "--revision", "v2"]) == 0
    assert calls["repo_id"] == "org/other" and calls["revision"] == "v2"
