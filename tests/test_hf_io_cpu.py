"""The native safetensors reader / writer (csrc/safetensors.cc) behind ``models/hf_io.py``: every stored dtype,
several files in one directory, the header layout, threaded and ranged reads, and interchange with the
``safetensors`` package."""
import json
import struct

import pytest
import torch

from cverl_b200.models.hf_io import HfModelLoader, write_safetensors


def _tensors():
    g = torch.Generator().manual_seed(3)
    return {
        "a.f32": torch.randn(5, 7, generator=g), "b.f16": torch.randn(4, 3, generator=g).half(),
        "c.bf16": torch.randn(2, 3, 4, generator=g).bfloat16(), "d.i64": torch.arange(9).reshape(3, 3),
        "e.i32": torch.arange(6, dtype=torch.int32), "f.u8": torch.arange(11, dtype=torch.uint8),
        "g.scalar": torch.tensor(2.5), "h.empty": torch.zeros(0, 4),
    }


def test_round_trip_header_layout_and_package_interchange(tmp_path):
    tensors = _tensors()
    path = tmp_path / "model.safetensors"
    write_safetensors(path, tensors)
    raw = path.read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    assert (8 + hlen) % 8 == 0 and header["__metadata__"] == {"format": "pt"}
    assert header["c.bf16"] == {"dtype": "BF16", "shape": [2, 3, 4], "data_offsets": header["c.bf16"]["data_offsets"]}
    loader = HfModelLoader(path).load_metadata()
    assert sorted(loader.names()) == sorted(tensors)
    for name, t in tensors.items():
        got = loader.load_tensor(name)
        assert got.dtype == t.dtype and got.shape == t.shape and torch.equal(got, t), name
    with pytest.raises(KeyError):
        loader.load_tensor("missing")
    # files written by the safetensors package are read here, and the other way round
    st = pytest.importorskip("safetensors.torch")
    theirs = st.load_file(str(path))
    assert all(torch.equal(theirs[n], t) for n, t in tensors.items())
    other = tmp_path / "theirs.safetensors"
    st.save_file({k: v for k, v in tensors.items()}, str(other))
    back = HfModelLoader(other).load_metadata()
    assert all(torch.equal(back.load_tensor(n), t) for n, t in tensors.items())
    # a cast on write applies to floating tensors only
    write_safetensors(tmp_path / "cast.safetensors", tensors, dtype=torch.bfloat16)
    cast = HfModelLoader(tmp_path / "cast.safetensors").load_metadata()
    assert cast.info("a.f32").dtype == torch.bfloat16 and cast.info("d.i64").dtype == torch.int64


def test_directory_of_shards_and_bad_inputs(tmp_path):
    d = tmp_path / "dir"
    d.mkdir()
    write_safetensors(d / "model-00001-of-00002.safetensors", {"x": torch.ones(3)})
    write_safetensors(d / "model-00002-of-00002.safetensors", {"y": torch.zeros(2, 2)})
    (d / "model.safetensors.index.json").write_text("{}")          # ignored, as by the reference's loader
    loader = HfModelLoader(d).load_metadata()
    assert loader.names() == ["x", "y"] and loader.has("y") and not loader.has("z")
    with pytest.raises(RuntimeError):
        HfModelLoader(tmp_path / "nowhere").load_metadata()
    (tmp_path / "bad.safetensors").write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00{ not a header")
    with pytest.raises(RuntimeError):
        HfModelLoader(tmp_path / "bad.safetensors").load_metadata()
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(RuntimeError):
        HfModelLoader(empty).load_metadata()


def test_threaded_and_ranged_reads_of_a_large_tensor(tmp_path):
    big = torch.arange(10 * 1024 * 1024, dtype=torch.int32).reshape(1024, -1)      # 40 MiB: several pread pieces
    write_safetensors(tmp_path / "big.safetensors", {"pad": torch.zeros(3, dtype=torch.uint8), "big": big})
    loader = HfModelLoader(tmp_path / "big.safetensors").load_metadata()
    assert torch.equal(loader.load_tensor("big"), big)
    for threads in (1, 4, 7):
        assert torch.equal(loader.load_rows("big", 100, 901, threads=threads), big[100:901])
    assert loader.bytes_read == big.numel() * 4 + 3 * 801 * big.shape[1] * 4
    assert loader.load_rows("big", 1024, 1024).numel() == 0
    with pytest.raises(ValueError):
        loader.load_rows("big", 5, 4)


def test_tensor_names_with_escapes_and_unicode(tmp_path):
    """Names travel through the JSON header: quotes, backslashes, control characters and non-ASCII text written
    here are read back by the safetensors package, and a header that spells non-ASCII names as \\uXXXX escapes
    (surrogate pairs included) is decoded to the same UTF-8 names."""
    st = pytest.importorskip("safetensors.torch")
    names = ['plain', 'q"uote', 'back\\slash', 'tab\there', 'line\nbreak', 'ü.weight', '数学', 'emoji🙂']
    tensors = {n: torch.full((2,), float(i)) for i, n in enumerate(names)}
    path = tmp_path / "names.safetensors"
    write_safetensors(path, tensors)
    theirs = st.load_file(str(path))
    assert sorted(theirs) == sorted(names) and all(float(theirs[n][0]) == float(tensors[n][0]) for n in names)
    # the same content with an ASCII-only header
    raw = path.read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.dumps(json.loads(raw[8:8 + hlen]), ensure_ascii=True).encode()
    assert b"\\ud83d\\ude42" in header and b"\\u6570" in header
    header += b" " * ((8 - (8 + len(header)) % 8) % 8)
    ascii_path = tmp_path / "ascii.safetensors"
    ascii_path.write_bytes(struct.pack("<Q", len(header)) + header + raw[8 + hlen:])
    loader = HfModelLoader(ascii_path).load_metadata()
    assert sorted(loader.names()) == sorted(names)
    assert all(torch.equal(loader.load_tensor(n), tensors[n]) for n in names)


def test_reference_loader_reads_directories_written_here():
    """``baseline/ref_loader_check.py``: the reference's own ``HfModelLoader`` (its compiled object, linked into a small
    driver) reads a dense and a mixture-of-experts model directory written by this package and finds the same
    tensors, element counts and values.  Skipped where the reference objects have not been built."""
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    p = subprocess.run([sys.executable, str(root / "baseline" / "ref_loader_check.py")], capture_output=True, text=True,
                       timeout=900, cwd=root)
    if p.returncode == 3:
        pytest.skip(p.stdout.strip()[-300:])
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-1500:]
    rows = [json.loads(ln) for ln in p.stdout.strip().splitlines() if ln.startswith("{")]
    assert [r["model"] for r in rows] == ["qwen3_5", "qwen3_moe"] and all(r["agree"] for r in rows)
