"""The host runtime under AddressSanitizer + UBSan and under ThreadSanitizer: the C ABI self-test driver
(``csrc/host_selftest_main.cc``: RL math from four threads, argument validation, planner, safetensors round trip,
byte tokenizer, reward extraction, JSONL reader, the BPE tokenizer from two threads on one handle, shared-memory
transport with a server and a client thread) must exit 0 without a sanitizer report."""
import subprocess
from pathlib import Path

import pytest

from cverl_b200 import _build


@pytest.mark.parametrize("kind", ["address", "thread"])
def test_host_runtime_under_sanitizer(kind):
    try:
        exe = _build.build_sanitized(kind)
    except RuntimeError as exc:
        if "no C++ compiler with the runtime" in str(exc):
            pytest.skip(str(exc))
        raise
    tokenizer = Path(__file__).resolve().parent / "fixtures" / "synthetic_tokenizer.json"
    p = subprocess.run([str(exe), str(tokenizer)], capture_output=True, text=True, timeout=300)   # BPE from two threads
    assert p.returncode == 0, p.stdout + p.stderr
    assert "host self-test passed" in p.stdout
    for word in ("AddressSanitizer", "ThreadSanitizer", "runtime error:", "LeakSanitizer"):
        assert word not in p.stderr, p.stderr[-3000:]


def test_plain_selftest_executable_is_built_with_the_host_library():
    _build.build_host()
    exe = _build.LIB_DIR / "host_selftest"
    assert exe.exists()
    p = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0 and "host self-test passed" in p.stdout, p.stdout + p.stderr
