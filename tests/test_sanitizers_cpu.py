"""The host runtime under AddressSanitizer + UBSan and under ThreadSanitizer: the C ABI self-test driver
(``csrc/host_selftest_main.cc``: RL math from four threads, argument validation, planner, safetensors round trip,
byte tokenizer, reward extraction, JSONL reader, the BPE tokenizer from two threads on one handle, the rollout plugin loader, shared-memory
transport with a server and a client thread) must exit 0 without a sanitizer report."""
import os
import subprocess
from pathlib import Path

import pytest

from cverl_b200 import _build


@pytest.mark.parametrize("kind", ["address", "thread"])
def test_host_runtime_under_sanitizer(kind, tmp_path):
    try:
        exe = _build.build_sanitized(kind)
    except RuntimeError as exc:
        if "no C++ compiler with the runtime" in str(exc):
            pytest.skip(str(exc))
        raise
    tokenizer = Path(__file__).resolve().parent / "fixtures" / "synthetic_tokenizer.json"
    _build.build_host()                                           # the plugin fixture the loader opens
    plugin = _build.LIB_DIR / "libplugin_worker_fixture.so"
    # the dynamic loader keeps what a dlopen'ed library's C++ runtime allocates at load time: not this code's leak
    supp = tmp_path / "lsan.supp"
    supp.write_text("leak:_dl_catch_exception\nleak:dlopen\n")
    env = dict(os.environ, LSAN_OPTIONS=f"suppressions={supp}:print_suppressions=0")
    p = subprocess.run([str(exe), str(tokenizer), str(plugin)], capture_output=True, text=True, timeout=300, env=env)
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
