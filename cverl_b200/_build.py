"""In-tree native build: nvcc for the sm_100a kernels, g++ for the host runtime.

Two shared libraries are produced under ``cverl_b200/lib``:

* ``libcverl_b200_cuda.so`` - every ``cuda/*.cu`` kernel file, compiled with
  ``-gencode arch=compute_100a,code=sm_100a`` (cross-compiles without a GPU);
* ``libcverl.so`` - the host-side C/C++ runtime (public C ABI of the RL math,
  topology, pipeline schedule, safetensors, tokenizers, reward, transports,
  plugin loader);
* ``libcverl_nccl.so`` - the native NCCL communicator (``nccl/nccl_backend.cc``),
  built against the ``nccl.h`` / ``libnccl.so.2`` of the installed ``nvidia-nccl``
  wheel (the library ``torch`` itself loads), skipped when that wheel is absent.

Objects are cached under ``build/`` and rebuilt when a source or header is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
LIB_DIR = PKG / "lib"
OBJ_DIR = ROOT / "build" / "obj"
CUDA_LIB = LIB_DIR / "libcverl_b200_cuda.so"
HOST_LIB = LIB_DIR / "libcverl.so"
NCCL_LIB = LIB_DIR / "libcverl_nccl.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _newest(paths) -> float:
    return max((p.stat().st_mtime for p in paths), default=0.0)


def _run(cmd, log_path: Path | None = None) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if log_path is not None:
        log_path.write_text(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("command failed: " + " ".join(map(str, cmd)))


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    srcs = sorted((PKG / "cuda").glob("*.cu"))
    hdrs = list((PKG / "cuda").glob("*.cuh")) + list((PKG / "cuda").glob("*.h"))
    hdr_time = _newest(hdrs)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in srcs:
        obj = OBJ_DIR / (src.stem + ".cu.o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        if verbose:
            print(f"[nvcc] {src.name}", flush=True)
        _run([nvcc, *NVCC_FLAGS, "-I", str(PKG / "cuda"), "-c", str(src), "-o", str(obj)],
             OBJ_DIR / (src.stem + ".ptxas.log"))

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        list(ex.map(compile_one, jobs))
    if jobs or not CUDA_LIB.exists():
        _run([nvcc, "-shared", "-o", str(CUDA_LIB), *map(str, objs), "-lcudart", "-Xlinker", "-z,noexecstack"])
    return CUDA_LIB


def build_host(force: bool = False, verbose: bool = False) -> Path:
    srcs = sorted(p for p in (PKG / "csrc").glob("*.cc") if not p.name.endswith("_main.cc")
                  and not p.name.endswith("_fixture.cc"))
    hdrs = list((PKG / "csrc" / "include").rglob("*.h"))
    hdr_time = _newest(hdrs)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    cxx = os.environ.get("CXX", "g++")
    jobs, objs = [], []
    for src in srcs:
        obj = OBJ_DIR / (src.stem + ".cc.o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        if verbose:
            print(f"[g++] {src.name}", flush=True)
        _run([cxx, *CXX_FLAGS, "-I", str(PKG / "csrc" / "include"), "-c", str(src), "-o", str(obj)])

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        list(ex.map(compile_one, jobs))
    if jobs or not HOST_LIB.exists():
        _run([cxx, "-shared", "-o", str(HOST_LIB), *map(str, objs), "-ldl", "-lrt", "-pthread"])
    # stand-alone executables and the plugin fixture
    inc = ["-I", str(PKG / "csrc" / "include")]
    for src in sorted((PKG / "csrc").glob("*_main.cc")):
        exe = LIB_DIR / src.stem.replace("_main", "")
        if force or not exe.exists() or exe.stat().st_mtime < max(src.stat().st_mtime, hdr_time, HOST_LIB.stat().st_mtime):
            _run([cxx, *CXX_FLAGS, *inc, str(src), "-o", str(exe), f"-L{LIB_DIR}", "-lcverl",
                  f"-Wl,-rpath,{LIB_DIR}", "-ldl", "-lrt", "-pthread"])
    for src in sorted((PKG / "csrc").glob("*_fixture.cc")):
        so = LIB_DIR / ("lib" + src.stem + ".so")
        if force or not so.exists() or so.stat().st_mtime < max(src.stat().st_mtime, hdr_time):
            _run([cxx, *CXX_FLAGS, *inc, "-shared", str(src), "-o", str(so)])
    return HOST_LIB


def _sanitizer_cxx(flags) -> str:
    """The first C++ compiler whose installation has the sanitizer runtime (a toolchain may ship without it)."""
    import shutil
    import tempfile
    seen = []
    for cand in (os.environ.get("CXX"), shutil.which("g++"), "/usr/bin/g++", shutil.which("clang++")):
        if not cand or cand in seen or not Path(cand).exists():
            continue
        seen.append(cand)
        with tempfile.TemporaryDirectory() as d:
            src = Path(d) / "probe.cc"
            src.write_text("int main() { return 0; }\n")
            r = subprocess.run([cand, *flags, str(src), "-o", str(Path(d) / "probe")], capture_output=True)
            if r.returncode == 0:
                return cand
    raise RuntimeError("no C++ compiler with the runtime for " + " ".join(flags) + " (tried " + ", ".join(seen) + ")")


def build_sanitized(kind: str, verbose: bool = False) -> Path:
    """The host runtime and its self-test driver (``csrc/host_selftest_main.cc``) as ONE executable built with a
    sanitizer: ``kind`` = "address" (AddressSanitizer + UBSan) or "thread" (ThreadSanitizer).  Returns the path;
    run it on a CPU box - exit code 0 and no sanitizer report is the pass criterion.  The executable links the
    sources directly (a sanitized shared library cannot be loaded into an unsanitized Python)."""
    flags = {"address": ["-fsanitize=address,undefined", "-fno-omit-frame-pointer"],
             "thread": ["-fsanitize=thread"]}[kind]
    srcs = sorted(p for p in (PKG / "csrc").glob("*.cc") if not p.name.endswith("_main.cc")
                  and not p.name.endswith("_fixture.cc"))
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    exe = LIB_DIR / f"host_selftest_{kind}"
    newest = max(_newest(srcs), _newest(list((PKG / "csrc" / "include").rglob("*.h"))),
                 (PKG / "csrc" / "host_selftest_main.cc").stat().st_mtime)
    if exe.exists() and exe.stat().st_mtime >= newest:
        return exe
    if verbose:
        print(f"[g++ -fsanitize={kind}] host runtime + self-test", flush=True)
    cxx = _sanitizer_cxx(flags)
    base = [f for f in CXX_FLAGS if f not in ("-O2", "-O3", "-fPIC")]
    _run([cxx, *base, "-O1", "-g", *flags, "-I", str(PKG / "csrc" / "include"), *map(str, srcs),
          str(PKG / "csrc" / "host_selftest_main.cc"), "-o", str(exe), "-ldl", "-lrt", "-pthread"])
    return exe


def _nccl_paths():
    """(include dir, library file) of the NCCL that ``torch`` uses, or (None, None)."""
    import site
    for sp in site.getsitepackages():
        inc, lib = Path(sp) / "nvidia/nccl/include", Path(sp) / "nvidia/nccl/lib/libnccl.so.2"
        if (inc / "nccl.h").exists() and lib.exists():
            return inc, lib
    for inc, lib in ((Path("/usr/include"), Path("/usr/lib/x86_64-linux-gnu/libnccl.so.2")),):
        if (inc / "nccl.h").exists() and lib.exists():
            return inc, lib
    return None, None


def build_nccl(force: bool = False, verbose: bool = False) -> Path | None:
    src = PKG / "nccl" / "nccl_backend.cc"
    inc, lib = _nccl_paths()
    if inc is None:
        if verbose:
            print("[g++] nccl_backend.cc skipped: no nccl.h / libnccl.so.2 on this machine", flush=True)
        return None
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    if not force and NCCL_LIB.exists() and NCCL_LIB.stat().st_mtime >= src.stat().st_mtime:
        return NCCL_LIB
    if verbose:
        print("[g++] nccl_backend.cc", flush=True)
    cuda_home = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    _run([os.environ.get("CXX", "g++"), *CXX_FLAGS, "-shared", "-I", str(inc), "-I", str(cuda_home / "include"),
          str(src), "-o", str(NCCL_LIB), str(lib), f"-L{cuda_home / 'lib64'}", "-lcudart",
          f"-Wl,-rpath,{lib.parent}", f"-Wl,-rpath,{cuda_home / 'lib64'}"])
    return NCCL_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_host(force, verbose)
    build_cuda(force, verbose)
    build_nccl(force, verbose)


if __name__ == "__main__":
    if "--sanitize" in sys.argv:
        print("built:", build_sanitized(sys.argv[sys.argv.index("--sanitize") + 1], verbose=True))
        sys.exit(0)
    build_all(force="--force" in sys.argv, verbose=True)
    print("built:", CUDA_LIB, HOST_LIB)
