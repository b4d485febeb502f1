"""Shared by the ``baseline/ref_*_check.py`` scripts: link a small driver against the built reference.

``link_driver(source, name)`` compiles ``source`` (a driver of this directory, or one of the reference's own tools,
unmodified) against the reference's headers and ``baseline/_ref/lib/libcverl_ref.so`` plus LibTorch, and caches the
executable under ``baseline/_ref/bin/`` (rebuilt when the source or the library is newer).  Returns the path, or
raises ``Unavailable`` with the reason (reference not built, compile error).
"""
from __future__ import annotations

import subprocess
import sys
from pathlib import Path
from typing import Sequence

HERE = Path(__file__).resolve().parent
REF_LIB_DIR = HERE / "_ref" / "lib"
REF_BIN_DIR = HERE / "_ref" / "bin"


class Unavailable(RuntimeError):
    pass


def reference_source_dir() -> Path:
    sys.path.insert(0, str(HERE))
    try:
        import build_ref
        return build_ref.default_source_dir()
    finally:
        sys.path.pop(0)


def link_driver(source: Path, name: str, *, link_library: bool = True, extra_objects: Sequence[Path] = ()) -> Path:
    import torch
    sys.path.insert(0, str(HERE))
    try:
        import build_ref
        paths, src = build_ref.find_paths(), build_ref.default_source_dir()
    except Exception as exc:  # noqa: BLE001 - every failure here means "no reference on this machine"
        raise Unavailable(f"{type(exc).__name__}: {exc}") from exc
    finally:
        sys.path.pop(0)
    library = REF_LIB_DIR / "libcverl_ref.so"
    needed = [library] if link_library else list(extra_objects)
    if not all(Path(n).exists() for n in needed):
        raise Unavailable("reference not built (python baseline/build_ref.py)")
    source = Path(source)
    if not source.exists():
        raise Unavailable(f"{source} not found")
    REF_BIN_DIR.mkdir(parents=True, exist_ok=True)
    exe = REF_BIN_DIR / name
    newest = max([source.stat().st_mtime, Path(__file__).stat().st_mtime] + [Path(n).stat().st_mtime for n in needed])
    if exe.exists() and exe.stat().st_mtime >= newest:
        return exe
    lib = Path(torch.__file__).parent / "lib"
    incs = [src / "include", HERE / "shim", paths["json_inc"], *paths["torch_inc"]]
    cmd = ["g++", "-std=c++17", "-O1", f"-D_GLIBCXX_USE_CXX11_ABI={paths['cxx11_abi']}", str(source),
           *map(str, extra_objects), *[f for i in incs for f in ("-I", str(i))]]
    if link_library:
        cmd += ["-L", str(REF_LIB_DIR), "-lcverl_ref", f"-Wl,-rpath,{REF_LIB_DIR}"]
    cmd += ["-L", str(lib), "-ltorch", "-ltorch_cpu", "-lc10", f"-Wl,-rpath,{lib}", "-o", str(exe)]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise Unavailable("compiling the driver failed: " + p.stderr[-300:])
    return exe
