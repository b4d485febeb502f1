#!/usr/bin/env python
"""Out-of-tree build of the UNMODIFIED reference (HaitaoWuTJU/cverl) for the benchmark's reference arm.

The reference is a CMake + LibTorch C++ project.  Its CMake configure step stops on a missing
``pcre2.h`` (CMakeLists.txt:91-105), which one translation unit needs
(src/text/hf_bpe_tokenizer.cc:3-7); the image has the PCRE2 runtime library but no header.  This
script therefore compiles the reference's own source files, untouched and read in place, with a
plain command list:

* every file of the ``cverl`` library target (CMakeLists.txt:139-174) plus the CUDA and NCCL
  sources that ``CVERL_ENABLE_CUDA`` / ``CVERL_ENABLE_NCCL`` add (CMakeLists.txt:206-230), with
  the same two compile definitions;
* the trainer executable ``tools/model/qwen3_5_pp_tp_ppo_trainer.cc`` (CMakeLists.txt:444-446);
* include paths: the reference's ``include/``, LibTorch's headers from the installed ``torch``
  wheel, ``nccl.h`` from the ``nvidia-nccl`` wheel, a ``nlohmann/json.hpp`` that another wheel
  vendors, and ``baseline/shim`` whose ``pcre2.h`` only declares the seven documented PCRE2
  functions the tokenizer calls;
* the two ``.cu`` files are compiled for sm_100a (the reference names no architecture).

Outputs (git-ignored): ``baseline/_ref/bin/qwen3_5_pp_tp_ppo_trainer`` and
``baseline/_ref/lib/libcverl_ref.so`` (the whole library, for timing the reference's CPU C ABI).

    python baseline/build_ref.py [--src DIR] [--jobs N] [--force]
"""
from __future__ import annotations

import argparse
import glob
import os
import shutil
import site
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"

LIB_SOURCES = """
src/status.cc src/hf_downloader.cc src/data/hf_dataset.cc src/distributed/collectives.cc
src/distributed/cp_attention_cuda_stub.cc src/distributed/context_parallel.cc
src/distributed/optimizer_sharding.cc src/distributed/expert_parallel.cc src/distributed/parallel_ops.cc
src/distributed/pipeline.cc src/distributed/topology.cc src/distributed/weight_sync.cc
src/model/hf_model_loader.cc src/model/qwen_linear_attention_cuda_stub.cc src/model/qwen3_5_text.cc
src/model/safetensors_writer.cc src/reward/gsm8k.cc src/rollout/rollout_batch.cc src/rollout/policy_worker.cc
src/rollout/plugin_worker.cc src/rollout/shared_memory.cc src/rollout/shared_memory_transport.cc
src/rollout/transport.cc src/rollout/worker.cc src/text/byte_tokenizer.cc src/text/hf_bpe_tokenizer.cc
src/core_algos_c_api.cc src/torch/causal_lm_policy.cc src/torch/core_algos_torch.cc
src/torch/fp32_master_adamw.cc src/torch/qwen3_5_causal_lm_policy.cc src/torch/simple_grpo_trainer.cc
src/torch/tiny_causal_lm_policy.cc src/torch/tiny_causal_policy.cc
src/rollout/gpu_ipc_rollout_batch.cc src/distributed/nccl_collectives.cc src/rollout/nccl_gpu_batch_transport.cc
""".split()
CUDA_SOURCES = ["cuda/core_algos_cuda.cu", "cuda/cp_attention_cuda.cu", "cuda/qwen_linear_attention_cuda.cu"]
TRAINER_MAIN = "tools/model/qwen3_5_pp_tp_ppo_trainer.cc"


def default_source_dir() -> Path:
    env = os.environ.get("CVERL_REFERENCE_SRC")
    if env:
        return Path(env)
    return HERE.parent.parent / "reference"


def find_paths():
    import torch
    from torch.utils import cpp_extension
    torch_lib = Path(torch.__file__).parent / "lib"
    incs = list(cpp_extension.include_paths())
    nccl_inc = nccl_lib = json_inc = None
    for sp in site.getsitepackages():
        if nccl_inc is None and (Path(sp) / "nvidia/nccl/include/nccl.h").exists():
            nccl_inc = Path(sp) / "nvidia/nccl/include"
            nccl_lib = Path(sp) / "nvidia/nccl/lib"
        if json_inc is None:
            hits = glob.glob(str(Path(sp) / "**/nlohmann/json.hpp"), recursive=True)
            if hits:
                json_inc = Path(hits[0]).parent.parent
    pcre = None
    for cand in ("/usr/lib/x86_64-linux-gnu/libpcre2-8.so.0", "/usr/lib64/libpcre2-8.so.0", "/usr/lib/libpcre2-8.so.0"):
        if Path(cand).exists():
            pcre = Path(cand)
            break
    missing = [n for n, v in (("nccl.h", nccl_inc), ("nlohmann/json.hpp", json_inc), ("libpcre2-8.so.0", pcre)) if v is None]
    if missing:
        raise RuntimeError("reference build: not found on this image: " + ", ".join(missing))
    cuda_home = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    return dict(torch_lib=torch_lib, torch_inc=incs, nccl_inc=nccl_inc, nccl_lib=nccl_lib, json_inc=json_inc,
                pcre=pcre, cuda_home=cuda_home, cxx11_abi=int(torch._C._GLIBCXX_USE_CXX11_ABI))


def run(cmd, log: Path):
    proc = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    log.write_text(" ".join(str(c) for c in cmd) + "\n" + proc.stdout + proc.stderr)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout[-4000:] + proc.stderr[-8000:])
        raise RuntimeError(f"reference build failed: see {log}")


def build(src: Path, jobs: int, force: bool) -> Path:
    if not (src / TRAINER_MAIN).exists():
        raise RuntimeError(f"reference sources not found under {src}")
    p = find_paths()
    obj_dir, bin_dir, lib_dir = OUT / "obj", OUT / "bin", OUT / "lib"
    for d in (obj_dir, bin_dir, lib_dir):
        d.mkdir(parents=True, exist_ok=True)
    includes = [src / "include", HERE / "shim", p["json_inc"], p["nccl_inc"], p["cuda_home"] / "include", *p["torch_inc"]]
    inc_flags = [f for i in includes for f in ("-I", str(i))]
    defs = [f"-D_GLIBCXX_USE_CXX11_ABI={p['cxx11_abi']}", "-DCVERL_ENABLE_CUDA=1", "-DCVERL_ENABLE_NCCL=1",
            f'-DCVERL_HF_DOWNLOAD_SCRIPT="{src}/tools/hf_snapshot_download.py"',
            f'-DCVERL_HF_DATASET_SCRIPT="{src}/tools/hf_dataset_download.py"']
    cxx = [os.environ.get("CXX", "g++"), "-std=c++17", "-O2", "-fPIC", "-pthread", *defs, *inc_flags]
    nvcc = [p["cuda_home"] / "bin/nvcc", "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a",
            "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", *defs, *inc_flags]

    work = []
    for rel in LIB_SOURCES + [TRAINER_MAIN]:
        obj = obj_dir / (rel.replace("/", "__") + ".o")
        work.append((cxx + ["-c", src / rel, "-o", obj], obj, src / rel))
    for rel in CUDA_SOURCES:
        obj = obj_dir / (rel.replace("/", "__") + ".o")
        work.append((nvcc + ["-c", src / rel, "-o", obj], obj, src / rel))

    def one(item):
        cmd, obj, s = item
        if not force and obj.exists() and obj.stat().st_mtime >= s.stat().st_mtime:
            return
        print(f"[ref] {s.relative_to(src)}", flush=True)
        run(cmd, obj.with_suffix(".log"))

    with ThreadPoolExecutor(max_workers=jobs) as ex:
        list(ex.map(one, work))

    lib_objs = [o for _, o, s in work if s != src / TRAINER_MAIN]
    main_obj = [o for _, o, s in work if s == src / TRAINER_MAIN]
    rpaths = [p["torch_lib"], p["nccl_lib"], p["cuda_home"] / "lib64", p["pcre"].parent]
    link = ["-L", p["torch_lib"], "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
            "-L", p["cuda_home"] / "lib64", "-lcudart", p["nccl_lib"] / "libnccl.so.2", p["pcre"],
            "-lrt", "-ldl", "-pthread", *[f"-Wl,-rpath,{r}" for r in rpaths]]
    lib = lib_dir / "libcverl_ref.so"
    exe = bin_dir / "qwen3_5_pp_tp_ppo_trainer"
    print("[ref] link", flush=True)
    run([cxx[0], "-shared", "-o", lib, *lib_objs, "-Wl,--no-as-needed", *link], lib_dir / "link_lib.log")
    run([cxx[0], "-o", exe, *main_obj, *lib_objs, "-Wl,--no-as-needed", *link], bin_dir / "link_exe.log")
    (OUT / "BUILD_INFO.txt").write_text(
        f"source: {src}\ncompiler: {shutil.which(cxx[0])}\nnvcc arch: sm_100a\n"
        f"torch: {p['torch_lib'].parent}\nnccl: {p['nccl_lib']}\n")
    return exe


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", type=Path, default=default_source_dir())
    ap.add_argument("--jobs", type=int, default=min(8, os.cpu_count() or 1))
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    exe = build(args.src.resolve(), args.jobs, args.force)
    print("built", exe)


if __name__ == "__main__":
    main()
