"""Builds the C-ABI shared library ``kvx_b200/lib/libkvx_b200.so`` in-tree with nvcc + gcc.

The library holds the CUDA-free validators (``csrc/kvx_abi.c``), the launch layer and
kernels (``csrc/kvx_paged_kv.cu``), the host-buffer pipeline (``csrc/kvx_host.cu``) and the decode
attention over the paged cache (``csrc/kvx_attention.cu``),
compiled for sm_100a only.  Run ``python -m kvx_b200.build`` or call :func:`build`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "kvx_b200", "csrc")
LIB_DIR = os.path.join(ROOT, "kvx_b200", "lib")
LIB_PATH = os.path.join(LIB_DIR, "libkvx_b200.so")
INCLUDE = os.path.join(ROOT, "include")
BUILD_DIR = os.path.join(ROOT, "build")

NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-I" + INCLUDE]
CU_SOURCES = ["kvx_paged_kv.cu", "kvx_host.cu", "kvx_attention.cu"]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if any source is newer than it; returns the library path."""
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(BUILD_DIR, exist_ok=True)
    cu = [os.path.join(CSRC, f) for f in CU_SOURCES if os.path.exists(os.path.join(CSRC, f))]
    c_src = os.path.join(CSRC, "kvx_abi.c")
    headers = [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    if not force and not _stale(LIB_PATH, cu + [c_src] + headers):
        return LIB_PATH
    c_obj = os.path.join(BUILD_DIR, "kvx_abi.o")
    run = lambda cmd: subprocess.run(cmd, check=True, stdout=None if verbose else subprocess.PIPE,
                                     stderr=subprocess.STDOUT)
    run(["gcc", "-std=c11", "-O2", "-fPIC", "-Wall", "-I" + INCLUDE, "-c", c_src, "-o", c_obj])
    # the translation units are independent: compile them side by side
    objs, jobs = [], []
    for src in cu:
        obj = os.path.join(BUILD_DIR, os.path.basename(src) + ".o")
        jobs.append((src, subprocess.Popen([_nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj],
                                           stdout=None if verbose else subprocess.PIPE, stderr=subprocess.STDOUT)))
        objs.append(obj)
    for src, job in jobs:
        out, _ = job.communicate()
        if job.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n" + (out.decode(errors="replace") if out else ""))
    run([_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", *objs, c_obj, "-o", LIB_PATH])
    return LIB_PATH


TORCH_OPS_SRC = os.path.join(CSRC, "kvx_torch_ops.cpp")
TORCH_OPS_PATH = os.path.join(LIB_DIR, "libkvx_b200_torch.so")


def build_torch_ops(force: bool = False, verbose: bool = False) -> str:
    """Compile the torch operator library (``torch.ops.kvx_b200.*``) against the installed
    torch and link it to ``libkvx_b200.so`` (found at load time next to it, via $ORIGIN)."""
    from torch.utils import cpp_extension as ext
    import torch

    build(force=False, verbose=verbose)
    headers = [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    if not force and not _stale(TORCH_OPS_PATH, [TORCH_OPS_SRC, LIB_PATH] + headers):
        return TORCH_OPS_PATH
    cuda_home = os.path.dirname(os.path.dirname(_nvcc()))
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-Wall",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-I" + INCLUDE, "-I" + os.path.join(cuda_home, "include")]
    cmd += ["-isystem" + p for p in ext.include_paths()]
    cmd += [TORCH_OPS_SRC, "-o", TORCH_OPS_PATH, "-L" + LIB_DIR, "-lkvx_b200", "-Wl,-rpath,$ORIGIN"]
    for d in ext.library_paths():
        cmd += ["-L" + d, "-Wl,-rpath," + d]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch"]
    subprocess.run(cmd, check=True, stdout=None if verbose else subprocess.PIPE, stderr=subprocess.STDOUT)
    return TORCH_OPS_PATH


PROGRAMS = {  # native programs over the C ABI: source -> binary under build/
    "kvx_bench": os.path.join(ROOT, "benchmarks", "kvx_bench.cu"),
    "kvx_kernel_test": os.path.join(ROOT, "tests", "kvx_kernel_test.cu"),
}


def build_programs(force: bool = False, verbose: bool = False) -> dict:
    """Compile the native benchmark and the native kernel test against ``libkvx_b200.so``
    (found at run time through an rpath relative to the binary).  Returns name -> path."""
    build(force=False, verbose=verbose)
    headers = [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    out = {}
    for name, src in PROGRAMS.items():
        exe = os.path.join(BUILD_DIR, name)
        out[name] = exe
        if not force and not _stale(exe, [src, LIB_PATH] + headers):
            continue
        cmd = [_nvcc(), "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-I" + INCLUDE, src, "-o", exe,
               "-L" + LIB_DIR, "-lkvx_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../kvx_b200/lib", "-lpthread"]
        subprocess.run(cmd, check=True, stdout=None if verbose else subprocess.PIPE, stderr=subprocess.STDOUT)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
    print(build_programs(force="--force" in sys.argv, verbose=True))
    print(build_torch_ops(force="--force" in sys.argv, verbose=True))
