"""Builds the checker libraries -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

``libkvx_oracle.so``      the C restatement in this folder (gcc).
``_ref/libkvx_ref.so``    the reference project's own sources (its validators and its CUDA
                          launch layer), compiled unmodified from where they lie for
                          sm_100a.  Only built where the reference checkout is present;
                          the product is git-ignored and contains no copied source.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
ORACLE_LIB = os.path.join(HERE, "libkvx_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_LIB = os.path.join(REF_DIR, "libkvx_ref.so")
REFERENCE_ROOT = os.environ.get("KVX_REFERENCE_ROOT", "/root/reference")


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_oracle(force: bool = False) -> str:
    srcs = [os.path.join(HERE, f) for f in ("kvx_oracle.c", "kvx_cpu_baseline.c", "kvx_oracle.h")]
    srcs.append(os.path.join(ROOT, "include", "kvx_abi.h"))
    srcs.append(os.path.join(ROOT, "include", "kvx_attention.h"))
    if force or _stale(ORACLE_LIB, srcs):
        subprocess.run(["gcc", "-std=c11", "-O2", "-Wall", "-Wextra", "-fPIC", "-shared",
                        "-I" + os.path.join(ROOT, "include"), srcs[0], srcs[1], "-o", ORACLE_LIB,
                        "-lm", "-lpthread"], check=True)
    return ORACLE_LIB


def build_reference(force: bool = False) -> str | None:
    """Compile the reference's kvx_abi.c + kernels/kvx_paged_kv.cu into _ref/libkvx_ref.so."""
    abi_c = os.path.join(REFERENCE_ROOT, "kvx_abi.c")
    kern = os.path.join(REFERENCE_ROOT, "kernels", "kvx_paged_kv.cu")
    if not (os.path.exists(abi_c) and os.path.exists(kern)):
        return REF_LIB if os.path.exists(REF_LIB) else None
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        return REF_LIB if os.path.exists(REF_LIB) else None
    os.makedirs(REF_DIR, exist_ok=True)
    if force or _stale(REF_LIB, [abi_c, kern]):
        obj = os.path.join(REF_DIR, "kvx_abi_ref.o")
        subprocess.run(["gcc", "-std=c11", "-O2", "-fPIC", "-I" + REFERENCE_ROOT, "-c", abi_c, "-o", obj],
                       check=True)
        subprocess.run([nvcc, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a",
                        "-Xcompiler", "-fPIC", "-shared", "-I" + REFERENCE_ROOT,
                        "-I" + os.path.join(REFERENCE_ROOT, "kernels"), kern, obj, "-o", REF_LIB],
                       check=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return REF_LIB


def build_reference_programs(force: bool = False) -> dict:
    """Compile the reference's own GPU test and micro-benchmark, unmodified, twice: linked
    against the reference's kernels (``*_ref``) and against this repository's library
    (``*_ours``).  Outputs go to _ref/ only.  Returns {name: path} of what exists."""
    out = {}
    tests_cu = os.path.join(REFERENCE_ROOT, "tests", "kvx_kernel_test.cu")
    bench_cu = os.path.join(REFERENCE_ROOT, "benchmarks", "kvx_bench.cu")
    ours = os.path.join(ROOT, "kvx_b200", "lib", "libkvx_b200.so")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    have_src = os.path.exists(tests_cu) and os.path.exists(bench_cu) and os.path.exists(nvcc)
    os.makedirs(REF_DIR, exist_ok=True)
    for name, src, lib in (("kvx_kernel_test_ref", tests_cu, REF_LIB), ("kvx_kernel_test_ours", tests_cu, ours),
                           ("kvx_bench_ref", bench_cu, REF_LIB), ("kvx_bench_ours", bench_cu, ours)):
        exe = os.path.join(REF_DIR, name)
        if have_src and os.path.exists(lib) and (force or _stale(exe, [src, lib])):
            libdir, libname = os.path.dirname(lib), os.path.basename(lib)[3:-3]
            inc = REFERENCE_ROOT if lib == REF_LIB else os.path.join(ROOT, "include")
            subprocess.run([nvcc, "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-I" + inc, src, "-o", exe,
                            "-L" + libdir, "-l" + libname, "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/" +
                            os.path.relpath(libdir, REF_DIR)], check=True, stdout=subprocess.PIPE,
                           stderr=subprocess.STDOUT)
        if os.path.exists(exe):
            out[name] = exe
    return out


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_reference(force="--force" in sys.argv))
    print(build_reference_programs(force="--force" in sys.argv))
