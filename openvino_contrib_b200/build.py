"""In-tree build of libb2a.so (sm_100a only) with nvcc — no JIT cache, no torch extension machinery.

    python -m openvino_contrib_b200.build [--force] [--verbose]

Objects go to ``openvino_contrib_b200/_build/``, the library to ``openvino_contrib_b200/libb2a.so``.
A source is recompiled when it, or any header of ``csrc/``, ``host/`` or ``include/``, is newer than its object.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
BUILD = os.path.join(PKG, "_build")
LIB = os.path.join(PKG, "libb2a.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-Xcompiler", "-Wno-unknown-pragmas",
    "--expt-relaxed-constexpr",
]

CU_SOURCES = ["csrc/api.cu", "csrc/attn_generic.cu", "csrc/paged_kv_store.cu", "csrc/paged_decode.cu",
              "csrc/sdpa_tcgen05.cu", "csrc/shard_group.cu", "csrc/paged_kv_state.cu", "csrc/paged_scores.cu"]
# host side in the library: the block manager, the operator classes (registered with the operation registry when the
# library is loaded) and the host-tensor pipeline built on them
CXX_SOURCES = ["host/kv_block_manager.cpp", "host/attention_ops.cpp", "host/host_pipeline.cpp",
               "host/kv_pool_state.cpp"]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libb2a.so cannot be built")
    return exe


def _headers_mtime() -> float:
    m = 0.0
    for d in (os.path.join(PKG, "csrc"), os.path.join(PKG, "host"), os.path.join(ROOT, "include")):
        for dirpath, _, files in os.walk(d):
            for f in files:
                if f.endswith((".h", ".hpp", ".cuh")):
                    m = max(m, os.path.getmtime(os.path.join(dirpath, f)))
    return m


def _compile(src: str, obj: str, verbose: bool, extra=()):
    cmd = [nvcc(), *NVCC_FLAGS, *extra, "-I", os.path.join(ROOT, "include"), "-I", os.path.join(PKG, "csrc"),
           "-I", os.path.join(PKG, "host"), "-c", os.path.join(PKG, src), "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    return src, r.stderr


def build_library(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(BUILD, exist_ok=True)
    hdr = _headers_mtime()
    jobs, objs = [], []
    for src in CU_SOURCES + CXX_SOURCES:
        obj = os.path.join(BUILD, os.path.basename(src) + ".o")
        objs.append(obj)
        s = os.path.getmtime(os.path.join(PKG, src))
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(s, hdr):
            jobs.append((src, obj))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for src, log in ex.map(lambda j: _compile(j[0], j[1], verbose), jobs):
                if verbose and log:
                    print(f"--- {src}\n{log}", file=sys.stderr)
    if jobs or not os.path.exists(LIB):
        cmd = [nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


HOST_TEST_SOURCES = ["host/host_tests.cpp"]
HOST_TESTS = os.path.join(BUILD, "host_tests")


def build_host_tests(force: bool = False) -> str:
    """The C++ operator classes and their test program, linked against libb2a.so (found through $ORIGIN/..)."""
    lib = build_library()
    srcs = [os.path.join(PKG, s) for s in HOST_TEST_SOURCES]
    newest = max([os.path.getmtime(s) for s in srcs] + [_headers_mtime(), os.path.getmtime(lib)])
    if force or not os.path.exists(HOST_TESTS) or os.path.getmtime(HOST_TESTS) < newest:
        cmd = [nvcc(), "-O2", "-std=c++17", "-Xcompiler", "-Wall", "-I", os.path.join(ROOT, "include"),
               "-I", os.path.join(PKG, "host"), *srcs, "-o", HOST_TESTS, "-L", PKG, "-lb2a",
               "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/.."]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"host tests failed to build:\n{r.stdout}\n{r.stderr}")
    return HOST_TESTS


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_host_tests(force="--force" in sys.argv))
