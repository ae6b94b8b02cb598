"""Builds the native pieces in-tree.

  libhkv.so          the product: CUDA kernels + C ABI (nvcc, sm_100a only)
  libhkv_dist.so     the multi-GPU host (C++ over libhkv + NCCL) behind include/hkv_dist.h
  hkv_host_tests     C++ host adapter tests (registry shim + KV cache objects)
  hkv_watch_tests    CPU-only C++ tests of the host-side failure detection (no CUDA)
  hkv_seqsplit_tests C++ test of the sequence-split decoder (one process per GPU)
  hkv_gemma4_tests   C++ tests of the heterogeneous/shared cache owner and the per-layer decode loop
  oracle/_build, oracle/_ref   the test-only checkers (see oracle/Makefile)

Run as a script (`python hector-engine_b200/build.py`) or through __graft_entry__.build().
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
HOST = os.path.join(PKG_DIR, "host")
LIB = os.path.join(PKG_DIR, "libhkv.so")
DIST_LIB = os.path.join(PKG_DIR, "libhkv_dist.so")
HOST_TESTS = os.path.join(REPO, "tests", "cpp", "hkv_host_tests")
WATCH_TESTS = os.path.join(REPO, "tests", "cpp", "hkv_watch_tests")
SEQSPLIT_TESTS = os.path.join(REPO, "tests", "cpp", "hkv_seqsplit_tests")
GEMMA4_TESTS = os.path.join(REPO, "tests", "cpp", "hkv_gemma4_tests")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libhkv can only be built with the CUDA toolkit")
    return nvcc


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _sources(*dirs: str) -> list[str]:
    out = [os.path.join(REPO, "include", "hkv.h")]
    for d in dirs:
        for name in sorted(os.listdir(d)):
            if name.endswith((".cu", ".cuh", ".cpp", ".hpp", ".h")):
                out.append(os.path.join(d, name))
    return out


def build_lib(force: bool = False, verbose: bool = False) -> str:
    srcs = _sources(CSRC)
    if not force and _newer(LIB, srcs):
        return LIB
    cmd = [_nvcc(), *ARCH, *NVCC_FLAGS, "-shared", "-o", LIB, os.path.join(CSRC, "hkv_api.cu")]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    subprocess.run(cmd, check=True)
    return LIB


def build_host_tests(force: bool = False) -> str | None:
    """C++ tests of the registry adapter (tests/cpp): link libhkv and, as the checker only,
    the CPU oracle. Call after build_oracle()."""
    main = os.path.join(REPO, "tests", "cpp", "hkv_host_tests.cpp")
    oracle_dir = os.path.join(REPO, "oracle", "_build")
    if not os.path.exists(main):
        return None
    srcs = _sources(HOST) + [main, os.path.join(REPO, "tests", "cpp", "hkv_engine_shim.hpp")]
    if not force and _newer(HOST_TESTS, srcs + [LIB]):
        return HOST_TESTS
    cmd = [_nvcc(), *ARCH, "-O2", "-std=c++17", "-o", HOST_TESTS, main,
           os.path.join(HOST, "hkv_register.cpp"), "-I", os.path.join(REPO, "include"), "-I", HOST,
           "-L", PKG_DIR, "-lhkv", "-L", oracle_dir, "-lhkv_oracle",
           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../hector-engine_b200",
           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../oracle/_build"]
    subprocess.run(cmd, check=True)
    return HOST_TESTS


def reference_dir() -> str:
    """The reference engine's checkout, for the test-only checkers built from its sources:
    $HKV_REFERENCE_DIR, else a `reference` directory beside this repository; '' when absent."""
    cand = os.environ.get("HKV_REFERENCE_DIR") or os.path.join(os.path.dirname(REPO), "reference")
    return cand if os.path.isfile(os.path.join(cand, "kernels", "attention.cu")) else ""


def build_dist_lib(force: bool = False) -> str:
    """libhkv_dist.so: host/hkv_seqsplit.hpp behind include/hkv_dist.h; links libhkv and NCCL."""
    srcs = _sources(HOST) + [os.path.join(CSRC, "hkv_dist_api.cpp"), os.path.join(REPO, "include", "hkv_dist.h")]
    if not force and _newer(DIST_LIB, srcs + [LIB]):
        return DIST_LIB
    cmd = [_nvcc(), *ARCH, "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-o", DIST_LIB,
           os.path.join(CSRC, "hkv_dist_api.cpp"), "-I", os.path.join(REPO, "include"), "-I", HOST,
           "-L", PKG_DIR, "-lhkv", "-lnccl", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
    subprocess.run(cmd, check=True)
    return DIST_LIB


def build_watch_tests(force: bool = False) -> str | None:
    """CPU-only tests of hkv_step_watch.hpp (plain g++, no CUDA anywhere)."""
    main = os.path.join(REPO, "tests", "cpp", "hkv_watch_tests.cpp")
    if not os.path.exists(main):
        return None
    srcs = [main, os.path.join(HOST, "hkv_step_watch.hpp")]
    if not force and _newer(WATCH_TESTS, srcs):
        return WATCH_TESTS
    cxx = shutil.which("g++") or "g++"
    subprocess.run([cxx, "-O2", "-std=c++17", "-pthread", "-o", WATCH_TESTS, main, "-I", HOST, "-lrt"], check=True)
    return WATCH_TESTS


def build_seqsplit_tests(force: bool = False) -> str | None:
    """C++ test of SeqSplitDecoder: one process per GPU, NCCL id handed over through a file."""
    main = os.path.join(REPO, "tests", "cpp", "hkv_seqsplit_tests.cpp")
    oracle_dir = os.path.join(REPO, "oracle", "_build")
    if not os.path.exists(main):
        return None
    srcs = _sources(HOST) + [main]
    if not force and _newer(SEQSPLIT_TESTS, srcs + [LIB]):
        return SEQSPLIT_TESTS
    cmd = [_nvcc(), *ARCH, "-O2", "-std=c++17", "-o", SEQSPLIT_TESTS, main,
           "-I", os.path.join(REPO, "include"), "-I", HOST, "-L", PKG_DIR, "-lhkv", "-lnccl",
           "-L", oracle_dir, "-lhkv_oracle",
           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../hector-engine_b200",
           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../oracle/_build"]
    subprocess.run(cmd, check=True)
    return SEQSPLIT_TESTS


def build_gemma4_tests(force: bool = False) -> str | None:
    """C++ tests of Gemma4KVCache and the per-layer BatchedDecodeLoop (oracle linked as the checker)."""
    main = os.path.join(REPO, "tests", "cpp", "hkv_gemma4_tests.cpp")
    oracle_dir = os.path.join(REPO, "oracle", "_build")
    if not os.path.exists(main):
        return None
    srcs = _sources(HOST) + [main]
    if not force and _newer(GEMMA4_TESTS, srcs + [LIB]):
        return GEMMA4_TESTS
    cmd = [_nvcc(), *ARCH, "-O2", "-std=c++17", "-o", GEMMA4_TESTS, main,
           "-I", os.path.join(REPO, "include"), "-I", HOST, "-L", PKG_DIR, "-lhkv", "-L", oracle_dir, "-lhkv_oracle",
           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../hector-engine_b200",
           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../oracle/_build"]
    subprocess.run(cmd, check=True)
    return GEMMA4_TESTS


def build_oracle() -> None:
    subprocess.run(["make", "-s", "-C", os.path.join(REPO, "oracle"), "all", f"REF={reference_dir()}"], check=True)


def build_dropin() -> None:
    """Drop-in test binary against the real engine (only where the reference checkout exists)."""
    subprocess.run(["make", "-s", "-C", os.path.join(REPO, "oracle"), "dropin", f"REF={reference_dir()}"], check=True)


def build_all(force: bool = False) -> None:
    build_lib(force=force)
    build_dist_lib(force=force)
    build_oracle()
    build_host_tests(force=force)
    build_watch_tests(force=force)
    build_seqsplit_tests(force=force)
    build_gemma4_tests(force=force)
    build_dropin()


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built", LIB)
