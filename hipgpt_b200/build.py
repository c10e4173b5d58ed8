"""Builds libhipgpt_attn.so for sm_100a with nvcc, in-tree (hipgpt_b200/_lib/).

    python -m hipgpt_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library holds the CUDA kernels, the C ABI
(include/hipgpt_attn.h) and the reference-named C++ launchers (include/hipgpt_launchers.hpp).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "_lib")
LIB = os.path.join(LIBDIR, "libhipgpt_attn.so")
OBJDIR = os.path.join(LIBDIR, "obj")

SOURCES = ["attn_fwd_rows.cu", "attn_fwd_tc.cu", "attn_fwd_bf16.cu", "attn_fwd_tc16.cu", "attn_fwd_head.cu", "attn_fwd_generic.cu", "attn_unfused.cu", "attn_bwd.cu", "layer_ops.cu", "attn_decode.cu", "gpt_decode.cu", "probe.cu", "wait_probe.cu", "capi.cu",
           "compat_launchers.cpp", "checkpoint.cpp", "sharded.cpp", "shard_push.cu", "gemm_tc.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "-I", os.path.join(ROOT, "include"), "-I", CSRC]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the library cannot be built here")
    return exe


def _deps():
    out = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    out += [os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include"))]
    out.append(os.path.abspath(__file__))
    return out


def up_to_date() -> bool:
    if not os.path.exists(LIB):
        return False
    t = os.path.getmtime(LIB)
    return all(os.path.getmtime(p) <= t for p in _deps())


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and up_to_date():
        return LIB
    os.makedirs(OBJDIR, exist_ok=True)
    cc = nvcc()
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJDIR, os.path.splitext(src)[0] + ".o")
        cmd = [cc, *ARCH, *NVCC_FLAGS, *extra, "-x", "cu", "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    cmd = [cc, *ARCH, "-shared", "-o", LIB, *objs, "-Xcompiler", "-fPIC", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
