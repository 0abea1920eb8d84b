"""Builds `libkn_b200.so` (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m kyanite_b200.build [--force]

Objects go to `kyanite_b200/csrc/build/`, the library next to this file.  A source is recompiled
when it, or any header, is newer than its object.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(CSRC, "build")
LIB_PATH = os.path.join(PKG_DIR, "libkn_b200.so")

SOURCES = [
    "ir.cpp",
    "strided.cpp",
    "plan.cpp",
    "comm.cpp",
    "executor.cu",
    "kernels/elementwise.cu",
    "kernels/rows.cu",
    "kernels/rows_f16.cu",
    "kernels/gather.cu",
    "kernels/contract_simt.cu",
    "kernels/contract_tc.cu",
    "kernels/conv_chain.cu",
    "kernels/gemm_persistent.cu",
    "kernels/attn_softmax.cu",
    "kernels/attention.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function",
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found")
    return nvcc


def _headers():
    out = [os.path.join(ROOT, "include", "kn_b200.h")]
    for d, _, files in os.walk(CSRC):
        if os.path.basename(d) == "build":
            continue
        out += [os.path.join(d, f) for f in files if f.endswith(".h")]
    return out


def _compile(src: str, force: bool, header_mtime: float, verbose: bool):
    path = os.path.join(CSRC, src)
    obj = os.path.join(OBJ_DIR, src.replace("/", "_") + ".o")
    if not force and os.path.exists(obj):
        if os.path.getmtime(obj) >= max(os.path.getmtime(path), header_mtime):
            return obj, False
    cmd = [_nvcc(), *NVCC_FLAGS, "-x", "cu", "-c", path, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj, True


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile (if needed) and return the path of the shared library."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    header_mtime = max(os.path.getmtime(h) for h in _headers())
    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as pool:
        results = list(pool.map(lambda s: _compile(s, force, header_mtime, verbose), SOURCES))
    objs = [o for o, _ in results]
    rebuilt = any(r for _, r in results)
    if rebuilt or not os.path.exists(LIB_PATH):
        cmd = [_nvcc(), "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", LIB_PATH, *objs, "-lpthread", "-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
