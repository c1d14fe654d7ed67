"""Builds librocwmma_b200.so (all CUDA kernels + the C ABI) for sm_100a, in-tree.

Run as `python -m rocwmma_b200.build`.  nvcc cross-compiles without a GPU.  One object per
.cu file (compiled in parallel, skipped when up to date), then one shared library next to
this file.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
REPO_DIR = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(PKG_DIR, "_obj")
LIB_PATH = os.path.join(PKG_DIR, "librocwmma_b200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-I", os.path.join(REPO_DIR, "include"),
]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime():
    newest = 0.0
    for root in (CSRC, os.path.join(REPO_DIR, "include")):
        for dirpath, _, files in os.walk(root):
            for f in files:
                if f.endswith((".h", ".hpp", ".cuh")):
                    newest = max(newest, os.path.getmtime(os.path.join(dirpath, f)))
    return newest


def _compile_one(src, hdr_mtime, verbose, extra):
    obj = os.path.join(OBJ_DIR, src[:-3] + ".o")
    src_path = os.path.join(CSRC, src)
    if os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src_path), hdr_mtime):
        return obj, ""
    cmd = [NVCC, *NVCC_FLAGS, *extra, "-c", src_path, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    return obj, (res.stdout + res.stderr) if verbose else ""


def build(verbose: bool = False, ptxas_info: bool = False) -> str:
    """Compile every kernel for sm_100a and link librocwmma_b200.so.  Returns its path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    hdr_mtime = _headers_mtime()
    srcs = _sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile_one(s, hdr_mtime, verbose or ptxas_info, extra), srcs))
    objs = [o for o, _ in results]
    for _, log in results:
        if log:
            print(log)
    if (not os.path.exists(LIB_PATH)) or any(os.path.getmtime(o) > os.path.getmtime(LIB_PATH) for o in objs):
        cmd = [NVCC, "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv))
