"""Builds libb200kv.so (the C-ABI library) in-tree with nvcc for sm_100a.

Usage: python build.py [--force] [--verbose]
The library lands beside the Python binding (b200kv/libb200kv.so) so that it travels with the tree.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
OUT = os.path.join(HERE, "b200kv", "libb200kv.so")

SOURCES = [
    "capi.cu",
    "kv_move.cu", "kv_gather_tma.cu",
    "mla_decode_simt.cu",
    "mla_decode_tc.cu",
    "kv_block_pool.cpp",
    "kv_arena.cpp",
    "kv_partition.cpp",
    "aclnn_shim.cu", "aclnn_other_ops.cu", "kv_stages.cu", "kv_peer.cu", "kv_indexer.cu", "kv_indexer_tc.cu",
    "no_alloc.cu",
    "kv_engine.cpp",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-I", os.path.join(ROOT, "include"),
    "-I", CSRC,
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the B200 library cannot be built")
    return nvcc


def _host_compiler_args() -> list[str]:
    # Prefer the distribution compiler over a wrapper exported through CXX.
    for cand in ("/usr/bin/g++",):
        if os.path.exists(cand):
            return ["-ccbin", cand]
    return []


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".hpp"))]
    headers.append(os.path.join(ROOT, "include", "b200kv.h"))
    headers.append(os.path.join(ROOT, "include", "b200kv_aclnn.h"))
    headers.append(os.path.abspath(__file__))
    nvcc = _nvcc()
    ccbin = _host_compiler_args()
    sources = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]

    def compile_one(src: str) -> str:
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ_DIR, os.path.splitext(src)[0] + ".o")
        if force or _stale(obj, [path] + headers):
            cmd = [nvcc, *ccbin, *NVCC_FLAGS, "-x", "cu", "-c", path, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            res = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or res.returncode != 0:
                sys.stderr.write(res.stdout + res.stderr)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(compile_one, sources))
    if force or _stale(OUT, objs):
        cmd = [nvcc, *ccbin, "-shared", "-o", OUT, *objs, "-lcudart", "-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link of libb200kv.so failed")
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
