"""Builds ``libsparsetir_b200.so`` in-tree with nvcc for sm_100a.

Usage: ``python -m sparsetir_b200.build [--force] [--verbose]``.
Objects go to ``build/`` at the repository root; the shared library is written next to this
file so that it travels with the source tree.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(ROOT, "include")
OBJ_DIR = os.path.join(ROOT, "build", "obj")
LIB_PATH = os.path.join(PKG_DIR, "libsparsetir_b200.so")

SOURCES = [
    "runtime.cc", "abi.cc", "format.cc", "validate.cu",
    "csrmm.cu", "hyb_spmm.cu", "sddmm.cu", "bsrmm.cu", "bsrmm_tc.cu", "rgms.cu", "rgms_tc.cu", "rgms_fused.cu", "rgms_noalloc.cu", "rgms_ell3d.cu", "rgms_f16.cu", "tcspmm.cu", "csr_misc.cu", "fusedmm.cu", "peer_scatter.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--extended-lambda", "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall",
    "-I", INCLUDE, "-I", CSRC,
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the library cannot be built")
    return exe


def _newest_header() -> float:
    newest = 0.0
    for d in (CSRC, INCLUDE):
        for f in os.listdir(d):
            if f.endswith((".h", ".cuh")):
                newest = max(newest, os.path.getmtime(os.path.join(d, f)))
    return newest


def _compile(src: str, force: bool, verbose: bool, hdr_mtime: float) -> str:
    obj = os.path.join(OBJ_DIR, src + ".o")
    path = os.path.join(CSRC, src)
    if (not force and os.path.exists(obj)
            and os.path.getmtime(obj) > max(os.path.getmtime(path), hdr_mtime)):
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-x", "cu", "-c", path, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(f"$ {' '.join(cmd)}\n{res.stdout}{res.stderr}")
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}")
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr = _newest_header()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as pool:
        objs = list(pool.map(lambda s: _compile(s, force, verbose, hdr), SOURCES))
    if (force or not os.path.exists(LIB_PATH)
            or os.path.getmtime(LIB_PATH) < max(os.path.getmtime(o) for o in objs)):
        cmd = [_nvcc(), "-shared", "-o", LIB_PATH, *objs, "-gencode",
               "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
