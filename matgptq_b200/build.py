"""Build libmatgptq_b200.so in-tree with nvcc for sm_100a.

    python -m matgptq_b200.build [--force] [--verbose]

The library has no torch or Python dependency: it is the C-ABI boundary declared in
``include/matgptq_b200.h``.  Objects are rebuilt only when a source or header is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")
BUILD_DIR = os.path.join(PKG_DIR, "build")
LIB_PATH = os.path.join(PKG_DIR, "libmatgptq_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libmatgptq_b200")
    return nvcc


def _sources() -> list[str]:
    return sorted(name for name in os.listdir(CSRC) if name.endswith(".cu"))


def _newest_header_mtime() -> float:
    """Newest header, or source that another source includes (gemv_zp.cu compiles gemv.cu a second time)."""
    mt = 0.0
    for d in (CSRC, INCLUDE):
        for name in os.listdir(d):
            if name.endswith((".h", ".cuh")) or name == "gemv.cu":
                mt = max(mt, os.path.getmtime(os.path.join(d, name)))
    return mt


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every ``.cu`` under ``csrc/`` and link the shared library. Returns its path."""
    nvcc = _nvcc()
    os.makedirs(BUILD_DIR, exist_ok=True)
    hdr_mtime = _newest_header_mtime()
    objects = []
    procs = []
    for src in _sources():
        src_path = os.path.join(CSRC, src)
        obj = os.path.join(BUILD_DIR, src.replace(".cu", ".o"))
        objects.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src_path), hdr_mtime)
        if stale:
            cmd = [nvcc, *NVCC_FLAGS, "-I", INCLUDE, "-I", CSRC, "-c", src_path, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
                print(" ".join(cmd), flush=True)
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            failed = True
            sys.stderr.write(f"--- nvcc failed on {src} ---\n{out}\n")
        elif verbose and out:
            print(out)
    if failed:
        raise RuntimeError("nvcc compilation failed")
    relink = force or procs or not os.path.exists(LIB_PATH)
    if relink:
        cmd = [nvcc, "-shared", "-o", LIB_PATH, *objects, "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
