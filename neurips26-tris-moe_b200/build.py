"""Builds libtrismoe_b200.so (sm_100a) in-tree with nvcc.

Run as ``python build.py`` from anywhere, or call :func:`build`.  The shared library is
written next to the sources (``csrc/libtrismoe_b200.so``) so that it travels with the
tree; it links the CUDA runtime statically and has no Python or torch dependency.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(CSRC, "libtrismoe_b200.so")
LAST_LOG = ""
SOURCES = ["grouped.cu", "grouped_tiled.cu", "tile_records.cu", "skinny_gemm.cu", "route.cu", "layer.cu", "paging.cu", "tc_gemm.cu", "grouped_umma.cu", "ep_peer.cu", "packed4.cu", "packed4_gemm.cu", "abi.cpp"]
HEADERS = ["common.cuh", "compact3_tile.cuh", "tile_records.cuh", "umma.cuh", os.path.join("..", "..", "include", "trismoe_b200.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _nvcc() -> str:
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found; the trismoe_b200 library cannot be built")
    return path


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every source for sm_100a and link the shared library; returns its path."""
    if not force and not _stale():
        return LIB
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, "-x", "cu", "-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    log = []
    for src, proc in procs:
        out, _ = proc.communicate()
        log.append(f"== {src}\n{out}")
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}")
    global LAST_LOG  # registers / spills / shared memory per kernel (-Xptxas -v), for callers that want it
    LAST_LOG = "\n".join(line for line in "\n".join(log).split("\n") if "Compile time" not in line)
    if verbose:
        print("\n".join(log))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
