"""Builds ``lib/libflashsinkhorn_b200.so`` from ``csrc/*.cu`` with nvcc for sm_100a (in-tree).

    python -m flash_sinkhorn_b200.build_ext [--force] [--verbose]

nvcc cross-compiles without a GPU. The library links the CUDA runtime statically and
resolves the one driver entry point it needs (tensor-map encoding) at run time, so it
has no load-time dependency beyond libstdc++.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "lib", "libflashsinkhorn_b200.so")
SOURCES = ["fs_api.cu", "fs_simt.cu", "fs_tc.cu", "fs_tck.cu", "fs_static.cu", "fs_micro.cu"]
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [
        os.path.join(os.path.dirname(HERE), "include", "flash_sinkhorn_b200.h"), os.path.abspath(__file__)]
    return any(os.path.getmtime(p) > t for p in deps if os.path.isfile(p))


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", OUT] + [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed ({res.returncode}): {' '.join(cmd)}")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
