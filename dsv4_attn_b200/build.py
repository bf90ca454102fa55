#!/usr/bin/env python3
"""Build libdsv4_attn.so in-tree with plain nvcc (no torch, no pybind needed).

    python -m dsv4_attn_b200.build            # builds dsv4_attn_b200/libdsv4_attn.so
    python -m dsv4_attn_b200.build --ptxas-v  # also prints registers / spills / shared memory

The recipe mirrors the reference project's standalone build
(hca/compile.py:68-83): one nvcc call, sm_100a only, a shared object that is
loaded with ctypes.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCE = HERE / "csrc" / "api.cu"
OUT = HERE / "libdsv4_attn.so"
DEPS = sorted((HERE / "csrc").glob("*")) + [HERE.parent / "include" / "dsv4_attn.h"]


def needs_build() -> bool:
    if not OUT.exists():
        return True
    t = OUT.stat().st_mtime
    return any(p.stat().st_mtime > t for p in DEPS)


def build(force: bool = False, ptxas_v: bool = False, quiet: bool = False) -> Path:
    if not force and not needs_build():
        return OUT
    nvcc = shutil.which(os.environ.get("NVCC", "nvcc")) or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-std=c++17", "-O3", "-lineinfo",
           "-gencode", "arch=compute_100a,code=sm_100a",
           "-shared", "-Xcompiler", "-fPIC",
           "-o", str(OUT), str(SOURCE)]
    if ptxas_v:
        cmd[1:1] = ["-Xptxas", "-v"]
    if not quiet:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return OUT


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--ptxas-v", action="store_true")
    args = ap.parse_args()
    build(force=args.force or args.ptxas_v, ptxas_v=args.ptxas_v)
    print(OUT)
    return 0


if __name__ == "__main__":
    sys.exit(main())
