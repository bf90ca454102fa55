#!/usr/bin/env python3
"""TEST INFRASTRUCTURE ONLY.  Compile two of the reference project's kernels from
its own sources, where they lie, together with the small C shims in this folder:
the split-KV merge (hca/sm100/combine.cu -> oracle/_ref/libref_combine.so) and
the CSA compressor reduce (csa/sm100/kernel.cuh -> oracle/_ref/libref_csa.so).

Only these two are built: they have no spin waits and are safe to run.  The
reference's decode kernel is not built or run (as committed it stalls on an
mbarrier and then traps, hca/sm100/kernel.cu:112-123 with
hca/sm100/helpers.h:29,183-206).

    python oracle/build_ref.py [--reference /path/to/reference]
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
OUT = OUT_DIR / "libref_combine.so"


def build(reference: Path, quiet: bool = False) -> Path | None:
    src = reference / "hca" / "sm100" / "combine.cu"
    if not src.exists():
        return None
    OUT_DIR.mkdir(exist_ok=True)
    nvcc = shutil.which(os.environ.get("NVCC", "nvcc")) or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a",
           "-shared", "-Xcompiler", "-fPIC", "-I", str(src.parent),
           "-o", str(OUT), str(HERE / "ref_combine_shim.cu"), str(src)]
    if not quiet:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    csa = reference / "csa" / "sm100" / "kernel.cuh"
    if csa.exists():
        cmd = [nvcc, "-std=c++17", "-O3", "--use_fast_math", "-gencode", "arch=compute_100a,code=sm_100a",
               "-shared", "-Xcompiler", "-fPIC", "-I", str(reference / "csa"),
               "-o", str(OUT_DIR / "libref_csa.so"), str(HERE / "ref_csa_shim.cu")]
        if not quiet:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
    return OUT


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("DSV4_REFERENCE", "/root/reference"))
    args = ap.parse_args()
    out = build(Path(args.reference))
    print(out if out else "reference sources not found; nothing built")
    return 0


if __name__ == "__main__":
    sys.exit(main())
