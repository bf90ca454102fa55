#!/usr/bin/env python3
"""TEST INFRASTRUCTURE ONLY.  Compile two of the reference project's kernels from
its own sources, where they lie, together with the small C shims in this folder:
the split-KV merge (hca/sm100/combine.cu -> oracle/_ref/libref_combine.so) and
the CSA compressor reduce (csa/sm100/kernel.cuh -> oracle/_ref/libref_csa.so);
and stage the reference's Python bench package (its PyTorch decode path
bench/bench/reference.py, its decode harness bench/bench/decode.py and its
candidate plug-ins) under oracle/_ref/pyref/bench, so that a machine without the
reference checkout can time the reference's own CPU code and run its unchanged
harness on this library.  oracle/_ref is a build output: it is not committed.

Only these two are built: they have no spin waits and are safe to run.  The
reference's decode kernel is not built or run (as committed it stalls on an
mbarrier and then traps, hca/sm100/kernel.cu:112-123 with
hca/sm100/helpers.h:29,183-206).

    python oracle/build_ref.py [--reference /path/to/reference]     (or DSV4_REFERENCE in the environment)
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


PYREF = OUT_DIR / "pyref"


def stage_python(reference: Path) -> Path | None:
    """Copy the reference's bench package (Python only, no cloud runner) to oracle/_ref/pyref/bench."""
    src = reference / "bench" / "bench"
    if not (src / "reference.py").exists():
        return None
    dst = PYREF / "bench"
    if dst.exists():
        shutil.rmtree(dst)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "modal", "modal_app.py", "*.pyc"))
    return dst


def reference_from_env() -> Path | None:
    """The reference checkout named by DSV4_REFERENCE, or None."""
    p = os.environ.get("DSV4_REFERENCE")
    return Path(p) if p else None


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("DSV4_REFERENCE"))
    args = ap.parse_args()
    if not args.reference:
        print("give --reference /path/to/reference or set DSV4_REFERENCE", file=sys.stderr)
        return 2
    staged = stage_python(Path(args.reference))
    print(staged if staged else "reference Python not found; nothing staged")
    out = build(Path(args.reference))
    print(out if out else "reference sources not found; nothing built")
    return 0


if __name__ == "__main__":
    sys.exit(main())
