"""The reference's own decode harness (bench/bench/decode.py: run_decode_bench), unchanged, run on this
library: its two ctypes candidates bind `hca_decode_fwd` from the shared object that DSV4_HCA_SO names
(bench/bench/candidates/hca_custom_decode.py:39-73), and this repository's plug-in goes through the same
harness.  The harness builds the inputs, runs its own PyTorch forward on them and applies its own tolerance;
the test asserts its verdict.

The harness is a copy of the reference's Python staged by oracle/build_ref.py into a git-ignored folder; it
runs in a child process whose module path puts that copy first, because its package is called `bench`."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
PYREF = ROOT / "oracle" / "_ref" / "pyref"

pytestmark = pytest.mark.gpu

CHILD = r"""
import json, sys, importlib
from dataclasses import asdict
import torch
from bench.decode import run_decode_bench
mod = importlib.import_module(sys.argv[1])
over = json.loads(sys.argv[2])
res = run_decode_bench(mod.candidate, candidate_name=mod.NAME, spec_overrides=over, iters=20, warmup=5,
                       device="cuda", dtype="fp8_dequant", flush_l2=True, seed=0)
print("RESULT " + json.dumps(asdict(res)))
"""

CASES = [
    # the shape the reference harness is run at (B = 64, 128 heads, 896 compressed + 128 window tokens)
    ("bench.candidates.hca_custom_decode", dict(B=64, M_cur=896, swa_len=128)),
    ("bench.candidates.hca_custom_decode_graph", dict(B=64, M_cur=896, swa_len=128)),
    # this repository's plug-in at the 100k-context shape (782 + 128), whose lengths are no multiple of the tile
    ("dsv4_attn_b200.candidates.hca_b200_decode", dict(B=64, M_cur=782, swa_len=128)),
]


@pytest.mark.parametrize("module,overrides", CASES, ids=[c[0].rsplit(".", 1)[1] for c in CASES])
def test_reference_harness_accepts_the_library(module, overrides):
    if not (PYREF / "bench" / "decode.py").exists():
        pytest.skip("the reference's Python is not staged (python oracle/build_ref.py with DSV4_REFERENCE set)")
    from dsv4_attn_b200 import _lib
    env = dict(os.environ)
    env["DSV4_HCA_SO"] = str(_lib.library_path())
    env["PYTHONPATH"] = os.pathsep.join([str(PYREF), str(ROOT)])
    p = subprocess.run([sys.executable, "-c", CHILD, module, json.dumps(overrides)], cwd=str(PYREF), env=env,
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    line = [x for x in p.stdout.splitlines() if x.startswith("RESULT ")][-1]
    res = json.loads(line[len("RESULT "):])
    keep = os.environ.get("DSV4_HARNESS_RESULTS")          # a folder to keep the harness's result records in
    if keep:
        Path(keep).mkdir(parents=True, exist_ok=True)
        (Path(keep) / f"reference_harness_{res['candidate']}.json").write_text(json.dumps(res, indent=1) + "\n")
    print(res)
    assert res["correct"], res
    assert res["message"] == ""
    assert res["cand_ms_mean"] > 0
