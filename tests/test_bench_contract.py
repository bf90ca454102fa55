"""The benchmark's reference arm runs on the host cores alone: check its one JSON line
carries the keys the measurement contract names (the GPU arm prints the same keys plus
roofline / clocks; it is exercised on the GPU box)."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_prints_one_json_line():
    import os
    # a launcher's OMP_NUM_THREADS=1 must not put the CPU arm on one core
    env = dict(os.environ, OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "decode_attn_kv_bandwidth" and d["unit"] == "TB/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 1
    assert d["value"] > 0 and d["ms_per_step"] > 0
    assert d["config"]["workload"] == "hca_b64_h128_ctx100k"
    cb = d["cpu_baseline"]
    staged = (ROOT / "oracle" / "_ref" / "pyref" / "bench" / "reference.py").exists()
    assert cb["kind"] == ("reference" if staged else "port")
    assert cb["value"] == d["value"] and "sample" in cb
    usable = len(os.sched_getaffinity(0))
    assert cb["cores"] == usable if staged else cb["cores"] >= 1
    e = d["e2e"]
    assert e["value"] == d["value"] and e["unit"] == d["unit"] and e["h2d_bytes_per_step"] == 0 and e["d2h_bytes_per_step"] == 0
