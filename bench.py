#!/usr/bin/env python3
"""Decode-attention benchmark (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the decode-attention hot path over one batch of synthetic
requests whose KV cache is already resident in HBM (as it is in a serving
engine and in the reference's own decode harness).  The headline workload is
HCA dense decode at B=64 requests per GPU, H=128 heads, 100,000 tokens of raw
context (782 compressed entries + a 128-entry window); the CSA configurations
are measured in the same run and reported under "other_workloads".

Metric: achieved KV bytes per second = (entries attended to x 656 bytes) / step
time, aggregated over all GPUs, next to microseconds per layer.

Timing: the K timed steps are captured into one CUDA graph and replayed between
two events, the way a serving engine runs its decode layers (and the way the
reference's own graph candidate is timed).  Step i works on instance i mod R of
the workload - R independent copies with their own KV pools, queries and outputs,
R chosen so that the copies together are several times larger than L2 - so every
step finds its inputs in HBM, not in L2, without a flush inside the timed region
(the timed replay follows an untimed replay, the barrier and one untimed pass over
the instances in rotation order; where a workload is too small for such a rotation
L2 is emptied before the timed replay instead).
The same step timed alone (L2 emptied by a 512 MiB write and a read of the same buffer before each launch, one
event pair per launch, eager launch) is reported beside it as "isolated".
`--impl reference` times the reference's own PyTorch decode path
(bench/bench/reference.py, hca_decode_forward in fp32 mode on exactly dequantised,
gathered rows) on the host cores, on a bounded sample of the same workload; where
the staged copy of the reference's Python is absent it falls back to the numpy
restatement (the oracle) and says "port".

After every timed region, and outside it, a sample of rows of the step's result is
compared with the CPU oracle; the line carries the errors and the run fails when they
are out of tolerance.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

ENTRY_BYTES = 656
L2_FLUSH_BYTES = 512 << 20
METRIC = "decode_attn_kv_bandwidth"
UNIT = "TB/s"

WORKLOADS = {
    # name: (kind, kwargs)  -- shapes of the benchmark configurations.  num_splits = n: the static grid of
    # rows x head groups x n blocks; plan_splits = n: resident blocks walking a plan of the device scheduler
    # (n = 0: the scheduler balances, n >= 1: exactly n pieces per row and head group)
    "hca_b64_h128_ctx100k": ("hca", dict(B=64, s_q=1, H=128, kv_len=782, win_len=128, num_splits=1)),
    "csa_b64_h128_topk512_ctx3072": ("csa", dict(B=64, s_q=1, H=128, n_entries=768, topk=512, num_splits=1)),
    # configuration 3 with the 8 splits it names: as 8 scheduled pieces per row, and on the static grid
    "csa_b128_nextn2_topk2048_ctx100k_split8": ("csa", dict(B=128, s_q=2, H=128, n_entries=25000, topk=2048, plan_splits=8)),
    "csa_b128_nextn2_topk2048_ctx100k_split8_static_grid": ("csa", dict(B=128, s_q=2, H=128, n_entries=25000, topk=2048, num_splits=8)),
    # the same shape with the cutting left to the scheduler
    "csa_b128_nextn2_topk2048_ctx100k_planned": ("csa", dict(B=128, s_q=2, H=128, n_entries=25000, topk=2048, plan_splits=0)),
    "csa_b64_h128_topk2048_ctx100k": ("csa", dict(B=64, s_q=1, H=128, n_entries=25000, topk=2048, num_splits=1)),
    # small batches, where the scheduler has to spread few rows over all SMs
    "hca_b8_h128_ctx100k_planned": ("hca", dict(B=8, s_q=1, H=128, kv_len=782, win_len=128, plan_splits=0)),
    "csa_b8_h128_topk2048_ctx100k_planned": ("csa", dict(B=8, s_q=1, H=128, n_entries=25000, topk=2048, plan_splits=0)),
}
PARITY_ROWS = 16
TOL = dict(max_abs=2e-2, mean_abs=2e-3, lse_rel=1e-3)
# The mixed data-parallel workload: a global batch of 1024 requests with log-normal raw
# context (median 8k, sigma 1.0 - the configuration leaves sigma open - clipped to
# [1k, 128k]), sharded over the GPUs by context length; one CSA layer and one HCA layer
# back to back per step.  Strong scaling: the global batch is fixed.
MIXED = "mixed_1024req_lognormal_csa+hca"
MIXED_REQUESTS = 1024
DEFAULT_WORKLOAD = "hca_b64_h128_ctx100k"
# DRAM bytes (read + write) of ONE launch of the decode kernel on the workload, from an ncu
# capture of that launch (dram__bytes_read.sum + dram__bytes_write.sum); the summaries
# under profiles/ hold the figures and the command lines.
NCU_DRAM_TRAFFIC = {"hca_b64_h128_ctx100k": 47.79e6, "csa_b64_h128_topk512_ctx3072": 32.43e6,
                    # captured on the B = 16 slice of the same shape (27.51 MB per launch) and scaled by the rows
                    "csa_b64_h128_topk2048_ctx100k": 4 * 27.51e6}
NCU_TRAFFIC_SOURCE = "ncu capture of one launch (profiles/decode_mma_kernel_*.md)"


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def tensor_view(kv_bytes, H, ms):
    """Achieved tensor throughput of one step (QK over 576 columns + PV over 512 per head and
    attended entry) against the measured dense BF16 GEMM peak, for context next to the HBM view."""
    flops = 2.0 * H * (576 + 512) * (kv_bytes / ENTRY_BYTES)
    peak = None
    try:
        peak = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops"])
    except Exception:
        pass
    tf = flops / (ms * 1e-3) / 1e12
    src = "measured" if peak else "fallback"
    peak = peak or 1590.0
    return {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "peak_source": src,
            "note": "useful FLOPs only; each block also recomputes QK for the other half of the value columns"}


# ───────────────────────── clocks sampling ─────────────────────────

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, reasons = [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 7:
                    continue
                try:
                    sm.append(float(f[0]))
                    out["sm_max_mhz"] = float(f[1])
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out["sm_mhz"] = statistics.median(sm)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


# ───────────────────────── our arm ─────────────────────────

def build_workload(name, seed, device):
    from dsv4_attn_b200 import synth
    kind, kw = WORKLOADS[name]
    kw = dict(kw)
    mode = {"num_splits": kw.pop("num_splits", None), "plan_splits": kw.pop("plan_splits", None)}
    if kind == "hca":
        w = synth.make_hca(seed, device=device, **kw)
    else:
        w = synth.make_csa(seed, device=device, **kw)
    return kind, w, mode


def build_mixed(rank, world, device):
    from dsv4_attn_b200 import dp, synth
    ctx = synth.lognormal_contexts(MIXED_REQUESTS, seed=0)
    mine = dp.shard_requests(MIXED_REQUESTS, world, rank, cost=ctx, balance="sorted_round_robin")
    return synth.make_mixed(4000 + rank, [ctx[i] for i in mine], device=device), len(mine)


def make_step(kind, w, mode):
    """Returns (fn() -> (out, lse), launches per call, description of the split mode, status, plan).  All buffers
    (outputs, split workspace, the plan) are made once, outside the timed region: a plan depends on the
    batch's lengths only and serves every layer of a decode step."""
    import torch
    import dsv4_attn_b200 as lib
    B, s_q, H, _ = w.q.shape
    rows = B * s_q
    dev = w.q.device
    plan_splits, splits = mode.get("plan_splits"), mode.get("num_splits")
    plan = ws = None
    if plan_splits is not None:
        if kind == "hca":
            plan = lib.plan_hca(B, s_q, H, w.kv_len, w.win_len, num_splits=plan_splits)
        else:
            plan = lib.plan_csa(B, s_q, H, w.indices.shape[-1], topk_len=w.topk_len, kv_len=w.kv_len, num_splits=plan_splits)
        desc = f"scheduled, {plan_splits if plan_splits else 'balanced'} pieces"
        launches = 2
    else:
        if splits is None:
            splits = lib.plan_splits(rows, H, w.max_len if kind == "hca" else w.indices.shape[-1])
        ws = lib.alloc_workspace(rows, H, splits, dev) if splits > 1 else None
        desc = f"static grid, {splits} split(s)"
        launches = 2 if splits > 1 else 1
    # out and lse live in one buffer, so that a host that wants them gets them with one copy
    res = torch.empty(rows * H * 512 * 2 + rows * H * 4, dtype=torch.uint8, device=dev)
    out = res[:rows * H * 512 * 2].view(torch.bfloat16).view(B, s_q, H, 512)
    lse = res[rows * H * 512 * 2:].view(torch.float32).view(B, s_q, H)
    status = lib.new_status(dev)
    if kind == "hca":
        def fn(q=None, kv_len=None, win_len=None):
            return lib.hca_dense_decode(w.q if q is None else q, w.kv_pool, w.block_table,
                                        w.kv_len if kv_len is None else kv_len, w.win_pool,
                                        w.win_len if win_len is None else win_len, w.sm_scale,
                                        attn_sink=w.attn_sink, num_splits=splits, out=out, lse=lse,
                                        workspace=ws, status=status, max_len=w.max_len, plan=plan)
    else:
        def fn(q=None, indices=None):
            return lib.csa_sparse_decode(w.q if q is None else q, w.kv_pool, w.block_table,
                                         w.indices if indices is None else indices, w.sm_scale, kv_len=w.kv_len,
                                         topk_len=w.topk_len, num_splits=splits, out=out, lse=lse, workspace=ws,
                                         status=status, plan=plan)
    fn.result = res
    return fn, launches, desc, status, plan


def parity_sample(kind, w, out, lse, count=PARITY_ROWS):
    """Rows of a step's result against the CPU oracle (outside every timed region).  Raises when out of tolerance."""
    from oracle import sample_check as sc
    if kind == "hca":
        rows = sc.pick_rows(w.kv_len + w.win_len, count)
        r = sc.check_hca_rows(w.q, w.kv_pool, w.block_table, w.kv_len, w.win_pool, w.win_len, w.sm_scale, out, lse, rows,
                              sink=w.attn_sink)
    else:
        rows = sc.pick_rows(w.topk_len, count)
        r = sc.check_csa_rows(w.q, w.kv_pool, w.block_table, w.indices, w.sm_scale, out, lse, rows, kv_len=w.kv_len,
                              topk_len=w.topk_len)
    if not sc.within_tolerance(r, **TOL):
        raise RuntimeError(f"result out of tolerance against the oracle: {r}")
    return {k: r[k] for k in ("parity_checked_rows", "max_abs", "mean_abs", "lse_rel")}


class L2Flush:
    """Empties L2 before an isolated launch: a write of a buffer four times the size of L2, then a read of it.  The
    write alone would leave L2 full of DIRTY lines, which the launch under test then has to write back while it
    runs (up to 126 MB of extra DRAM writes: 6-10 us on the short streaming kernels, against their times under the
    profiler); after the read what is left in L2 is clean."""

    def __init__(self, device):
        import torch
        self.buf = torch.empty(L2_FLUSH_BYTES // 4, dtype=torch.int32, device=device)
        self.sink = torch.empty((), dtype=torch.int64, device=device)

    def zero_(self):
        self.buf.zero_()
        self.sink.copy_(self.buf.sum())


def time_steps(fn, steps, warmup, flush, barrier):
    """Device time of `steps` calls, each timed alone with L2 flushed before it; returns list of ms."""
    import torch
    for _ in range(warmup):
        flush.zero_()
        fn()
    barrier()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        flush.zero_()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    barrier()
    return [s.elapsed_time(e) for s, e in zip(starts, ends)]


def time_rotating(fns, steps, warmup, flush, barrier, flush_first=True):
    """Device time (ms) of `steps` back-to-back calls, call i on fns[i % R], replayed from
    one CUDA graph; falls back to eager launches if capture is not possible.  Returns
    (total_ms, "graph" | "eager")."""
    import torch
    R = len(fns)
    for i in range(max(warmup, R)):
        fns[i % R]()
    torch.cuda.synchronize()
    graph = None
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(steps):
                fns[i % R]()
        graph = g
    except Exception as e:  # noqa: BLE001 - report and time eagerly instead
        print(f"[bench] CUDA graph capture failed ({type(e).__name__}: {e}); timing eager launches", file=sys.stderr)
        torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    if graph is not None:
        graph.replay()          # untimed: uploads the graph
    # Where the instances together are several times larger than L2 the timed replay follows the untimed one
    # directly (every step's inputs have been pushed out of L2 by the steps since their last use; clocks and
    # address translation are as warm as inside a decode step that has other layers around it).  Smaller
    # rotations get L2 emptied first.
    if flush_first:
        flush.zero_()
    barrier()
    torch.cuda.synchronize()
    if not flush_first:
        # One untimed pass in rotation order, enqueued directly ahead of the timed replay (after the barrier and the
        # synchronisation, whose idle time would otherwise let the clocks drop): instance 0, which the replay starts
        # with, is then the one used longest ago, and every instance is reused only after all the others.
        for f in fns:
            f()
    e0.record()
    if graph is not None:
        graph.replay()
    else:
        for i in range(steps):
            fns[i % R]()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1), ("graph" if graph is not None else "eager")


def bind_near_gpu(dev):
    """Keep this rank on the cores (and so its pinned buffers in the memory) of the NUMA node its GPU hangs on.
    A launcher leaves the ranks unbound, and a pinned buffer on the far socket has to cross the socket link on every
    copy.  Changes this process's CPU affinity only; returns what it found, for the record."""
    import torch
    info = {"numa_node": None, "cpus_before": None, "cpus_after": None}
    try:
        info["cpus_before"] = len(os.sched_getaffinity(0))
        pr = torch.cuda.get_device_properties(dev)
        bus = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        node = int(Path(f"/sys/bus/pci/devices/{bus}/numa_node").read_text().strip())
        info["numa_node"] = node
        if node >= 0:
            cpus = set()
            for part in Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
            cpus &= os.sched_getaffinity(0)
            if cpus:
                os.sched_setaffinity(0, cpus)
        info["cpus_after"] = len(os.sched_getaffinity(0))
    except Exception as e:  # noqa: BLE001 - a box without that sysfs view: stay unbound
        info["error"] = f"{type(e).__name__}: {e}"
    return info


def e2e_steps(kind, insts, steps, warmup, flush, barrier):
    """Same metric through the public API with HOST buffers: every step copies its inputs
    (q and the per-step index / length tensors) from pinned host memory, runs the decode,
    and reads the result (out, lse) back to pinned host memory.  The inputs of a step lie in ONE pinned
    buffer and go up in one copy; out and lse share one device buffer and come back in one copy.  The three
    stages run on their own streams (copy-in, compute, copy-out) chained by events, so that the copies of
    neighbouring steps overlap the compute, as a serving engine would run them; step i
    works on instance i mod R (its own KV pool, staging and output buffers).  Returns
    (total ms of the K steps, h2d bytes per step, d2h bytes per step, copy rates) - the last being the
    host link measured with the same buffers and no compute: uploads alone, downloads alone, both at once."""
    import torch
    R = len(insts)
    dev = insts[0][0].q.device
    s_in, s_c, s_out = (torch.cuda.Stream(dev) for _ in range(3))
    main = torch.cuda.current_stream(dev)
    slots = []
    for w, fn, _ in insts:
        parts = [w.q] + ([w.kv_len, w.win_len] if kind == "hca" else [w.indices])
        offs, total = [], 0
        for t in parts:
            offs.append(total)
            total += -(-t.numel() * t.element_size() // 256) * 256
        hin = torch.empty(total, dtype=torch.uint8).pin_memory()
        din = torch.empty(total, dtype=torch.uint8, device=dev)
        views = []
        for t, o in zip(parts, offs):
            nb = t.numel() * t.element_size()
            hin[o:o + nb].copy_(t.contiguous().view(-1).view(torch.uint8).cpu())
            views.append(din[o:o + nb].view(t.dtype).view(t.shape))
        fn()
        hres = torch.empty(fn.result.numel(), dtype=torch.uint8).pin_memory()
        slots.append(dict(fn=fn, hin=hin, din=din, views=views, hres=hres, ev_in=torch.cuda.Event(), ev_c=None, ev_o=None))
    z = slots[0]
    h2d = sum(t.numel() * t.element_size() for t in z["views"])
    d2h = z["hres"].numel()
    torch.cuda.synchronize()

    def run(n):
        for i in range(n):
            k = slots[i % R]
            with torch.cuda.stream(s_in):
                if k["ev_c"] is not None:
                    s_in.wait_event(k["ev_c"])          # this instance's staging buffer is free again
                k["din"].copy_(k["hin"], non_blocking=True)
                k["ev_in"].record(s_in)
            with torch.cuda.stream(s_c):
                s_c.wait_event(k["ev_in"])
                if k["ev_o"] is not None:
                    s_c.wait_event(k["ev_o"])           # its previous result has been read back
                k["fn"](*k["views"])
                k["ev_c"] = torch.cuda.Event()
                k["ev_c"].record(s_c)
            with torch.cuda.stream(s_out):
                s_out.wait_event(k["ev_c"])
                k["hres"].copy_(k["fn"].result, non_blocking=True)
                k["ev_o"] = torch.cuda.Event()
                k["ev_o"].record(s_out)

    run(max(warmup, R))
    torch.cuda.synchronize()
    side = (s_in, s_c, s_out)

    def fresh_events():
        for k in slots:
            k["ev_c"] = k["ev_o"] = None
            k["ev_in"] = torch.cuda.Event()

    # The K steps (copies, launches and their event edges over the three streams) are captured into
    # one CUDA graph: enqueueing them from Python takes longer per step than the step itself.
    graph = None
    try:
        fresh_events()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            cap = torch.cuda.current_stream(dev)
            for st in side:
                st.wait_stream(cap)
            run(steps)
            for st in side:
                cap.wait_stream(st)
        graph = g
        graph.replay()
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001 - report and time eager enqueueing instead
        print(f"[bench] e2e graph capture failed ({type(e).__name__}: {e}); timing eager launches", file=sys.stderr)
        torch.cuda.synchronize()
        fresh_events()
    flush.zero_()
    barrier()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record(main)
    if graph is not None:
        graph.replay()
    else:
        for st in side:
            st.wait_event(e0)
        run(steps)
        for st in side:
            done = torch.cuda.Event()
            done.record(st)
            main.wait_event(done)
    e1.record(main)
    torch.cuda.synchronize()
    barrier()
    total = e0.elapsed_time(e1)

    # the host link alone, all ranks at the same time: the same buffers, no compute
    def copies(up, down):
        barrier()
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record(main)
        s_in.wait_event(a0)
        s_out.wait_event(a0)
        for i in range(steps):
            k = slots[i % R]
            if up:
                with torch.cuda.stream(s_in):
                    k["din"].copy_(k["hin"], non_blocking=True)
            if down:
                with torch.cuda.stream(s_out):
                    k["hres"].copy_(k["fn"].result, non_blocking=True)
        main.wait_stream(s_in)
        main.wait_stream(s_out)
        a1.record(main)
        torch.cuda.synchronize()
        return a0.elapsed_time(a1) / steps
    copies(True, True)
    up_ms, down_ms, both_ms = copies(True, False), copies(False, True), copies(True, True)
    rates = {"h2d_alone_gbs": h2d / up_ms / 1e6, "d2h_alone_gbs": d2h / down_ms / 1e6,
             "both_ms_per_step": both_ms, "both_gbs_sum": (h2d + d2h) / both_ms / 1e6}
    return total, h2d, d2h, rates


PYREF = ROOT / "oracle" / "_ref" / "pyref"


def claim_host_threads():
    """All host cores for the CPU arm: launchers such as torchrun export OMP_NUM_THREADS=1, which would
    time the reference on one core.  Has to run before torch (and its OpenMP runtime) is imported."""
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0)) or n
    except (AttributeError, OSError):
        pass
    for var in ("OMP_NUM_THREADS", "MKL_NUM_THREADS", "OPENBLAS_NUM_THREADS"):
        os.environ[var] = str(n)
    return n


def reference_python():
    """The reference's own decode forward (bench/bench/reference.py, staged unchanged by oracle/build_ref.py
    into a git-ignored folder), or None when it has not been staged."""
    if not (PYREF / "bench" / "reference.py").exists():
        return None
    # loaded by path under a name of its own: the reference's package is called "bench", like this file
    name = "dsv4_reference_python"
    if name in sys.modules:
        return sys.modules[name]
    try:
        import importlib.util
        spec = importlib.util.spec_from_file_location(name, PYREF / "bench" / "reference.py")
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod
    except Exception as e:  # noqa: BLE001
        sys.modules.pop(name, None)
        print(f"[bench] staged reference does not import ({type(e).__name__}: {e}); using the oracle port", file=sys.stderr)
        return None


def cpu_sample_case(kind, name, seed, sample_B):
    """A bounded sample of the workload as host arrays: (q [rows, H, 576], rows of exactly dequantised cache
    entries per query row [rows, n, 576], sink or None, sm_scale, attended entries).  Every row of these
    workloads attends to the same number of entries, so the sample is one dense batch."""
    import numpy as np
    from oracle import dsv4_oracle as orc
    kw = {k: v for k, v in WORKLOADS[name][1].items() if k not in ("num_splits", "plan_splits")}
    kw["B"] = sample_B
    if kind == "hca":
        c = orc.make_hca_case(seed, **kw)
        rows = []
        for b in range(sample_B):
            for j in range(kw["s_q"]):
                n, wl = int(c.kv_len[b, j]), int(c.win_len[b, j])
                ent = np.concatenate([orc.gather_rows(c.pool, c.block_table[b], np.arange(n)), c.win[b, :wl]], 0)
                rows.append(orc.unpack_entries(ent))
        sink = c.sink
    else:
        c = orc.make_csa_case(seed, **kw)
        rows = [orc.unpack_entries(orc.gather_rows(c.pool, c.block_table[b], c.indices[b, j]))
                for b in range(sample_B) for j in range(kw["s_q"])]
        sink = None
    kv = np.stack(rows)
    q = c.q.reshape(-1, c.q.shape[2], c.q.shape[3])
    return q, kv, sink, c.sm_scale, int(kv.shape[0] * kv.shape[1])


def cpu_baseline(kind, name, seed=0, target_s=10.0, sample_B=4):
    """The reference's CPU implementation of the decode path, timed on the host cores on a bounded sample
    of the workload's requests: the reference's own hca_decode_forward(dtype="fp32") (bench/bench/reference.py:471-546)
    on the exactly dequantised (and, for the sparse layer, gathered) rows - what the reference itself checks its
    kernels against.  Falls back to the numpy restatement (kind "port") when the reference's Python is not staged."""
    import numpy as np
    full_B = WORKLOADS[name][1]["B"]
    q, kv, sink, sm_scale, entries = cpu_sample_case(kind, name, seed, sample_B)
    ref = reference_python()
    if ref is not None:
        import torch
        threads = claim_host_threads()
        torch.set_num_threads(threads)
        H = q.shape[1]
        tq = torch.from_numpy(q).to(torch.bfloat16)
        tk = torch.from_numpy(kv)
        empty = torch.zeros(tk.shape[0], 0, 512)
        inp = ref.HCADecodeInputs(
            Q=tq, Kc=tk[..., :512].contiguous(), Kc_rope=tk[..., 512:].to(torch.bfloat16), Kc_scales=None,
            Kswa=empty, Kswa_rope=torch.zeros(tk.shape[0], 0, 64, dtype=torch.bfloat16), Kswa_scales=None,
            sink_logits=torch.full((H,), float("-inf")) if sink is None else torch.from_numpy(sink), sm_scale=float(sm_scale))
        run = lambda: ref.hca_decode_forward(inp, dtype="fp32")
        kind_s, how = "reference", "the reference's hca_decode_forward(dtype='fp32'), torch CPU"
        threads_used = torch.get_num_threads()
    else:
        from oracle import dsv4_oracle as orc
        run = lambda: [orc.attend(q[i], kv[i], sm_scale, sink) for i in range(q.shape[0])]
        kind_s, how = "port", "numpy float32 restatement (the staged reference Python was not found)"
        try:
            import threadpoolctl
            threads_used = max([p.get("num_threads", 1) for p in threadpoolctl.threadpool_info()] or [1])
        except Exception:
            threads_used = os.cpu_count() or 1
    run()
    t0 = time.perf_counter()
    iters = 0
    while True:
        run()
        iters += 1
        if time.perf_counter() - t0 > target_s or iters >= 5000:
            break
    dt = (time.perf_counter() - t0) / iters
    return {"value": entries * ENTRY_BYTES / dt / 1e12, "unit": UNIT, "cores": threads_used, "kind": kind_s,
            "sample": f"{sample_B} of {full_B} requests of {name}, {iters} passes, {how}",
            "ms_per_sample_pass": dt * 1e3, "ms_per_full_step": dt * 1e3 * full_B / sample_B, "host_cpus": os.cpu_count()}


AUX_CASES = ("csa_compress_reduce_b1_n65536_c512", "hca_compress_insert_b1_n65536_c576_m128", "kv_quantize_insert_65536rows",
             "rope_norm_65536x16x576", "combine_fp32_partials_8x256rows", "indexer_topk_b64_n25000_k2048")
# decode cases for profiler captures only: a quarter of the batch of the 100k-context sparse configuration
PROFILE_CASES = {
    "csa_b16_h128_topk2048_ctx100k": ("csa", dict(B=16, s_q=1, H=128, n_entries=25000, topk=2048, num_splits=1)),
    "csa_b16_h128_topk2048_ctx100k_split8_static_grid": ("csa", dict(B=16, s_q=1, H=128, n_entries=25000, topk=2048, num_splits=8)),
    "csa_b16_h128_topk2048_ctx100k_split8": ("csa", dict(B=16, s_q=1, H=128, n_entries=25000, topk=2048, plan_splits=8)),
}


def aux_case(name, dev):
    """The kernels either side of the decode (cache write, pre-pass, merge, indexer) on fixed synthetic inputs.
    Returns (fn, algorithmic bytes per call, extra fields for the report, check() to call after timing)."""
    import torch
    import dsv4_attn_b200 as lib
    ok = lambda: None
    if name == "csa_compress_reduce_b1_n65536_c512":
        # the CSA compressor's second pass (a pure streaming kernel)
        Bc, nc, cc = 1, 65536, 512
        streams = [torch.randn(Bc, nc, cc, device=dev).to(torch.bfloat16) for _ in range(4)]
        biases = [torch.randn(4, cc, device=dev).to(torch.bfloat16) for _ in range(2)]
        cout = torch.empty(Bc, nc // 4, cc, dtype=torch.bfloat16, device=dev)
        return (lambda: lib.csa_compress_reduce_fwd(*streams, *biases, 4, out=cout)), 4 * Bc * nc * cc * 2 + cout.numel() * 2, {}, ok
    if name == "hca_compress_insert_b1_n65536_c576_m128":
        # the HCA compressor fused with the FP8 quantiser and the paged-cache insert
        nh, ch, mh = 65536, 576, 128
        Ch = torch.randn(1, nh, ch, device=dev).to(torch.bfloat16)
        Zh = (2 * torch.randn(1, nh, ch, device=dev)).to(torch.bfloat16)
        bh = torch.randn(mh, ch, device=dev).to(torch.bfloat16)
        n_new = nh // mh
        pages = (n_new + 63) // 64
        pool_h = torch.zeros(pages, 64, ENTRY_BYTES, dtype=torch.uint8, device=dev)
        bt_h = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
        pos_h = torch.zeros(1, dtype=torch.int32, device=dev)
        return (lambda: lib.hca_compress_fwd(Ch, Zh, bh, mh, kv_pool=pool_h, block_table=bt_h, insert_pos=pos_h, want_out=False)), \
            2 * nh * ch * 2 + n_new * ENTRY_BYTES, {}, ok
    if name == "kv_quantize_insert_65536rows":
        Tq, ch = 65536, 576
        rows_q = torch.randn(1, Tq, ch, device=dev).to(torch.bfloat16)
        pages = Tq // 64
        pool_q = torch.zeros(pages, 64, ENTRY_BYTES, dtype=torch.uint8, device=dev)
        bt_q = torch.randperm(pages, device=dev).to(torch.int32).view(1, pages)
        pos = torch.zeros(1, dtype=torch.int32, device=dev)
        return (lambda: lib.kv_quantize_insert(rows_q, pool_q, bt_q, pos)), Tq * (ch * 2 + ENTRY_BYTES), {}, ok
    if name == "rope_norm_65536x16x576":
        # RoPE + RMS norm pre-pass on a prefill-sized batch of query vectors
        xr = torch.randn(65536, 16, 576, device=dev).to(torch.bfloat16)
        posr = torch.randint(0, 100000, (65536,), dtype=torch.int32, device=dev)
        wr = torch.ones(576, dtype=torch.bfloat16, device=dev)
        outr = torch.empty_like(xr)
        return (lambda: lib.rope_norm(xr, posr, norm_weight=wr, out=outr)), 2 * xr.numel() * 2, {}, ok
    if name.startswith("combine_"):
        # the split merge on its own: 8 splits of 256 rows x 128 heads x 512 values, the shape of the sparse
        # configuration with 8 splits, on FP32 partials (the reference's convention: its merge kernel reads
        # the same bytes; the library's own split path writes BF16 partials and is covered by the split cases)
        S, N, H = 8, 256, 128
        po = torch.randn(S, N, H, 512, device=dev)
        pl = torch.randn(S, N, H, device=dev)
        out = torch.empty(N, H, 512, dtype=torch.bfloat16, device=dev)
        lse = torch.empty(N, H, dtype=torch.float32, device=dev)
        return (lambda: lib.combine(po, pl, out=out, lse=lse)), po.numel() * po.element_size() + pl.numel() * 4 + out.numel() * 2 + lse.numel() * 4, {}, ok
    if name == "indexer_topk_b64_n25000_k2048":
        # the step before the sparse decode: FP8 scoring of every visible entry + top-k
        Bi, ni, ki = 64, 25000, 2048
        pages_per = (ni + 63) // 64
        qf = torch.randint(0, 120, (Bi, 1, 64, 128), dtype=torch.uint8, device=dev)       # positive e4m3 bytes below NaN
        qf = qf | (torch.randint(0, 2, qf.shape, dtype=torch.uint8, device=dev) << 7)      # random signs
        qw = torch.randn(Bi, 1, 64, device=dev)
        kp = torch.randint(0, 120, (Bi * pages_per, 8448), dtype=torch.uint8, device=dev)
        kp[:, :8192] |= (torch.randint(0, 2, (Bi * pages_per, 8192), dtype=torch.uint8, device=dev) << 7)
        kp[:, 8192:] = torch.rand(Bi * pages_per, 64, device=dev).add_(0.5).view(torch.uint8).view(Bi * pages_per, 256)
        bti = torch.randperm(Bi * pages_per, device=dev).to(torch.int32).view(Bi, pages_per)
        nv = torch.full((Bi, 1), ni, dtype=torch.int32, device=dev)
        sc_ws = torch.empty(Bi, pages_per * 64, dtype=torch.float32, device=dev)
        oi = torch.empty(Bi, 1, ki, dtype=torch.int32, device=dev)
        st_i = lib.new_status(dev)

        def check():
            if st_i.cpu().tolist() != [0, 0, 0, 0]:
                raise RuntimeError("indexer: the kernel reported a status")
        return (lambda: lib.indexer_topk(qf, qw, kp, bti, nv, ki, scores=sc_ws, out=oi, status=st_i)), Bi * ni * 132, {"launches": 2}, check
    raise KeyError(name)


def run_single(args):
    """One instance of one case, W + K eager calls with L2 flushed before each: the small run that profiler
    captures are taken on.  Prints one short JSON line (not the benchmark's line)."""
    import torch
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = L2Flush(dev)
    name = args.single
    parity = None
    if name in AUX_CASES:
        fn, nbytes, _, check = aux_case(name, dev)
    else:
        kind, kw = {**WORKLOADS, **PROFILE_CASES}[name]
        from dsv4_attn_b200 import synth
        kw = dict(kw)
        mode = {"num_splits": kw.pop("num_splits", None), "plan_splits": kw.pop("plan_splits", None)}
        w = (synth.make_hca if kind == "hca" else synth.make_csa)(1000, device=dev, **kw)
        fn, _, _, status, _ = make_step(kind, w, mode)
        nbytes = w.kv_bytes

        def check():
            if status.cpu().tolist() != [0, 0, 0, 0]:
                raise RuntimeError(f"{name}: the decode kernel reported status={status.cpu().tolist()}")
    t = time_steps(fn, args.steps, args.warmup, flush, lambda: None)
    check()
    if name not in AUX_CASES:
        o, l = fn()
        torch.cuda.synchronize()
        parity = parity_sample(kind, w, o, l, count=8)
    ms = statistics.mean(t)
    print(json.dumps({"single": name, "us": ms * 1e3, "bytes": nbytes, "gb_per_s": nbytes / (ms * 1e-3) / 1e9, "parity": parity}),
          file=args.out, flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    binding = bind_near_gpu(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        barrier = lambda: dist.barrier()
    else:
        barrier = lambda: None
    flush = L2Flush(dev)

    l2_bytes = int(torch.cuda.get_device_properties(dev).L2_cache_size)

    def measure(name, steps, warmup, with_e2e):
        """R instances of the workload (together > 3x L2); the K steps rotate over them."""
        insts = []
        kind, w, mode = build_workload(name, seed=1000 + rank, device=dev)
        B, s_q, H, _ = w.q.shape
        footprint = w.kv_bytes + w.q.numel() * 2 + B * s_q * H * 512 * 2
        R = max(1, min(12, -(-3 * l2_bytes // footprint)))
        plan_ms = None
        for r in range(R):
            if r > 0:
                kind, w, mode = build_workload(name, seed=1000 + rank + 101 * r, device=dev)
            fn, launches, desc, status, plan = make_step(kind, w, mode)
            insts.append((w, fn, status))
        if plan is not None:
            # what making a plan costs (one launch of the scheduler kernel), outside the step: a plan depends on
            # the batch's lengths only, so a decode step makes it once and all its layers use it
            plan_ms = statistics.mean(time_steps(plan.remake, 5, 3, flush, barrier))
        covers_l2 = R * footprint >= 3 * l2_bytes
        total_ms, tmode = time_rotating([f for _, f, _ in insts], steps, warmup, flush, barrier, flush_first=not covers_l2)
        w0, fn0, _ = insts[0]
        iso = time_steps(fn0, max(3, min(steps, 10)), 3, flush, barrier)
        res = {"kind": kind, "kv_bytes": w0.kv_bytes, "total_ms": total_ms, "mode": tmode, "instances": R, "covers_l2": covers_l2,
               "isolated_ms": iso, "launches": launches, "splits": desc, "plan_us": None if plan_ms is None else plan_ms * 1e3}
        if plan is not None:
            # what the scheduler made of the request: pieces of a row that fell to the same pair of SMs run as one item
            items, slots, over, _ = plan.info()
            res["plan"] = {"rows_x_head_groups": B * s_q * ((H + 127) // 128), "items": items, "partial_slots": slots}
        if with_e2e:
            et, h2d, d2h, copies = e2e_steps(kind, insts, steps, warmup, flush, barrier)
            res.update(e2e_total_ms=et, h2d=h2d, d2h=d2h, copies=copies)
        # the result of the last timed call on the first instance, against the oracle (not timed)
        o, l = fn0()
        torch.cuda.synchronize()
        res["parity"] = parity_sample(kind, w0, o, l)
        for _, _, status in insts:
            st = status.cpu().tolist()
            if st != [0, 0, 0, 0]:
                raise RuntimeError(f"{name}: the decode kernel reported status={st}")
        del insts, w, w0
        torch.cuda.empty_cache()
        return res

    def reduce_max(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def reduce_sum(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    sampler = ClockSampler(int(os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[local]) if os.environ.get("CUDA_VISIBLE_DEVICES") else local)
    if rank == 0:
        sampler.start()
    head = measure(args.workload, args.steps, args.warmup, with_e2e=True)
    clocks = sampler.stop() if rank == 0 else None

    total_ms = reduce_max(head["total_ms"])
    fastest_rank_ms = -reduce_max(-head["total_ms"]) / args.steps
    total_bytes = reduce_sum(head["kv_bytes"])
    ms_per_step = total_ms / args.steps
    value = total_bytes / (ms_per_step * 1e-3) / 1e12
    isolated_ms = reduce_max(statistics.mean(head["isolated_ms"]))
    e2e_ms = reduce_max(head["e2e_total_ms"]) / args.steps
    e2e_value = total_bytes / (e2e_ms * 1e-3) / 1e12
    # the host link per rank (slowest and fastest rank), measured with all ranks copying at once
    link = {}
    for key, val in head["copies"].items():
        link[key] = {"min_over_ranks": -reduce_max(-val), "max_over_ranks": reduce_max(val)} if world > 1 else val
    link["compute_ms_per_step"] = ms_per_step
    link["host_binding_rank0"] = binding
    peak, peak_src = measured_peak_gbs()
    per_gpu_gbs = head["kv_bytes"] / (head["total_ms"] / args.steps * 1e-3) / 1e9

    others = {}
    if "mixed" in args.extras:
        (csa_w, hca_w), n_mine = build_mixed(rank, world, dev)
        msteps = max(3, min(args.steps, 10))
        mixed = {}
        # the same two layers on the static grid (split count from the host rule) and on plans of the scheduler
        for label, mode in (("static_grid", {"num_splits": None}), ("scheduled", {"plan_splits": 0})):
            fc, lc, sc, st_c, pc = make_step("csa", csa_w, dict(mode))
            fh, lh, sh, st_h, ph = make_step("hca", hca_w, dict(mode))

            def both(fc=fc, fh=fh):
                fc()
                fh()
            # one instance: each layer streams far more than L2 holds
            tot, mixed_mode = time_rotating([both], msteps, 3, flush, barrier, flush_first=False)
            ms = reduce_max(tot) / msteps
            oc, lc_ = fc()
            oh, lh_ = fh()
            torch.cuda.synchronize()
            par = {"csa": parity_sample("csa", csa_w, oc, lc_), "hca": parity_sample("hca", hca_w, oh, lh_)}
            if st_c.cpu().tolist() != [0, 0, 0, 0] or st_h.cpu().tolist() != [0, 0, 0, 0]:
                raise RuntimeError("mixed workload: the decode kernel reported a status")
            plan_us = None
            if pc is not None:
                plan_us = reduce_max(statistics.mean(time_steps(lambda: (pc.remake(), ph.remake()), 5, 3, flush, barrier))) * 1e3
            mixed[label] = {"ms_per_step": ms, "split_mode": {"csa": sc, "hca": sh}, "timing": mixed_mode, "parity": par,
                            "plan_us_both_layers": plan_us}
            del fc, fh, pc, ph
        mixed_bytes = reduce_sum(csa_w.kv_bytes + hca_w.kv_bytes)
        best = min(mixed, key=lambda k: mixed[k]["ms_per_step"])
        mixed_ms = mixed[best]["ms_per_step"]
        others[MIXED] = {"tokens_per_s": MIXED_REQUESTS / (mixed_ms * 1e-3), "ms_per_step": mixed_ms,
                         "us_per_layer": mixed_ms * 1e3 / 2, "kv_tb_per_s": mixed_bytes / (mixed_ms * 1e-3) / 1e12,
                         "kv_bytes": mixed_bytes, "requests_per_gpu": n_mine, "layers_per_step": 2,
                         "scaling": "strong", "path": best, "paths": mixed,
                         "scheduled_over_static": mixed["static_grid"]["ms_per_step"] / mixed["scheduled"]["ms_per_step"],
                         "sharding": "sorted by context, dealt round-robin",
                         "note": "plans are made once per step, outside the layers; their cost is plan_us_both_layers"}
        del csa_w, hca_w
        torch.cuda.empty_cache()
    if "head_sharded" in args.extras and world > 1 and 128 % world == 0:
        # Optional variant, for comparison only: every rank holds the WHOLE headline batch (same seed) and
        # computes 128 / world heads of every request; one NCCL all-gather of out (+ lse) over NVLink.
        # The KV bytes counted are those of one copy of the batch; every rank streams all of them.
        import dsv4_attn_b200 as lib
        from dsv4_attn_b200 import dp
        kind_h, wh, _ = build_workload(args.workload, seed=777, device=dev)
        if kind_h == "hca":
            Bh, sq_h, Hh, _ = wh.q.shape
            h0, h1 = dp.head_shard(Hh, world, rank)
            out_l = torch.empty(Bh, sq_h, h1 - h0, 512, dtype=torch.bfloat16, device=dev)
            lse_l = torch.empty(Bh, sq_h, h1 - h0, dtype=torch.float32, device=dev)

            def dec(qs, sink):
                return lib.hca_dense_decode(qs, wh.kv_pool, wh.block_table, wh.kv_len, wh.win_pool, wh.win_len, wh.sm_scale,
                                            attn_sink=sink, num_splits=1, out=out_l, lse=lse_l, max_len=wh.max_len)
            hs = time_steps(lambda: dp.head_sharded_decode(dec, wh.q, wh.attn_sink), max(3, min(args.steps, 10)), 3, flush, barrier)
            hs_ms = reduce_max(statistics.mean(hs))
            others["head_sharded_" + args.workload] = {
                "us_per_layer": hs_ms * 1e3, "kv_tb_per_s": wh.kv_bytes / (hs_ms * 1e-3) / 1e12, "kv_bytes_one_copy": wh.kv_bytes,
                "kv_bytes_read_all_ranks": wh.kv_bytes * world, "heads_per_rank": h1 - h0, "collective": "all_gather(out) + all_gather(lse), NCCL",
                "scaling": "strong", "timing": "isolated (L2 flushed, eager)"}
        del wh
        torch.cuda.empty_cache()
    if world == 1:
        groups = {"cache_write": ("csa_compress_reduce_b1_n65536_c512", "hca_compress_insert_b1_n65536_c576_m128",
                                  "kv_quantize_insert_65536rows", "rope_norm_65536x16x576", "combine_fp32_partials_8x256rows"),
                  "indexer": ("indexer_topk_b64_n25000_k2048",)}
        for group, names in groups.items():
            if group not in args.extras:
                continue
            for name in names:
                fn, nbytes, extra, check = aux_case(name, dev)
                t = statistics.mean(time_steps(fn, max(3, min(args.steps, 10)), 3, flush, barrier))
                check()
                key = "key_" if name.startswith("indexer") else ""
                others[name] = {"us": t * 1e3, key + "gb_per_s": nbytes / (t * 1e-3) / 1e9, "hbm_frac": nbytes / (t * 1e-3) / 1e9 / peak,
                                key + "bytes": nbytes, **extra}
                del fn, check
                torch.cuda.empty_cache()
    if "decode" in args.extras and world == 1:
        # the reference's own entry point and cache layout (448 e4m3 + 7 UE8M0 + 64 bf16 per token), at the
        # shape the reference harness runs it: B=64, 128 heads, 768 compressed + 128 window tokens
        import dsv4_attn_b200 as lib
        Br, Mr, Wr = 64, 768, 128
        Qr = (0.5 * torch.randn(Br, 128, 512, device=dev)).to(torch.bfloat16)
        mk = lambda n: (torch.randint(0, 120, (Br, n, 448), dtype=torch.uint8, device=dev) |
                        (torch.randint(0, 2, (Br, n, 448), dtype=torch.uint8, device=dev) << 7))
        Kc, Ks = mk(Mr), mk(Wr)
        Kc_s = torch.full((Br, Mr, 7), 119, dtype=torch.uint8, device=dev)          # 2^-8
        Ks_s = torch.full((Br, Wr, 7), 119, dtype=torch.uint8, device=dev)
        Kc_r = (0.5 * torch.randn(Br, Mr, 64, device=dev)).to(torch.bfloat16)
        Ks_r = (0.5 * torch.randn(Br, Wr, 64, device=dev)).to(torch.bfloat16)
        sink_r = 0.1 * torch.randn(128, device=dev)
        Or = torch.empty(Br, 128, 512, dtype=torch.bfloat16, device=dev)
        Sr = (Mr + Wr) // 128
        pOr = torch.empty(Sr, Br, 128, 512, dtype=torch.float32, device=dev)
        plr = torch.empty(Sr, Br, 128, dtype=torch.float32, device=dev)
        rt = time_steps(lambda: lib.hca_decode_fwd(Qr, Kc, Kc_s, Kc_r, Ks, Ks_s, Ks_r, sink_r, 512 ** -0.5, M_cur=Mr, swa_len=Wr,
                                                   O=Or, partial_O=pOr, partial_lse=plr), max(3, min(args.steps, 10)), 3, flush, barrier)
        rbytes = Br * (Mr + Wr) * 583
        rms = statistics.mean(rt)
        others["hca_decode_fwd_reference_layout_b64_m768_w128"] = {
            "isolated_us": rms * 1e3, "kv_tb_per_s": rbytes / (rms * 1e-3) / 1e12, "hbm_frac": rbytes / (rms * 1e-3) / 1e9 / peak,
            "kv_bytes": rbytes, "timing": "isolated (L2 flushed, eager)"}
        del Kc, Ks, pOr
        torch.cuda.empty_cache()
        for name in WORKLOADS:
            if name == args.workload:
                continue
            osteps = max(3, min(args.steps, 10))
            r = measure(name, osteps, 3, with_e2e=False)
            ms = r["total_ms"] / osteps
            others[name] = {"us_per_layer": ms * 1e3, "kv_tb_per_s": r["kv_bytes"] / (ms * 1e-3) / 1e12,
                            "hbm_frac": r["kv_bytes"] / (ms * 1e-3) / 1e9 / peak, "kv_bytes": r["kv_bytes"],
                            "split_mode": r["splits"], "plan_us": r["plan_us"], "plan": r.get("plan"), "isolated_us": statistics.mean(r["isolated_ms"]) * 1e3,
                            "timing": r["mode"], "instances": r["instances"], "parity": r["parity"],
                            "traffic": NCU_DRAM_TRAFFIC.get(name)}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    kind, kw = WORKLOADS[args.workload]
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "us_per_layer": ms_per_step * 1e3, "us_per_layer_fastest_rank": fastest_rank_ms * 1e3,
        "isolated_us_per_layer": isolated_ms * 1e3,
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": "fp16 tensor-core operands (fp8-e4m3 KV dequantised with its fp32 scales, bf16 q and the probabilities converted), fp32 accumulate, bf16 out",
        "data": "synthetic",
        "config": {"workload": args.workload, **{k: v for k, v in kw.items()}, "requests_per_gpu": kw["B"],
                   "split_mode": head["splits"], "entry_bytes": ENTRY_BYTES,
                   "timing": f"{head['mode']} replay of the K steps" if head["mode"] == "graph" else "eager back-to-back launches",
                   "l2": f"inputs larger than L2: the steps rotate over {head['instances']} independent instances of the workload "
                         f"({head['instances']} KV pools, queries and outputs, together more than 3 x L2 = {l2_bytes >> 20} MiB); the timed replay "
                         f"of the captured steps follows an untimed replay and one untimed pass over the instances in rotation "
                         f"order, so that every instance was last used before all the others; the isolated figure empties L2 "
                         f"with a {L2_FLUSH_BYTES >> 20} MiB write followed by a read of the same buffer before each launch",
                   "kv_bytes_per_gpu_step": head["kv_bytes"], "parallelism": f"dp{world} over requests, no collective"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": head["h2d"], "d2h_bytes_per_step": head["d2h"],
                "ms_per_step": e2e_ms, "host_link": link,
                "note": "every step copies q and its length/index tensors from one pinned host buffer (one copy) and reads out+lse back to pinned host memory (one copy); copy-in, compute and copy-out run on their own streams chained by events, K steps timed as a whole; the KV cache is device-resident state; host_link is the same buffers copied with no compute, all ranks at once"},
        "gpu_launches": head["launches"] * args.steps,
        "roofline": {"bound": "hbm", "achieved": per_gpu_gbs, "peak": peak, "unit": "GB/s", "frac": per_gpu_gbs / peak,
                     "traffic": NCU_DRAM_TRAFFIC.get(args.workload), "traffic_source": NCU_TRAFFIC_SOURCE if args.workload in NCU_DRAM_TRAFFIC else None,
                     "algorithmic_bytes": head["kv_bytes"], "peak_source": peak_src, "kernel": "decode_mma_kernel" + ("+combine_kernel" if head["launches"] > 1 else "")},
        # the same launch against the tensor-core bound: 2 x H x (576 + 512) FLOP per attended entry
        "roofline_tensor": tensor_view(head["kv_bytes"], kw["H"], head["total_ms"] / args.steps),
        "clocks": clocks,
        "parity": {**head["parity"], "tolerance": TOL, "against": "CPU oracle, rows of the first instance after the timed region"},
        "other_workloads": others,
    }
    if world == 1:
        line["cpu_baseline"] = cpu_baseline(kind, args.workload)
        line["e2e_vs_cpu_baseline"] = e2e_value / line["cpu_baseline"]["value"]
    print(json.dumps(line), file=args.out, flush=True)
    if world > 1:
        dist.destroy_process_group()


# ───────────────────────── reference arm ─────────────────────────

def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    claim_host_threads()
    kind, kw = WORKLOADS[args.workload]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    vals, base = [], None
    for i in range(args.warmup + args.steps):
        base = cpu_baseline(kind, args.workload, target_s=1.5, sample_B=8)
        if i >= args.warmup:
            vals.append(base)
    v = statistics.mean(b["value"] for b in vals)
    ms = statistics.mean(b["ms_per_full_step"] for b in vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32 (torch CPU)" if base["kind"] == "reference" else "fp32 (numpy)", "data": "synthetic",
        "config": {"workload": args.workload, **kw},
        "cpu_baseline": {**base, "value": v},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's own PyTorch decode path on the host cores, each step a bounded sample of the workload "
                "(ms_per_step is the sample's time scaled to the whole batch); the reference's CUDA decode kernel is not "
                "run: as committed it stalls on an mbarrier and then traps",
    }
    print(json.dumps(line), file=args.out, flush=True)


def _claim_stdout():
    """Keep stdout for the one JSON line: libraries (NCCL's version banner, for
    one) write to file descriptor 1, so send that to stderr for the duration of
    the run and return a handle on the real stdout."""
    sys.stdout.flush()
    real = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    return real


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=list(WORKLOADS))
    ap.add_argument("--no-extras", action="store_true", help="skip the other workloads")
    ap.add_argument("--single", default=None, choices=list(WORKLOADS) + list(PROFILE_CASES) + list(AUX_CASES),
                    help="run one instance of one case a few times and exit (for profiler captures); prints a short line of its own")
    ap.add_argument("--extras", default="mixed,head_sharded,cache_write,indexer,decode",
                    help="which groups of other workloads to run: mixed, head_sharded (N > 1), cache_write, indexer, decode (comma-separated)")
    args = ap.parse_args()
    args.extras = set() if args.no_extras else {x for x in args.extras.split(",") if x}
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    args.out = _claim_stdout()
    if args.single:
        run_single(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
