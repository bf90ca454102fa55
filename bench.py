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
step finds its inputs in HBM, not in L2, without a flush inside the timed region.
The same step timed alone (L2 flushed by a 512 MiB write before each launch, one
event pair per launch, eager launch) is reported beside it as "isolated".
`--impl reference` times the CPU restatement of the reference's PyTorch decode
path (the oracle) on a bounded sample of the same workload on the host cores.
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
    # name: (kind, kwargs)  -- shapes of the benchmark configurations
    "hca_b64_h128_ctx100k": ("hca", dict(B=64, s_q=1, H=128, kv_len=782, win_len=128)),
    "csa_b64_h128_topk512_ctx3072": ("csa", dict(B=64, s_q=1, H=128, n_entries=768, topk=512, num_splits=1)),
    "csa_b128_nextn2_topk2048_ctx100k_split8": ("csa", dict(B=128, s_q=2, H=128, n_entries=25000, topk=2048, num_splits=8)),
    # the same shape with the split count left to the library's planner
    "csa_b128_nextn2_topk2048_ctx100k_planned": ("csa", dict(B=128, s_q=2, H=128, n_entries=25000, topk=2048)),
    "csa_b64_h128_topk2048_ctx100k": ("csa", dict(B=64, s_q=1, H=128, n_entries=25000, topk=2048)),
}
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
NCU_DRAM_TRAFFIC = {"hca_b64_h128_ctx100k": 47.79e6, "csa_b64_h128_topk512_ctx3072": 32.38e6}
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
    splits = kw.pop("num_splits", None)
    if kind == "hca":
        w = synth.make_hca(seed, device=device, **kw)
    else:
        w = synth.make_csa(seed, device=device, **kw)
    return kind, w, splits


def build_mixed(rank, world, device):
    from dsv4_attn_b200 import dp, synth
    ctx = synth.lognormal_contexts(MIXED_REQUESTS, seed=0)
    mine = dp.shard_requests(MIXED_REQUESTS, world, rank, cost=ctx, balance="sorted_round_robin")
    return synth.make_mixed(4000 + rank, [ctx[i] for i in mine], device=device), len(mine)


def make_step(kind, w, splits):
    """Returns (fn() -> (out, lse), launches per call, num_splits).  All buffers
    (outputs, split workspace) are allocated once, outside the timed region."""
    import torch
    import dsv4_attn_b200 as lib
    B, s_q, H, _ = w.q.shape
    rows = B * s_q
    if kind == "hca":
        if splits is None:
            splits = lib.plan_splits(rows, H, w.max_len)
    else:
        if splits is None:
            splits = lib.plan_splits(rows, H, w.indices.shape[-1])
    out = torch.empty(B, s_q, H, 512, dtype=torch.bfloat16, device=w.q.device)
    lse = torch.empty(B, s_q, H, dtype=torch.float32, device=w.q.device)
    ws = lib.alloc_workspace(rows, H, splits, w.q.device) if splits > 1 else None
    status = lib.new_status(w.q.device)
    if kind == "hca":
        def fn(q=None, kv_len=None, win_len=None):
            return lib.hca_dense_decode(w.q if q is None else q, w.kv_pool, w.block_table,
                                        w.kv_len if kv_len is None else kv_len, w.win_pool,
                                        w.win_len if win_len is None else win_len, w.sm_scale,
                                        attn_sink=w.attn_sink, num_splits=splits, out=out, lse=lse,
                                        workspace=ws, status=status, max_len=w.max_len)
    else:
        def fn(q=None, indices=None):
            return lib.csa_sparse_decode(w.q if q is None else q, w.kv_pool, w.block_table,
                                         w.indices if indices is None else indices, w.sm_scale, kv_len=w.kv_len,
                                         topk_len=w.topk_len, num_splits=splits, out=out, lse=lse, workspace=ws,
                                         status=status)
    return fn, (2 if splits > 1 else 1), splits, status


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


def time_rotating(fns, steps, warmup, flush, barrier):
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
    flush.zero_()
    barrier()
    torch.cuda.synchronize()
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


def e2e_steps(kind, insts, steps, warmup, flush, barrier):
    """Same metric through the public API with HOST buffers: every step copies its inputs
    (q and the per-step index / length tensors) from pinned host memory, runs the decode,
    and reads the result (out, lse) back to pinned host memory.  The three stages run on
    their own streams (copy-in, compute, copy-out) chained by events, so that the copies of
    neighbouring steps overlap the compute, as a serving engine would run them; step i
    works on instance i mod R (its own KV pool, staging and output buffers).  Returns
    (total ms of the K steps, h2d bytes per step, d2h bytes per step)."""
    import torch
    R = len(insts)
    dev = insts[0][0].q.device
    # One copy-in stream: back-to-back uploads on one stream reach the host link's rate (52 GB/s measured
    # for 9.4 MB pieces), and while results are read back at the same time a split upload was slower
    # (270 against 250 us per step; copies alone: 241 against 211 us per step for both directions).
    s_in, s_c, s_out = (torch.cuda.Stream(dev) for _ in range(3))
    main = torch.cuda.current_stream(dev)
    slots = []
    for w, fn, _ in insts:
        hq = w.q.cpu().pin_memory()
        dq = torch.empty_like(w.q)
        if kind == "hca":
            h1, h2 = w.kv_len.cpu().pin_memory(), w.win_len.cpu().pin_memory()
            d1, d2 = torch.empty_like(w.kv_len), torch.empty_like(w.win_len)
        else:
            h1, d1 = w.indices.cpu().pin_memory(), torch.empty_like(w.indices)
            h2 = d2 = None
        out, lse = fn()
        ho = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        hl = torch.empty(lse.shape, dtype=lse.dtype).pin_memory()
        slots.append(dict(fn=fn, hq=hq, dq=dq, h1=h1, d1=d1, h2=h2, d2=d2, ho=ho, hl=hl, ev_in=torch.cuda.Event(),
                          ev_c=None, ev_o=None))
    z = slots[0]
    h2d = z["hq"].numel() * z["hq"].element_size() + z["h1"].numel() * z["h1"].element_size() + \
        (z["h2"].numel() * z["h2"].element_size() if z["h2"] is not None else 0)
    d2h = z["ho"].numel() * z["ho"].element_size() + z["hl"].numel() * z["hl"].element_size()
    torch.cuda.synchronize()

    def run(n):
        for i in range(n):
            k = slots[i % R]
            with torch.cuda.stream(s_in):
                if k["ev_c"] is not None:
                    s_in.wait_event(k["ev_c"])          # this instance's staging buffers are free again
                k["dq"].copy_(k["hq"], non_blocking=True)
                k["d1"].copy_(k["h1"], non_blocking=True)
                if k["h2"] is not None:
                    k["d2"].copy_(k["h2"], non_blocking=True)
                k["ev_in"].record(s_in)
            with torch.cuda.stream(s_c):
                s_c.wait_event(k["ev_in"])
                if k["ev_o"] is not None:
                    s_c.wait_event(k["ev_o"])           # its previous result has been read back
                o, l = k["fn"](k["dq"], k["d1"], k["d2"]) if kind == "hca" else k["fn"](k["dq"], k["d1"])
                k["ev_c"] = torch.cuda.Event()
                k["ev_c"].record(s_c)
            with torch.cuda.stream(s_out):
                s_out.wait_event(k["ev_c"])
                k["ho"].copy_(o, non_blocking=True)
                k["hl"].copy_(l, non_blocking=True)
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
    return e0.elapsed_time(e1), h2d, d2h


def cpu_baseline(kind, name, seed=0, target_s=10.0):
    """The oracle (numpy restatement of the reference's PyTorch decode path)
    timed on the host cores on a bounded sample of the workload's requests."""
    import numpy as np
    from oracle import dsv4_oracle as orc
    _, kw = WORKLOADS[name]
    kw = {k: v for k, v in kw.items() if k != "num_splits"}
    sample_B = 4
    kw["B"] = sample_B
    if kind == "hca":
        c = orc.make_hca_case(seed, **kw)
        run = lambda: orc.hca_dense_decode(c.q, c.pool, c.block_table, c.kv_len, c.win, c.win_len, c.sm_scale)
        entries = int(c.kv_len.sum() + c.win_len.sum())
    else:
        c = orc.make_csa_case(seed, **kw)
        run = lambda: orc.csa_sparse_decode(c.q, c.pool, c.block_table, c.indices, c.sm_scale, kv_len=c.kv_len)
        entries = int((c.indices >= 0).sum())
    run()
    t0 = time.perf_counter()
    iters = 0
    while True:
        run()
        iters += 1
        if time.perf_counter() - t0 > target_s or iters >= 50:
            break
    dt = (time.perf_counter() - t0) / iters
    try:
        import threadpoolctl
        threads = max([p.get("num_threads", 1) for p in threadpoolctl.threadpool_info()] or [1])
    except Exception:
        threads = os.cpu_count() or 1
    return {"value": entries * ENTRY_BYTES / dt / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{sample_B} of {WORKLOADS[name][1]['B']} requests of {name}, {iters} passes, numpy float32 oracle",
            "ms_per_sample_pass": dt * 1e3, "host_cpus": os.cpu_count()}


def run_ours(args):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        barrier = lambda: dist.barrier()
    else:
        barrier = lambda: None
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)

    l2_bytes = int(torch.cuda.get_device_properties(dev).L2_cache_size)

    def measure(name, steps, warmup, with_e2e):
        """R instances of the workload (together > 3x L2); the K steps rotate over them."""
        insts = []
        kind, w, splits = build_workload(name, seed=1000 + rank, device=dev)
        B, s_q, H, _ = w.q.shape
        footprint = w.kv_bytes + w.q.numel() * 2 + B * s_q * H * 512 * 2
        R = max(1, min(12, -(-3 * l2_bytes // footprint)))
        for r in range(R):
            if r > 0:
                kind, w, splits = build_workload(name, seed=1000 + rank + 101 * r, device=dev)
            fn, launches, splits_used, status = make_step(kind, w, splits)
            insts.append((w, fn, status))
        total_ms, mode = time_rotating([f for _, f, _ in insts], steps, warmup, flush, barrier)
        w0, fn0, _ = insts[0]
        iso = time_steps(fn0, max(3, min(steps, 10)), 3, flush, barrier)
        res = {"kind": kind, "kv_bytes": w0.kv_bytes, "total_ms": total_ms, "mode": mode, "instances": R,
               "isolated_ms": iso, "launches": launches, "splits": splits_used}
        if with_e2e:
            et, h2d, d2h = e2e_steps(kind, insts, steps, warmup, flush, barrier)
            res.update(e2e_total_ms=et, h2d=h2d, d2h=d2h)
        for _, _, status in insts:
            st = status.cpu().tolist()
            if st != [0, 0, 0, 0]:
                raise RuntimeError(f"{name}: a kernel wait timed out: status={st}")
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
    total_bytes = reduce_sum(head["kv_bytes"])
    ms_per_step = total_ms / args.steps
    value = total_bytes / (ms_per_step * 1e-3) / 1e12
    isolated_ms = reduce_max(statistics.mean(head["isolated_ms"]))
    e2e_ms = reduce_max(head["e2e_total_ms"]) / args.steps
    e2e_value = total_bytes / (e2e_ms * 1e-3) / 1e12
    peak, peak_src = measured_peak_gbs()
    per_gpu_gbs = head["kv_bytes"] / (head["total_ms"] / args.steps * 1e-3) / 1e9

    others = {}
    if "mixed" in args.extras:
        (csa_w, hca_w), n_mine = build_mixed(rank, world, dev)
        fc, lc, sc, st_c = make_step("csa", csa_w, None)
        fh, lh, sh, st_h = make_step("hca", hca_w, None)

        def both():
            fc()
            fh()
        # one instance: each layer streams far more than L2 holds
        msteps = max(3, min(args.steps, 10))
        mixed_total, mixed_mode = time_rotating([both], msteps, 3, flush, barrier)
        mixed_ms = reduce_max(mixed_total) / msteps
        mixed_bytes = reduce_sum(csa_w.kv_bytes + hca_w.kv_bytes)
        if st_c.cpu().tolist() != [0, 0, 0, 0] or st_h.cpu().tolist() != [0, 0, 0, 0]:
            raise RuntimeError("mixed workload: a kernel wait timed out")
        others[MIXED] = {"tokens_per_s": MIXED_REQUESTS / (mixed_ms * 1e-3), "ms_per_step": mixed_ms,
                         "us_per_layer": mixed_ms * 1e3 / 2, "kv_tb_per_s": mixed_bytes / (mixed_ms * 1e-3) / 1e12,
                         "kv_bytes": mixed_bytes, "requests_per_gpu": n_mine, "layers_per_step": 2,
                         "scaling": "strong", "num_splits": {"csa": sc, "hca": sh}, "timing": mixed_mode,
                         "sharding": "sorted by context, dealt round-robin"}
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
    if "cache_write" in args.extras and world == 1:
        # the cache-write side: CSA compressor second pass (a pure streaming kernel)
        import dsv4_attn_b200 as lib
        Bc, nc, cc = 1, 65536, 512
        streams = [torch.randn(Bc, nc, cc, device=dev).to(torch.bfloat16) for _ in range(4)]
        biases = [torch.randn(4, cc, device=dev).to(torch.bfloat16) for _ in range(2)]
        cout = torch.empty(Bc, nc // 4, cc, dtype=torch.bfloat16, device=dev)
        ct = time_steps(lambda: lib.csa_compress_reduce_fwd(*streams, *biases, 4, out=cout), max(3, min(args.steps, 10)), 3,
                        flush, barrier)
        cbytes = 4 * Bc * nc * cc * 2 + cout.numel() * 2
        cms = statistics.mean(ct)
        others["csa_compress_reduce_b1_n65536_c512"] = {"us": cms * 1e3, "gb_per_s": cbytes / (cms * 1e-3) / 1e9,
                                                        "hbm_frac": cbytes / (cms * 1e-3) / 1e9 / peak, "bytes": cbytes}
        del streams, cout
        # the HCA compressor fused with the FP8 quantiser and the paged-cache insert, and the
        # stand-alone quantise-and-insert step
        nh, ch, mh = 65536, 576, 128
        Ch = torch.randn(1, nh, ch, device=dev).to(torch.bfloat16)
        Zh = (2 * torch.randn(1, nh, ch, device=dev)).to(torch.bfloat16)
        bh = torch.randn(mh, ch, device=dev).to(torch.bfloat16)
        n_new = nh // mh
        pages = (n_new + 63) // 64
        pool_h = torch.zeros(pages, 64, ENTRY_BYTES, dtype=torch.uint8, device=dev)
        bt_h = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
        pos_h = torch.zeros(1, dtype=torch.int32, device=dev)
        ht = time_steps(lambda: lib.hca_compress_fwd(Ch, Zh, bh, mh, kv_pool=pool_h, block_table=bt_h, insert_pos=pos_h,
                                                     want_out=False), max(3, min(args.steps, 10)), 3, flush, barrier)
        hbytes = 2 * nh * ch * 2 + n_new * ENTRY_BYTES
        hms = statistics.mean(ht)
        others["hca_compress_insert_b1_n65536_c576_m128"] = {"us": hms * 1e3, "gb_per_s": hbytes / (hms * 1e-3) / 1e9,
                                                            "hbm_frac": hbytes / (hms * 1e-3) / 1e9 / peak, "bytes": hbytes}
        del Ch, Zh
        Tq = 65536
        rows_q = torch.randn(1, Tq, ch, device=dev).to(torch.bfloat16)
        pages = Tq // 64
        pool_q = torch.zeros(pages, 64, ENTRY_BYTES, dtype=torch.uint8, device=dev)
        bt_q = torch.randperm(pages, device=dev).to(torch.int32).view(1, pages)
        qt = time_steps(lambda: lib.kv_quantize_insert(rows_q, pool_q, bt_q, pos_h), max(3, min(args.steps, 10)), 3, flush, barrier)
        qbytes = Tq * (ch * 2 + ENTRY_BYTES)
        qms = statistics.mean(qt)
        others["kv_quantize_insert_65536rows"] = {"us": qms * 1e3, "gb_per_s": qbytes / (qms * 1e-3) / 1e9,
                                                  "hbm_frac": qbytes / (qms * 1e-3) / 1e9 / peak, "bytes": qbytes}
        # RoPE + RMS norm pre-pass on a prefill-sized batch of query vectors (65536 tokens x 16 heads x 576)
        xr = torch.randn(65536, 16, ch, device=dev).to(torch.bfloat16)
        posr = torch.randint(0, 100000, (65536,), dtype=torch.int32, device=dev)
        wr = torch.ones(ch, dtype=torch.bfloat16, device=dev)
        outr = torch.empty_like(xr)
        rt = time_steps(lambda: lib.rope_norm(xr, posr, norm_weight=wr, out=outr), max(3, min(args.steps, 10)), 3, flush, barrier)
        rbytes = 2 * xr.numel() * 2
        rms_ = statistics.mean(rt)
        others["rope_norm_65536x16x576"] = {"us": rms_ * 1e3, "gb_per_s": rbytes / (rms_ * 1e-3) / 1e9,
                                            "hbm_frac": rbytes / (rms_ * 1e-3) / 1e9 / peak, "bytes": rbytes}
        del xr, outr
        del rows_q, pool_q, pool_h
        torch.cuda.empty_cache()
    if "indexer" in args.extras and world == 1:
        # the step before the sparse decode: FP8 scoring of every visible entry + top-k
        import dsv4_attn_b200 as lib
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
        it = time_steps(lambda: lib.indexer_topk(qf, qw, kp, bti, nv, ki, scores=sc_ws, out=oi, status=st_i),
                        max(3, min(args.steps, 10)), 3, flush, barrier)
        if st_i.cpu().tolist() != [0, 0, 0, 0]:
            raise RuntimeError("indexer: a kernel wait timed out")
        ibytes = Bi * ni * 132
        ims = statistics.mean(it)
        others["indexer_topk_b64_n25000_k2048"] = {"us": ims * 1e3, "key_gb_per_s": ibytes / (ims * 1e-3) / 1e9,
                                                   "hbm_frac": ibytes / (ims * 1e-3) / 1e9 / peak, "key_bytes": ibytes,
                                                   "launches": 2}
        del qf, kp, sc_ws
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
                            "num_splits": r["splits"], "isolated_us": statistics.mean(r["isolated_ms"]) * 1e3,
                            "timing": r["mode"], "instances": r["instances"]}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    kind, kw = WORKLOADS[args.workload]
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "us_per_layer": ms_per_step * 1e3, "isolated_us_per_layer": isolated_ms * 1e3,
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 MMA over fp8-e4m3 KV, fp32 accumulate", "data": "synthetic",
        "config": {"workload": args.workload, **{k: v for k, v in kw.items()}, "requests_per_gpu": kw["B"],
                   "num_splits": head["splits"], "entry_bytes": ENTRY_BYTES,
                   "timing": f"{head['mode']} replay of the K steps" if head["mode"] == "graph" else "eager back-to-back launches",
                   "l2": f"inputs larger than L2: the steps rotate over {head['instances']} independent instances of the workload "
                         f"({head['instances']} KV pools, queries and outputs; L2 = {l2_bytes >> 20} MiB); the isolated figure flushes L2 "
                         f"with a {L2_FLUSH_BYTES >> 20} MiB write before each launch",
                   "kv_bytes_per_gpu_step": head["kv_bytes"], "parallelism": f"dp{world} over requests, no collective"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": head["h2d"], "d2h_bytes_per_step": head["d2h"],
                "ms_per_step": e2e_ms, "note": "every step copies q and its length/index tensors from pinned host memory and reads out+lse back to pinned host memory; copy-in, compute and copy-out run on their own streams chained by events, K steps timed as a whole; the KV cache is device-resident state"},
        "gpu_launches": head["launches"] * args.steps,
        "roofline": {"bound": "hbm", "achieved": per_gpu_gbs, "peak": peak, "unit": "GB/s", "frac": per_gpu_gbs / peak,
                     "traffic": NCU_DRAM_TRAFFIC.get(args.workload), "traffic_source": NCU_TRAFFIC_SOURCE if args.workload in NCU_DRAM_TRAFFIC else None,
                     "algorithmic_bytes": head["kv_bytes"], "peak_source": peak_src, "kernel": "decode_mma_kernel" + ("+combine_kernel" if head["launches"] > 1 else "")},
        # the same launch against the tensor-core bound: 2 x H x (576 + 512) FLOP per attended entry
        "roofline_tensor": tensor_view(head["kv_bytes"], kw["H"], head["total_ms"] / args.steps),
        "clocks": clocks,
        "other_workloads": others,
    }
    if world == 1:
        line["cpu_baseline"] = cpu_baseline(kind, args.workload)
    print(json.dumps(line), file=args.out, flush=True)
    if world > 1:
        dist.destroy_process_group()


# ───────────────────────── reference arm ─────────────────────────

def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    kind, kw = WORKLOADS[args.workload]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    vals, base = [], None
    for i in range(args.warmup + args.steps):
        base = cpu_baseline(kind, args.workload, target_s=1.5)
        if i >= args.warmup:
            vals.append(base)
    v = statistics.mean(b["value"] for b in vals)
    ms = statistics.mean(b["ms_per_sample_pass"] for b in vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32 (numpy)", "data": "synthetic",
        "config": {"workload": args.workload, **kw},
        "cpu_baseline": {**base, "value": v},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement (oracle port) of the reference's PyTorch decode path on a bounded sample; the reference's own CUDA decode kernel is not run: as committed it stalls on an mbarrier and then traps",
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
    ap.add_argument("--extras", default="mixed,head_sharded,cache_write,indexer,decode",
                    help="which groups of other workloads to run: mixed, head_sharded (N > 1), cache_write, indexer, decode (comma-separated)")
    args = ap.parse_args()
    args.extras = set() if args.no_extras else {x for x in args.extras.split(",") if x}
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    args.out = _claim_stdout()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
