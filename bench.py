#!/usr/bin/env python3
"""Benchmark of the quantised-matvec / routed-expert hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (N = 1): the decode matvec of the Q4_K [12288 x 4096] projection, batch 1,
over a rotating set of distinct weight copies larger than L2, so every pass reads HBM. One
"step" is one pass over the whole set. `value` is packed-weight-plus-activation bytes per
second with everything resident in HBM; `e2e` is the same metric through the host-buffer
entry point (activations copied in from pinned memory, outputs copied back, every call).
The same line also carries the other formats / batch sizes and the routed-expert layer
(tokens/s) as explanatory detail, the roofline of the dominant kernel, and the reference's
CPU path (the oracle port) timed on this host's cores as a baseline.

With --gpus N > 1 (launched under torchrun, one rank per GPU) each rank runs an independent
replica of the matvec workload on its own GPU (weak scaling, no data-path collective); the
routed layer runs expert-parallel with experts split N ways.

`--impl reference` times the reference's CPU implementation of the same workload (oracle
port, the reference's own threading rule) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED = 20260907
ROWS, COLS = 12288, 4096           # the large dense projection of the decode configuration
HEAD_KIND = 12                     # Q4_K
KIND_NAME = {8: "Q8_0", 12: "Q4_K", 14: "Q6_K"}
L2_BYTES = 126 * 1024 * 1024
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the headline kernel, from the ncu
# capture summarised in profiles/matvec_decode_i8_q4k_12288x4096_b1.md (same workload, same sizes).
HEAD_TRAFFIC_BYTES = 28_345_088
MOE = dict(n_experts=128, dim=2048, ff=768, top_k=8)


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def algorithmic_bytes(kind, rows, cols, batch):
    from exec_beholdd_b200 import synth

    return synth.packed_bytes(kind, rows, cols) + 4 * batch * (rows + cols)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        for s in self.samples:
            parts = [p.strip() for p in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------
# CPU arm: the reference's CPU path (oracle port) on the host cores
# ------------------------------------------------------------------------------------------

def cpu_matvec_baseline(budget_s=12.0, kind=HEAD_KIND):
    """Best-of-N wall time of one [ROWS x COLS] matvec through the oracle with the reference's
    threading rule, like the reference's own bench (examples/bench_q8_matvec.rs:69-79)."""
    import oracle
    from exec_beholdd_b200 import synth

    orc = oracle.load()
    packed = synth.matrix(kind, SEED, ROWS, COLS)
    x = synth.activations(SEED + 1, (COLS,))
    threads = orc.worker_count(ROWS, COLS, orc.available_parallelism())
    best, n, t_end = float("inf"), 0, time.perf_counter() + budget_s
    while n < 3 or (time.perf_counter() < t_end and n < 200):
        t0 = time.perf_counter()
        orc.matvec(packed, kind, ROWS, COLS, x)
        best = min(best, time.perf_counter() - t0)
        n += 1
    gbs = algorithmic_bytes(kind, ROWS, COLS, 1) / best / 1e9
    return {"value": gbs, "unit": "GB/s", "cores": int(threads), "kind": "port",
            "sample": f"best of {n} calls of one {KIND_NAME[kind]} {ROWS}x{COLS} batch-1 matvec ({best * 1e3:.1f} ms), "
                      f"oracle port with the reference threading rule (<= 8 row-chunk threads), "
                      f"{orc.available_parallelism()} logical CPUs visible"}


def cpu_moe_baseline(T=16, budget_s=10.0):
    import oracle
    from exec_beholdd_b200 import synth

    orc = oracle.load()
    m = MOE
    router = synth.router_weights(SEED, m["n_experts"], m["dim"])
    gate = synth.expert_slabs(SEED, m["n_experts"], m["ff"], m["dim"], 21)
    up = synth.expert_slabs(SEED, m["n_experts"], m["ff"], m["dim"], 22)
    down = synth.expert_slabs(SEED, m["n_experts"], m["dim"], m["ff"], 23)
    x = synth.activations(SEED + 2, (T, m["dim"]))
    best, n, t_end = float("inf"), 0, time.perf_counter() + budget_s
    while n < 2 or (time.perf_counter() < t_end and n < 50):
        t0 = time.perf_counter()
        orc.moe_layer(router, gate, up, down, m["ff"], x, m["top_k"])
        best = min(best, time.perf_counter() - t0)
        n += 1
    return {"tokens_per_s": T / best, "T": T, "ms": best * 1e3, "calls": n}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    per_step = []
    base = None
    for i in range(args.warmup + args.steps):
        base = cpu_matvec_baseline(budget_s=1.5)
        if i >= args.warmup:
            per_step.append(base["value"])
    value = max(per_step)
    line = {
        "impl": "reference", "metric": "q_matvec_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": algorithmic_bytes(HEAD_KIND, ROWS, COLS, 1) / value / 1e6, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{KIND_NAME[HEAD_KIND]} decode matvec {ROWS}x{COLS} batch 1 (CPU path of the reference, oracle port)"},
        "cpu_baseline": dict(base, value=value),
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------

def time_region(torch, fn, steps, warmup, barrier=None, graph=True):
    """W untimed steps, then K steps bracketed by synchronise (+ barrier) on both sides, timed
    with CUDA events on the launching stream. The step is captured once into a CUDA graph and
    replayed, so the host's per-call cost does not pace a launch-bound sequence of kernels."""
    fn()  # first call sizes the workspace and sets kernel attributes (not capturable)
    torch.cuda.synchronize()
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        fn = g.replay
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return start.elapsed_time(stop) / 1e3  # seconds


def build_rotating_set(dev, torch, kind, rows, cols, copies):
    from exec_beholdd_b200 import synth

    ws = []
    for i in range(copies):
        packed = torch.from_numpy(synth.matrix(kind, SEED + i, rows, cols)).cuda()
        ws.append(dev.wrap_weight(packed, kind, rows, cols))
    return ws


def bench_matvec(dev, torch, kind, batch, steps, warmup, barrier=None, copies=None):
    from exec_beholdd_b200 import synth

    wbytes = synth.packed_bytes(kind, ROWS, COLS)
    copies = copies or max(4, -(-2 * L2_BYTES // wbytes) + 1)
    ws = build_rotating_set(dev, torch, kind, ROWS, COLS, copies)
    x = torch.from_numpy(synth.activations(SEED + 1, (batch, COLS))).cuda()
    y = torch.empty((batch, ROWS), device="cuda")

    def step():
        for w in ws:
            dev.matvec_resident(w, x, y)

    l0 = dev.launch_count
    step()
    per_step_launches = dev.launch_count - l0   # counted on an eager step; the timed steps replay the same launches
    secs = time_region(torch, step, steps, warmup, barrier)
    launches = per_step_launches * steps
    bytes_per_step = copies * algorithmic_bytes(kind, ROWS, COLS, batch)
    res = {"gbs": bytes_per_step * steps / secs / 1e9, "ms_per_step": secs / steps * 1e3, "copies": copies,
           "us_per_matvec": secs / steps / copies * 1e6, "bytes_per_matvec": algorithmic_bytes(kind, ROWS, COLS, batch),
           "launches_timed": launches, "launches_per_step": per_step_launches}
    dev.check_status()
    for w in ws:
        w.free()
    return res, ws, x


def bench_matvec_e2e(dev, torch, kind, steps, warmup, copies):
    """Same workload through the host-buffer entry point: pinned x in, y out, every call."""
    from exec_beholdd_b200 import synth

    ws = build_rotating_set(dev, torch, kind, ROWS, COLS, copies)
    x = torch.from_numpy(synth.activations(SEED + 1, (1, COLS))).pin_memory()
    y = torch.empty((1, ROWS)).pin_memory()
    xn, yn = x.numpy(), y.numpy()

    def step():
        for w in ws:
            dev.matvec_host_resident(w, xn, yn)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    secs = time.perf_counter() - t0
    for w in ws:
        w.free()
    bytes_per_step = copies * algorithmic_bytes(kind, ROWS, COLS, 1)
    return {"value": bytes_per_step * steps / secs / 1e9, "unit": "GB/s", "h2d_bytes_per_step": copies * 4 * COLS,
            "d2h_bytes_per_step": copies * 4 * ROWS, "us_per_matvec": secs / steps / copies * 1e6}


def bench_prefill(dev, torch, M, N, K, steps, warmup, peak_tflops):
    """Q8_0 prefill matmul Y[M x N] = X[M x K] W^T (tensor-core bound for M >= 512)."""
    from exec_beholdd_b200 import synth

    packed = torch.from_numpy(synth.q8_0_matrix(SEED + 5, N, K)).cuda()
    w = dev.wrap_weight(packed, 8, N, K)
    x = torch.from_numpy(synth.activations(SEED + 6, (M, K), outliers=True)).cuda()
    y = torch.empty((M, N), device="cuda")
    secs = time_region(torch, lambda: dev.matmul_resident(w, x, y), steps, warmup)
    dev.check_status()
    w.free()
    tf = 2.0 * M * N * K * steps / secs / 1e12
    return {"us": round(secs / steps * 1e6, 1), "tflops": round(tf, 1), "frac_of_tensor_peak": round(tf / peak_tflops, 4)}


def bench_moe(dev, torch, T, steps, warmup, rank=0, world=1, barrier=None):
    """One routed-expert layer at the Qwen3-30B-A3B shapes; experts split `world` ways."""
    from exec_beholdd_b200 import Weight, synth
    from exec_beholdd_b200 import expert_parallel

    m = MOE
    layer = expert_parallel.ExpertParallelLayer.from_synthetic(dev, SEED, m["n_experts"], m["dim"], m["ff"], m["top_k"], rank, world)
    x = torch.from_numpy(synth.activations(SEED + 2, (T, m["dim"]))).cuda()
    y = torch.empty((T, m["dim"]), device="cuda")

    def step():
        layer.forward(x, y)

    secs = time_region(torch, step, steps, warmup, barrier, graph=(world == 1))
    if world > 1:
        import torch.distributed as dist

        t = torch.tensor([secs], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        secs = float(t.item())
    dev.check_status()
    counts = layer.last_counts.cpu().numpy()
    touched = int((counts > 0).sum())
    slab = 3 * synth.packed_bytes(8, m["ff"], m["dim"])
    bytes_touched = m["n_experts"] * m["dim"] * 4 + touched * slab + 8 * T * m["dim"]
    out = {"T_per_gpu": T, "tokens_per_s": world * T * steps / secs, "ms_per_layer": secs / steps * 1e3,
           "exchange": layer.exchange if world > 1 else "none", "experts_touched": touched,
           "gbs_of_touched_bytes": bytes_touched * steps / secs / 1e9,
           "tflops": world * T * m["top_k"] * 3 * 2 * m["ff"] * m["dim"] * steps / secs / 1e12}
    layer.free()
    return out


def bench_row_split(dev, torch, kind, batch, steps, warmup, rank, world, barrier):
    """One [ROWS x COLS] projection with its rows split over the ranks, all-gather included.
    Eager launches (the collective is not captured), device-timed, max over ranks."""
    import torch.distributed as dist
    from exec_beholdd_b200 import synth
    from exec_beholdd_b200.row_parallel import RowSplitLinear

    copies = 4  # distinct shards per step so that the weights come from HBM, not L2
    lins = [RowSplitLinear.from_host(dev, synth.matrix(kind, SEED + i, ROWS, COLS), kind, ROWS, COLS, rank, world) for i in range(copies)]
    x = torch.from_numpy(synth.activations(SEED + 1, (batch, COLS))).cuda()
    y = torch.empty((batch, ROWS), device="cuda")

    def step():
        for lin in lins:
            lin.forward(x, y)

    secs = time_region(torch, step, steps, warmup, barrier, graph=False)
    t = torch.tensor([secs], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    secs = float(t.item())
    dev.check_status()
    for lin in lins:
        lin.free()
    us = secs / steps / copies * 1e6
    return {"us_per_matvec": round(us, 2), "gbs_whole_weight": round(algorithmic_bytes(kind, ROWS, COLS, batch) / us / 1e3, 1),
            "rows_per_gpu": ROWS // world, "collective": "all_gather of y", "launch": "eager"}


def run_gpu_arm(args):
    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local)
    barrier = None
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
        barrier = dist.barrier

    from exec_beholdd_b200 import CudaDevice, build, synth

    build.build()
    dev = CudaDevice(local)
    peak, peak_kind = measured_peak_gbs()
    steps, warmup = args.steps, max(args.warmup, 3)

    with ClockSampler(local) as clocks:
        head, _, _ = bench_matvec(dev, torch, HEAD_KIND, 1, steps, warmup, barrier)
    secs_local = head["ms_per_step"] / 1e3 * steps
    if world > 1:
        t = torch.tensor([secs_local], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        secs = float(t.item())
    else:
        secs = secs_local
    bytes_per_step = head["copies"] * head["bytes_per_matvec"]
    value = world * bytes_per_step * steps / secs / 1e9

    sections = set(v for v in args.sections.split(",") if v)
    detail = {}
    if not args.quick and not args.skip_matvec_detail and "detail" in sections:
        for kind in (8, 12, 14):
            for batch in (1, 2, 4, 8):
                if kind == HEAD_KIND and batch == 1:
                    continue
                r, _, _ = bench_matvec(dev, torch, kind, batch, max(2, steps // 4), 3, barrier)
                detail[f"{KIND_NAME[kind]}_b{batch}"] = {"gbs": round(r["gbs"], 1), "us": round(r["us_per_matvec"], 2),
                                                        "frac_of_peak": round(r["gbs"] / peak, 4)}
    prefill = {}
    if not args.quick and "prefill" in sections and world == 1:
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
                tpeak = float(json.load(fh)["bf16_tflops_sustained"])
        except Exception:
            tpeak = 1400.0
        shapes = [tuple(int(d) for d in v.split("x")) for v in args.prefill_shapes.split(",") if v]
        for (M, N) in shapes:
            try:
                prefill[f"M{M}_N{N}"] = bench_prefill(dev, torch, M, N, 4096, max(2, steps // 4), 3, tpeak)
            except Exception as e:
                prefill[f"M{M}_N{N}"] = {"error": repr(e)}
    moe = {}
    try:
        for T in (() if (args.quick or "moe" not in sections) else tuple(int(v) for v in args.moe_tokens.split(",") if v)):
            moe[f"T{T}"] = bench_moe(dev, torch, T, max(2, steps // 4), 3, rank, world, barrier)
    except Exception as e:  # the headline number must still be reported
        moe["error"] = repr(e)

    row_split = None
    if world > 1 and not args.quick and ROWS % world == 0:
        try:
            row_split = {f"b{b}": bench_row_split(dev, torch, HEAD_KIND, b, max(2, steps // 4), 3, rank, world, barrier) for b in (1, 4)}
        except Exception as e:
            row_split = {"error": repr(e)}

    e2e = bench_matvec_e2e(dev, torch, HEAD_KIND, max(2, steps // 4), 3, head["copies"]) if world == 1 else None
    if world > 1:
        e2e_local = bench_matvec_e2e(dev, torch, HEAD_KIND, max(2, steps // 4), 3, head["copies"])
        t = torch.tensor([e2e_local["value"]], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        e2e = dict(e2e_local, value=float(t.item()))

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_matvec_baseline()
        if not args.quick:
            cpu["moe_layer"] = cpu_moe_baseline()

    if rank == 0:
        launch_us = head["us_per_matvec"]
        achieved = head["bytes_per_matvec"] / (launch_us * 1e-6) / 1e9
        line = {
            "metric": "q_matvec_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": secs / steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{KIND_NAME[HEAD_KIND]} decode matvec {ROWS}x{COLS} batch 1, {head['copies']} distinct "
                                   f"weight copies per step ({head['copies'] * synth.packed_bytes(HEAD_KIND, ROWS, COLS) >> 20} MiB "
                                   f"> 2x L2, so inputs exceed L2 between reuses)",
                       "parallelism": "replicas" if world > 1 else "single"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": HEAD_TRAFFIC_BYTES, "peak_source": peak_kind, "kernel": "k_matvec_decode_i8 (the only kernel of the step)",
                         "us_per_launch": launch_us},
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": head["launches_timed"],
            "clocks": clocks.summary(), "matvec_detail": detail, "prefill_q8_0_k4096": prefill, "moe_layer": moe,
            "row_split_projection": row_split,
        }
        print(json.dumps(line), flush=True)
    dev.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--quick", action="store_true", help="headline workload only")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--moe-tokens", default="1,16,64,512", help="token counts of the routed-layer detail runs")
    ap.add_argument("--skip-matvec-detail", action="store_true", help="skip the other formats / batch sizes")
    ap.add_argument("--sections", default="detail,prefill,moe", help="which detail runs follow the headline workload")
    ap.add_argument("--prefill-shapes", default="128x12288,128x4096,512x12288,512x4096,2048x12288,2048x4096",
                    help="MxN cases of the Q8_0 K=4096 prefill matmul detail run")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
