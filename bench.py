#!/usr/bin/env python3
"""Benchmark of the quantised-matvec / routed-expert hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (N = 1): the decode matvec of the Q4_K [12288 x 4096] projection, batch 1,
over a rotating set of distinct weight copies larger than L2, so every pass reads HBM. One
"step" is PASSES passes over the whole set (a few thousand matvecs, so that the timed region
is long enough for the clocks to settle). `value` is packed-weight-plus-activation bytes per
second with everything resident in HBM; `e2e` is the same metric through the host-buffer
entry points (activations read from page-locked host memory, outputs written back to it,
every call). The same line also carries the other formats / batch sizes, the Q8_0 prefill
matmul and the routed-expert layer (tokens/s) as explanatory detail, the roofline of the
dominant kernel, and the reference's CPU path (the oracle port) timed on this host's cores as
a baseline.

With --gpus N > 1 (launched under torchrun, one rank per GPU) each rank runs an independent
replica of the matvec workload on its own GPU (weak scaling, no data-path collective); the
routed layer runs expert-parallel with experts split N ways and the large projection with its
rows split N ways, and rank 0 checks both against its own single-GPU result.

`--impl reference` times the reference's CPU implementation of the same workload (oracle
port, the reference's own threading rule) on the host cores.

Failure handling with several ranks: nothing between two collectives is caught. A rank that
fails there prints its traceback and the job ends with a non-zero exit code; a rank never
skips a collective its peers enter. What a leg can report without desynchronising (the device
status word, a parity mismatch) is collected per rank after the leg's last collective and
agreed on by all ranks.
"""
from __future__ import annotations

import argparse
import faulthandler
import json
import os
import statistics
import subprocess
import sys
import threading
import time
import traceback

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED = 20260907
ROWS, COLS = 12288, 4096           # the large dense projection of the decode configuration
HEAD_KIND = 12                     # Q4_K
KIND_NAME = {8: "Q8_0", 12: "Q4_K", 14: "Q6_K"}
L2_BYTES = 126 * 1024 * 1024
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the headline kernel, from an ncu
# capture of one launch of the same workload at the same sizes.
HEAD_TRAFFIC_BYTES = 28_345_088
MOE = dict(n_experts=128, dim=2048, ff=768, top_k=8)
TOL = 2e-3                         # the path's floating-point tolerance
DTYPE = ("f32 in / f32 out; weights as packed (s8 / u4 / u6 quants, f16 block scales), activations as 16-bit "
         "block-floating integers (decode, routed experts) or fp16 (prefill), s32 + f32 accumulation")


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            d = json.load(fh)
        return float(d["hbm_gbs"]), float(d["bf16_tflops_sustained"]), "measured"
    except Exception:
        return 6650.0, 1400.0, "fallback"


def algorithmic_bytes(kind, rows, cols, batch):
    from exec_beholdd_b200 import synth

    return synth.packed_bytes(kind, rows, cols) + 4 * batch * (rows + cols)


def max_rel_err(got, want):
    """max_i |g_i - r_i| / max(|r_i|, rms(r)), the error measure of the parity tests."""
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    want = np.asarray(want, dtype=np.float64).reshape(-1)
    if want.size == 0:
        return 0.0
    rms = np.sqrt((want ** 2).mean())
    return float((np.abs(got - want) / np.maximum(np.abs(want), max(rms, 1e-30))).max())


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

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
            self.samples.append((time.perf_counter(), line.strip()))

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self, t0=None, t1=None):
        """All samples, or those taken between two perf_counter times (one leg)."""
        sm, mx, reasons = [], [], set()
        for (t, s) in list(self.samples):
            if t0 is not None and not (t0 <= t <= t1):
                continue
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


def head_workload_text(copies, passes):
    from exec_beholdd_b200 import synth

    return (f"{KIND_NAME[HEAD_KIND]} decode matvec {ROWS}x{COLS} batch 1; a step is {passes} passes over {copies} "
            f"distinct weight copies ({copies * synth.packed_bytes(HEAD_KIND, ROWS, COLS) >> 20} MiB > 2x L2, so "
            f"inputs exceed L2 between reuses)")


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
    copies = default_copies(HEAD_KIND)
    line = {
        "impl": "reference", "metric": "q_matvec_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": algorithmic_bytes(HEAD_KIND, ROWS, COLS, 1) / value / 1e6, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 (the reference's CPU arithmetic)", "data": "synthetic",
        "config": {"workload": head_workload_text(copies, args.passes), "parallelism": "replicas" if args.gpus > 1 else "single",
                   "sample": "each step is a bounded sample of that workload: matvecs of one weight copy for 1.5 s, best call"},
        "cpu_baseline": dict(base, value=value),
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------

def default_copies(kind):
    from exec_beholdd_b200 import synth

    return max(4, -(-2 * L2_BYTES // synth.packed_bytes(kind, ROWS, COLS)) + 1)


def time_region(torch, fn, steps, warmup, barrier=None, graph=True):
    """W untimed steps, then K steps bracketed by synchronise (+ barrier) on both sides, timed
    with CUDA events on the launching stream. The step is captured once into a CUDA graph and
    replayed, so the host's per-call cost does not pace a launch-bound sequence of kernels."""
    fn()  # first call sizes the workspace and sets kernel attributes (not capturable)
    torch.cuda.synchronize()
    if graph:
        g = torch.cuda.CUDAGraph()
        # thread_local: another thread of this process (a collective library's watchdog) may touch
        # the CUDA API while this thread captures
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
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


def bench_matvec(dev, torch, kind, batch, steps, warmup, passes, barrier=None, copies=None, clocks=None):
    from exec_beholdd_b200 import synth

    copies = copies or default_copies(kind)
    ws = build_rotating_set(dev, torch, kind, ROWS, COLS, copies)
    x = torch.from_numpy(synth.activations(SEED + 1, (batch, COLS))).cuda()
    y = torch.empty((batch, ROWS), device="cuda")

    def one_pass():
        for w in ws:
            dev.matvec_resident(w, x, y)

    def step():
        for _ in range(passes):
            one_pass()

    l0 = dev.launch_count
    one_pass()
    per_step_launches = (dev.launch_count - l0) * passes   # counted on an eager pass; the timed steps replay the same launches
    t_a = time.perf_counter()
    secs = time_region(torch, step, steps, warmup, barrier)
    t_b = time.perf_counter()
    n_matvec = copies * passes
    res = {"gbs": n_matvec * algorithmic_bytes(kind, ROWS, COLS, batch) * steps / secs / 1e9, "ms_per_step": secs / steps * 1e3,
           "copies": copies, "us_per_matvec": secs / steps / n_matvec * 1e6,
           "bytes_per_matvec": algorithmic_bytes(kind, ROWS, COLS, batch), "launches_timed": per_step_launches * steps,
           "launches_per_step": per_step_launches, "timed_ms": secs * 1e3}
    if clocks is not None:
        res["sm_mhz"] = clocks.summary(t_a, t_b)["sm_mhz"]
    dev.check_status()
    for w in ws:
        w.free()
    return res


def bench_matvec_e2e(dev, torch, kind, steps, warmup, copies, passes):
    """Same workload through the host-buffer entry points: x read from page-locked host memory and
    y written back to it, every call. `value`: calls queued with bhd_matvec_host_async and one
    bhd_sync per pass (the host reads y after each pass); `sync_per_call_us`: the blocking form."""
    from exec_beholdd_b200 import synth

    ws = build_rotating_set(dev, torch, kind, ROWS, COLS, copies)
    x = torch.from_numpy(synth.activations(SEED + 1, (1, COLS))).pin_memory()
    ys = [torch.empty((1, ROWS)).pin_memory() for _ in ws]
    xn, yn = x.numpy(), [y.numpy() for y in ys]

    def one_pass():
        for w, y in zip(ws, yn):
            dev.matvec_host_async(w, xn, y)
        dev.sync()
        return float(yn[-1][0, 0])  # the host reads a result

    for _ in range(max(warmup, 3)):
        one_pass()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps * passes):
        one_pass()
    secs = time.perf_counter() - t0
    n = copies * passes * steps
    # the blocking form, a bounded sample
    m, t1 = 0, time.perf_counter()
    while m < 300:
        for w, y in zip(ws, yn):
            dev.matvec_host_resident(w, xn, y)
            m += 1
    blocking_us = (time.perf_counter() - t1) / m * 1e6
    for w in ws:
        w.free()
    return {"value": n * algorithmic_bytes(kind, ROWS, COLS, 1) / secs / 1e9, "unit": "GB/s",
            "h2d_bytes_per_step": copies * passes * 4 * COLS, "d2h_bytes_per_step": copies * passes * 4 * ROWS,
            "us_per_matvec": secs / n * 1e6, "sync_per_call_us": blocking_us,
            "how": "bhd_matvec_host_async per matvec, bhd_sync and a host read of y once per pass over the weight copies"}


def bench_prefill(dev, torch, M, N, K, steps, warmup, peak_tflops, kind=8):
    """Q8_0 (or Q4_K) prefill matmul Y[M x N] = X[M x K] W^T (tensor-core bound for M >= 512)."""
    from exec_beholdd_b200 import synth

    packed = torch.from_numpy(synth.matrix(kind, SEED + 5, N, K)).cuda()
    w = dev.wrap_weight(packed, kind, N, K)
    x = torch.from_numpy(synth.activations(SEED + 6, (M, K), outliers=True)).cuda()
    y = torch.empty((M, N), device="cuda")
    secs = time_region(torch, lambda: dev.matmul_resident(w, x, y), steps, warmup)
    dev.check_status()
    w.free()
    tf = 2.0 * M * N * K * steps / secs / 1e12
    return {"us": round(secs / steps * 1e6, 1), "tflops": round(tf, 1), "frac_of_tensor_peak": round(tf / peak_tflops, 4),
            "timed_ms": round(secs * 1e3, 1)}


def bench_attention(dev, torch, n_query, start, steps, warmup):
    """Causal attention at the full-forward head shapes (32 query heads, 4 kv heads, head_dim 128): `n_query` positions from
    absolute position `start` against a cache of start + n_query positions. The sums are the reference's f64 chains."""
    from exec_beholdd_b200 import synth

    heads, kv, hd, n_pos = 32, 4, 128, start + n_query
    q = torch.from_numpy(synth.activations(SEED + 41, (n_query, heads, hd))).cuda()
    k = torch.from_numpy(synth.activations(SEED + 42, (n_pos, kv, hd))).cuda()
    v = torch.from_numpy(synth.activations(SEED + 43, (n_pos, kv, hd))).cuda()
    out = torch.empty((n_query, heads, hd), device="cuda")
    scale = float(1.0 / np.sqrt(np.float32(hd)))
    secs = time_region(torch, lambda: dev.attention_resident(out, q, k, v, start, n_pos, scale), steps, warmup)
    dev.check_status()
    pairs = sum(start + i + 1 for i in range(n_query)) * heads      # (query, head, visible position) triples
    return {"us": round(secs / steps * 1e6, 1), "f64_fma_per_s": round(2.0 * pairs * hd * steps / secs / 1e9, 1), "unit": "G fused multiply-adds/s",
            "timed_ms": round(secs * 1e3, 1)}


def route_margin(torch, probs, top_k):
    """Smallest gap between the last selected and the first rejected probability over all positions:
    how far the selection is from a tie that a one-ulp difference in expf could flip."""
    p = torch.sort(probs, dim=1, descending=True).values
    return float((p[:, top_k - 1] - p[:, top_k]).min().item())


def bench_moe_single(dev, torch, T, steps, warmup):
    """One routed-expert layer at the Qwen3-30B-A3B shapes on one GPU."""
    from exec_beholdd_b200 import expert_parallel, synth

    m = MOE
    layer = expert_parallel.ExpertParallelLayer.from_synthetic(dev, SEED, m["n_experts"], m["dim"], m["ff"], m["top_k"])
    x = torch.from_numpy(synth.activations(SEED + 2, (T, m["dim"]))).cuda()
    y = torch.empty((T, m["dim"]), device="cuda")
    secs = time_region(torch, lambda: layer.forward(x, y), steps, warmup)
    dev.check_status()
    counts = layer.last_counts.cpu().numpy()
    touched = int((counts > 0).sum())
    slab = 3 * synth.packed_bytes(8, m["ff"], m["dim"])
    bytes_touched = m["n_experts"] * m["dim"] * 4 + touched * slab + 8 * T * m["dim"]
    probs = torch.empty((T, m["n_experts"]), device="cuda")
    e = torch.empty((T, m["top_k"]), dtype=torch.int32, device="cuda")
    w = torch.empty((T, m["top_k"]), device="cuda")
    dev.moe_route(layer.router, x, m["top_k"], e, w, None, None, probs)
    out = {"T_per_gpu": T, "tokens_per_s": T * steps / secs, "ms_per_layer": secs / steps * 1e3, "exchange": "none",
           "experts_touched": touched, "gbs_of_touched_bytes": bytes_touched * steps / secs / 1e9,
           "weight_traffic_floor_us": bytes_touched / measured_peaks()[0] / 1e3,
           "tflops": T * m["top_k"] * 3 * 2 * m["ff"] * m["dim"] * steps / secs / 1e12,
           "min_route_margin": route_margin(torch, probs, m["top_k"]), "timed_ms": secs * 1e3}
    # the layer through host buffers: x copied in, y and the routing copied back, every call
    xh = torch.from_numpy(synth.activations(SEED + 2, (T, m["dim"]))).pin_memory().numpy()
    yh = torch.empty((T, m["dim"])).pin_memory().numpy()
    for _ in range(3):
        dev.moe_layer_host(layer.router, layer.gate, layer.up, layer.down, xh, yh, m["top_k"])
    n, t0 = max(5, steps), time.perf_counter()
    for _ in range(n):
        dev.moe_layer_host(layer.router, layer.gate, layer.up, layer.down, xh, yh, m["top_k"])
    out["e2e_host_buffers"] = {"tokens_per_s": T * n / (time.perf_counter() - t0), "h2d_bytes_per_step": 4 * T * m["dim"],
                               "d2h_bytes_per_step": 4 * T * m["dim"]}
    layer.free()
    return out


def bench_full_forward(dev, torch, dist, rank, world, prompt_len=512, n_new=128):
    """The full-forward configuration: a random-init 48-layer Qwen3-30B-A3B-architecture model in Q8_0, a 512-token
    prefill of uniform random token ids and 128 greedy decode steps with a KV cache; with several ranks every rank
    runs its own sequence and the experts are split over the ranks. Device-timed."""
    from exec_beholdd_b200 import synth
    from exec_beholdd_b200.qwen3moe import Qwen3MoeConfig, Qwen3MoeModel

    cfg = Qwen3MoeConfig()
    t0 = time.perf_counter()
    model = Qwen3MoeModel.random_init(dev, cfg, SEED, rank, world)
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t0
    ids = torch.from_numpy((synth.u64(SEED + 50 + rank, 3, prompt_len) % np.uint64(cfg.vocab)).astype(np.int32)).cuda()
    warm = model.forward(ids, start=0)                    # warm-up: sizes the workspace for the whole prompt, loads the kernels
    model.decode_greedy(warm, 3)                          # captures the decode step's CUDA graph
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    # The prefill is ~1000 launches issued one by one from Python: a busy host stretches it. Three passes (each rewrites
    # the same cache rows), the median reported and all three listed.
    prefill_runs = []
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        logits = model.forward(ids, start=0)
        e1.record()
        torch.cuda.synchronize()
        prefill_runs.append(e0.elapsed_time(e1) / 1e3)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev[0].record()
    out, logits = model.decode_greedy(logits, n_new)      # one graph launch per token
    ev[1].record()
    torch.cuda.synchronize()
    prefill_s, decode_s = statistics.median(prefill_runs), ev[0].elapsed_time(ev[1]) / 1e3
    status_error = None
    try:
        dev.check_status()
    except Exception as e:
        status_error = repr(e)
    finite = bool(torch.isfinite(logits).all())
    if world > 1:
        prefill_s, decode_s = max_over_ranks(torch, dist, prefill_s), max_over_ranks(torch, dist, decode_s)
    res = {"model": "Qwen3-30B-A3B architecture, random init, Q8_0 (separate Q8_0 LM head, f32 embeddings)", "layers": cfg.n_layers,
           "prefill_tokens_per_gpu": prompt_len, "decode_steps": n_new, "prefill_ms": prefill_s * 1e3,
           "prefill_ms_runs": [round(v * 1e3, 2) for v in prefill_runs],
           "prefill_tokens_per_s": world * prompt_len / prefill_s, "decode_ms_per_token": decode_s / (n_new - 1) * 1e3,
           "decode_tokens_per_s": world * (n_new - 1) / decode_s, "weights_generated_in_s": build_s, "logits_finite": finite,
           "generated_ids_head": out[:8].cpu().tolist(),
           "launch": "prefill: eager launches; decode: one CUDA graph launch per token (captured during warm-up)"}
    if status_error:
        res["status_error"] = status_error
    if world > 1:
        res["failed_on_some_rank"] = agree(torch, dist, status_error is not None or not finite)
    model.free()
    return res


# ---- several ranks ---------------------------------------------------------------------------

def agree(torch, dist, flag: bool) -> bool:
    """True on every rank if `flag` is set on any rank (called after a leg's last collective)."""
    t = torch.tensor([1 if flag else 0], device="cuda", dtype=torch.int32)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return bool(t.item())


def max_over_ranks(torch, dist, secs):
    t = torch.tensor([secs], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def bench_moe_parallel(dev, torch, dist, T, steps, warmup, rank, world, barrier, exchanges, single):
    """The routed layer with experts split over the ranks. Every rank owns T positions of its own
    (seeded per rank); rank 0 also holds all experts (`single`) and checks its slice of the
    result against the single-GPU layer run on the gathered global batch. Nothing in here is
    caught: see the module docstring."""
    from exec_beholdd_b200 import expert_parallel, synth

    m = MOE
    x = torch.from_numpy(synth.activations(SEED + 2 + 1000 * rank, (T, m["dim"]))).cuda()
    y = torch.empty((T, m["dim"]), device="cuda")
    x_all = torch.empty((world * T, m["dim"]), device="cuda")
    dist.all_gather_into_tensor(x_all, x)
    want = None
    n1 = None
    if rank == 0:
        y_all = torch.empty((world * T, m["dim"]), device="cuda")
        single.forward(x_all, y_all)
        want = y_all[:T].clone()
        # the same positions per GPU on one GPU: the denominator of the scaling efficiency
        y1 = torch.empty((T, m["dim"]), device="cuda")
        n1_secs = time_region(torch, lambda: single.forward(x, y1), steps, warmup)
        n1 = {"ms_per_layer": n1_secs / steps * 1e3, "tokens_per_s": T * steps / n1_secs}
    out = {"T_per_gpu": T}
    for exchange in exchanges:
        layer = expert_parallel.ExpertParallelLayer.from_synthetic(dev, SEED, m["n_experts"], m["dim"], m["ff"], m["top_k"], rank,
                                                                   world, exchange=exchange)
        secs = max_over_ranks(torch, dist, time_region(torch, lambda: layer.forward(x, y), steps, warmup, barrier,
                                                       graph=layer.capturable))
        phases = layer.timed_phases(x, y) if hasattr(layer, "timed_phases") else None
        y.fill_(float("nan"))
        layer.forward(x, y)
        torch.cuda.synchronize()
        status_error = None
        try:
            dev.check_status()
        except Exception as e:  # after the leg's last collective: reported, then agreed on below
            status_error = repr(e)
        entry = {"tokens_per_s": world * T * steps / secs, "ms_per_layer": secs / steps * 1e3,
                 "launch": "cuda graph" if layer.capturable else "eager",
                 "tflops": world * T * m["top_k"] * 3 * 2 * m["ff"] * m["dim"] * steps / secs / 1e12}
        if phases:
            entry["phase_us"] = phases
        if rank == 0:
            err = max_rel_err(y.cpu().numpy(), want.cpu().numpy())
            same = bool(torch.equal(y, want))
            need_bits = layer.bit_identical
            entry["parity"] = {"against": f"rank 0's single-GPU layer over the gathered batch of {world * T} positions",
                               "max_rel_err": err, "bit_identical": same, "bit_identity_required": need_bits,
                               "ok": bool(err <= TOL and (same or not need_bits))}
            entry["n1_same_run"] = n1
            entry["eff_vs_n1"] = entry["tokens_per_s"] / (world * n1["tokens_per_s"])
            bad = not entry["parity"]["ok"]
        else:
            bad = False
        if status_error:
            entry["status_error"] = status_error
        entry["failed_on_some_rank"] = agree(torch, dist, bad or status_error is not None)
        out[exchange] = entry
        layer.free()
    return out


def bench_row_split(dev, torch, dist, kind, batch, steps, warmup, rank, world, barrier):
    """One [ROWS x COLS] projection with its rows split over the ranks, the exchange of y included;
    device-timed, max over ranks. Rank 0 checks the assembled y against the whole weight on one GPU."""
    from exec_beholdd_b200 import Weight, synth
    from exec_beholdd_b200.row_parallel import RowSplitLinear

    copies = 4  # distinct shards per step so that the weights come from HBM, not L2
    hosts = [synth.matrix(kind, SEED + i, ROWS, COLS) for i in range(copies)]
    x = torch.from_numpy(synth.activations(SEED + 1, (batch, COLS))).cuda()
    y = torch.empty((batch, ROWS), device="cuda")
    y1 = n1_us = whole = None
    if rank == 0:
        whole = dev.upload_weight(Weight(hosts[-1], kind, ROWS, COLS))
        y1 = torch.empty((batch, ROWS), device="cuda")
        n1_secs = time_region(torch, lambda: dev.matvec_resident(whole, x, y1), max(steps, 20), warmup)
        n1_us = n1_secs / max(steps, 20) * 1e6
    out = {"rows_per_gpu": ROWS // world, "n1_same_run_us_warm_l2": n1_us}
    for exchange in ("peer", "all_gather"):
        lins = [RowSplitLinear.from_host(dev, h, kind, ROWS, COLS, rank, world, exchange=exchange) for h in hosts]

        def step():
            for lin in lins:
                lin.forward(x, y)

        graph = all(lin.capturable for lin in lins)
        secs = max_over_ranks(torch, dist, time_region(torch, step, steps, warmup, barrier, graph=graph))
        y.fill_(float("nan"))
        lins[-1].forward(x, y)
        torch.cuda.synchronize()
        status_error = None
        try:
            dev.check_status()
        except Exception as e:
            status_error = repr(e)
        us = secs / steps / copies * 1e6
        entry = {"us_per_matvec": round(us, 2), "gbs_whole_weight": round(algorithmic_bytes(kind, ROWS, COLS, batch) / us / 1e3, 1),
                 "launch": "cuda graph" if graph else "eager"}
        bad = False
        if rank == 0:
            err = max_rel_err(y.cpu().numpy(), y1.cpu().numpy())
            entry["parity"] = {"against": "the whole weight on rank 0", "max_rel_err": err, "ok": bool(err <= TOL)}
            bad = not entry["parity"]["ok"]
        if status_error:
            entry["status_error"] = status_error
        entry["failed_on_some_rank"] = agree(torch, dist, bad or status_error is not None)
        out[exchange] = entry
        for lin in lins:
            lin.free()
    if whole is not None:
        whole.free()
    return out


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
    peak, tpeak, peak_kind = measured_peaks()
    steps, warmup, passes = args.steps, max(args.warmup, 3), args.passes
    dsteps = max(steps, 20)   # the detail legs time at least this many steps
    errors = {}

    def leg(name, fn):
        """One rank: a failing detail leg must not take the headline number with it. Several ranks:
        nothing is caught here (a rank that skipped the rest of a leg would desynchronise the others)."""
        if world > 1:
            return fn()
        try:
            return fn()
        except Exception as e:
            traceback.print_exc()
            errors[name] = repr(e)
            return {"error": repr(e)}

    with ClockSampler(local) as clocks:
        head = bench_matvec(dev, torch, HEAD_KIND, 1, steps, warmup, passes, barrier, clocks=clocks)
        head_clocks = clocks.summary()
        secs = head["ms_per_step"] / 1e3 * steps
        if world > 1:
            secs = max_over_ranks(torch, dist, secs)
        value = world * head["copies"] * passes * head["bytes_per_matvec"] * steps / secs / 1e9

        sections = set(v for v in args.sections.split(",") if v)
        detail = {}
        if not args.quick and "detail" in sections:
            dpasses = max(1, passes // 4)
            for kind in (8, 12, 14):
                for batch in (1, 2, 4, 8):
                    if kind == HEAD_KIND and batch == 1:
                        continue
                    r = leg(f"detail_{KIND_NAME[kind]}_b{batch}",
                            lambda: bench_matvec(dev, torch, kind, batch, dsteps, 3, dpasses, barrier, clocks=clocks))
                    detail[f"{KIND_NAME[kind]}_b{batch}"] = r if "error" in r else {
                        "gbs": round(r["gbs"], 1), "us": round(r["us_per_matvec"], 2), "frac_of_peak": round(r["gbs"] / peak, 4),
                        "timed_ms": round(r["timed_ms"], 1), "sm_mhz": r.get("sm_mhz")}
        prefill, prefill_q4, prefill_q6 = {}, {}, {}
        if not args.quick and "prefill" in sections and world == 1:
            shapes = [tuple(int(d) for d in v.split("x")) for v in args.prefill_shapes.split(",") if v]
            for (M, N) in shapes:
                psteps = max(dsteps, min(2000, int(0.2 / (2.0 * M * N * 4096 / (0.5 * tpeak * 1e12)))))  # about 0.2 s per leg
                prefill[f"M{M}_N{N}"] = leg(f"prefill_M{M}_N{N}", lambda: bench_prefill(dev, torch, M, N, 4096, psteps, 3, tpeak))
            for (M, N) in shapes:   # the same kernel with Q4_K weights (from 256 tokens on), on the large row count
                if M >= 256 and N == max(n for _, n in shapes):
                    psteps = max(dsteps, min(2000, int(0.2 / (2.0 * M * N * 4096 / (0.5 * tpeak * 1e12)))))
                    prefill_q4[f"M{M}_N{N}"] = leg(f"prefill_q4_k_M{M}_N{N}", lambda: bench_prefill(dev, torch, M, N, 4096, psteps, 3, tpeak, kind=12))
                    prefill_q6[f"M{M}_N{N}"] = leg(f"prefill_q6_k_M{M}_N{N}", lambda: bench_prefill(dev, torch, M, N, 4096, psteps, 3, tpeak, kind=14))
        attention = {}
        if not args.quick and "attention" in sections and world == 1:
            attention["prefill_512"] = leg("attention_prefill", lambda: bench_attention(dev, torch, 512, 0, max(dsteps, 100), 3))
            attention["decode_at_600"] = leg("attention_decode", lambda: bench_attention(dev, torch, 1, 599, max(dsteps, 400), 3))
        moe = {}
        tokens = () if (args.quick or "moe" not in sections) else tuple(int(v) for v in args.moe_tokens.split(",") if v)
        if world == 1:
            for T in tokens:
                msteps = max(dsteps, 400 if T <= 64 else 200)
                moe[f"T{T}"] = leg(f"moe_T{T}", lambda: bench_moe_single(dev, torch, T, msteps, 3))
        elif tokens:
            from exec_beholdd_b200 import expert_parallel

            m = MOE
            single = (expert_parallel.ExpertParallelLayer.from_synthetic(dev, SEED, m["n_experts"], m["dim"], m["ff"], m["top_k"])
                      if rank == 0 else None)
            exchanges = [v for v in args.exchanges.split(",") if v]
            for T in tokens:
                moe[f"T{T}"] = bench_moe_parallel(dev, torch, dist, T, max(dsteps, 50), 3, rank, world, barrier, exchanges, single)
            if single is not None:
                single.free()

        row_split = None
        if world > 1 and not args.quick and ROWS % world == 0 and "rowsplit" in sections:
            row_split = {f"b{b}": bench_row_split(dev, torch, dist, HEAD_KIND, b, max(dsteps, 50), 3, rank, world, barrier)
                         for b in (1, 4)}

        full = None
        if not args.quick and "forward" in sections:
            full = leg("full_forward", lambda: bench_full_forward(dev, torch, dist, rank, world))

        e2e = leg("e2e", lambda: bench_matvec_e2e(dev, torch, HEAD_KIND, steps, 3, head["copies"], max(1, passes // 4)))
        if world > 1:  # whole-job figure: the replicas' rates add up
            e2e = dict(e2e, value=_sum_over_ranks(torch, dist, e2e["value"]))

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
            "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "config": {"workload": head_workload_text(head["copies"], passes),
                       "parallelism": "replicas" if world > 1 else "single"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": HEAD_TRAFFIC_BYTES, "peak_source": peak_kind,
                         "kernel": "k_matvec_decode_i8 (the only kernel of the step)", "us_per_launch": launch_us},
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": head["launches_timed"],
            "clocks": head_clocks, "matvec_detail": detail, "prefill_q8_0_k4096": prefill, "prefill_q4_k_k4096": prefill_q4, "prefill_q6_k_k4096": prefill_q6, "attention": attention, "moe_layer": moe,
            "row_split_projection": row_split, "full_forward": full,
        }
        if errors:
            line["errors"] = errors
        print(json.dumps(line), flush=True)
    dev.close()
    if world > 1:
        dist.destroy_process_group()


def _sum_over_ranks(torch, dist, v):
    t = torch.tensor([v], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t.item()


def main():
    faulthandler.enable()  # a fatal signal in any rank leaves that rank's Python stack on stderr
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--passes", type=int, default=100, help="passes over the rotating weight set per step of the headline workload")
    ap.add_argument("--quick", action="store_true", help="headline workload only")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--moe-tokens", default="1,16,64,512", help="token counts of the routed-layer detail runs")
    ap.add_argument("--exchanges", default="peer,alltoall,gather", help="expert-parallel exchanges to run with several ranks")
    ap.add_argument("--sections", default="detail,prefill,attention,moe,rowsplit,forward", help="which detail runs follow the headline workload")
    ap.add_argument("--prefill-shapes", default="128x12288,128x4096,512x12288,512x4096,2048x12288,2048x4096",
                    help="MxN cases of the Q8_0 K=4096 prefill matmul detail run")
    args = ap.parse_args()
    try:
        if args.impl == "reference":
            run_reference_arm(args)
        else:
            run_gpu_arm(args)
    except BaseException:
        # every rank's traceback reaches stderr before the launcher tears the job down
        sys.stderr.write(f"[bench rank {os.environ.get('RANK', '0')}] failed:\n{traceback.format_exc()}\n")
        sys.stderr.flush()
        raise


if __name__ == "__main__":
    main()
