#!/usr/bin/env python
"""Benchmark of the quantized-decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-moe] [--check-multi-rank]
    python bench.py --case NAME        # one small workload only (for a profiler), see run_case

Workload (``config.workload``): the mixed-format decode GEMVs at Llama-3-8B shapes,
batch 1, bf16 activations ~ N(0,1), weights quantized from seeded N(0, 0.02) fp32:
Q8_0 4096x4096, Q4_K 14336x4096, Q6_K 4096x14336. One STEP is one pass over
``rotate`` distinct copies of the three matrices (more bytes than two L2s, so every
weight byte comes from HBM), i.e. 3*rotate GEMV launches replayed from one CUDA graph.

Metric: GB/s of algorithmic bytes (packed weight bytes + x + y per GEMV, the
reference's own convention of counting the packed payload). ``roofline`` is the Q4_K
14336x4096 GEMV alone, timed with CUDA events on the launch stream, against the
measured HBM copy bandwidth in MEASURED_PEAKS.json; it also carries the read-only streaming
ceiling measured in the same run (``read_only_ceiling_GBps`` over 1 GiB, ``read_only_same_size_GBps`` over the
same 33 MB per launch), two and four matrices per launch (``matrices_per_launch``,
kdnn_b200_quant_gemv_multi), the measured DRAM bytes of one launch (``traffic``), the other shapes (``by_shape``)
and the batched sweep of 1..32 activation rows on the 14336x4096 matrix (``by_batch``).
``e2e`` is the same pass driven from pinned host buffers through
kdnn_b200_quant_gemv_host: per GEMV the activation row goes host->device and the result row
device->host inside the timed region, and the host results are checked.
``moe_decode`` carries the second headline number (tokens/s of the 48-layer, 128-expert,
top-8 MoE stack at 256 tokens) with the time per layer of every tile kernel, and
``moe_layer_c4`` the coarse configuration (8 experts, top-2, hidden 4096, FFN 14336, 64 tokens).

With --gpus N > 1 (launched under torchrun) every rank runs the same GEMV pass on its
own GPU (replicas: the GEMV does not shard at these sizes; ``gemv_rowsplit`` measures the
row split + all-gather it would take and where it starts to pay). The MoE stack is
expert-parallel over the ranks: its outputs are first checked against a one-rank run of the same
stack (untimed, two layers), then both exchange designs are timed.

``--impl reference`` times the reference's own CPU int8 GEMV (oracle/_ref, compiled
from the reference's headers; the C port when that library is absent) on the host
cores, on the same matrices.
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

Q8_0, Q4_K, Q6_K = 8, 12, 14
GEMV_SHAPES = [("Q8_0", Q8_0, 4096, 4096), ("Q4_K", Q4_K, 14336, 4096), ("Q6_K", Q6_K, 4096, 14336)]
SEED = 20261125
WORKLOAD = ("mixed-format decode GEMVs, Llama-3-8B shapes: Q8_0 4096x4096, Q4_K 14336x4096, Q6_K 4096x14336, "
            "batch 1, bf16 activations, fp32 outputs")


def algorithmic_bytes(dtype, rows, K, xbytes=2, ybytes=4):
    blk, bsz = {Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210)}[dtype]
    return rows * (K // blk) * bsz + K * xbytes + rows * ybytes


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index, enabled: bool = True):
        """gpu_index: one index, or a list of indices (one nvidia-smi call samples them all). Only one process of a
        multi-rank job should sample: a dozen concurrent nvidia-smi queries disturb the GPUs they look at."""
        self.idx = ",".join(str(i) for i in gpu_index) if isinstance(gpu_index, (list, tuple)) else str(gpu_index)
        self.enabled = enabled
        self.rows = []
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", self.idx], capture_output=True, text=True, timeout=5).stdout
                for line in out.strip().splitlines():
                    self.rows.append([c.strip() for c in line.split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        if self.enabled:
            self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self.enabled:
            self._t.join(timeout=6)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except Exception:
                continue
            for n, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def build_weights(pack):
    """Seeded N(0, 0.02) fp32 -> packed bytes, one matrix per shape (host numpy)."""
    out = []
    for i, (name, dt, rows, K) in enumerate(GEMV_SHAPES):
        out.append(pack.synth_weight(dt, rows, K, SEED + i, std=0.02))
    return out


# ---------------------------------------------------------------------------------------
def _cpu_engine(use_ref=True):
    from oracle import oracle as O
    O.build()
    if use_ref and O.Ref.available():
        return O, O.Ref(), "reference"
    return O, O.Port(), "port"


def _cpu_pass_fn(O, eng, kind, host_weights):
    rng = np.random.default_rng(SEED)
    xs = [O.bf16_round(rng.standard_normal(K).astype(np.float32)) for (_, _, _, K) in GEMV_SHAPES]
    ws = [O.aligned_copy(w) for w in host_weights]

    def one_pass():
        for (name, dt, rows, K), w, x in zip(GEMV_SHAPES, ws, xs):
            if kind == "reference":
                eng.quant_gemv(dt, w, rows, K, x, bf16=True, int8=True)
            else:
                eng.gemv_int8(dt, w, rows, K, x)
    return one_pass


def cpu_leg(host_weights, target_seconds, use_ref=True):
    """Times the reference's CPU int8 quant_gemv on the three matrices on all host threads and on one.
    Returns the `cpu_baseline` object (value = the median pass on all cores)."""
    O, eng, kind = _cpu_engine(use_ref)
    nbytes = sum(algorithmic_bytes(dt, rows, K) for (_, dt, rows, K) in GEMV_SHAPES)
    one_pass = _cpu_pass_fn(O, eng, kind, host_weights)
    out = {}
    for label, threads, budget in (("all", os.cpu_count() or 1, target_seconds * 0.7), ("one", 1, target_seconds * 0.3)):
        eng.set_threads(threads)
        one_pass()
        t0 = time.perf_counter()
        one_pass()
        t1 = time.perf_counter() - t0
        n = max(3, min(200, int(budget / max(t1, 1e-6))))
        times = []
        for _ in range(n):
            t0 = time.perf_counter()
            one_pass()
            times.append(time.perf_counter() - t0)
        out[label] = (threads, n, nbytes / statistics.median(times) / 1e9, nbytes / min(times) / 1e9)
    cores, n, med, best = out["all"]
    how = "reference functor bodies under a stand-in OpenMP scheduler" if kind == "reference" else "C restatement with OpenMP"
    return {"value": med, "unit": "GB/s", "cores": cores, "kind": kind, "statistic": "median pass",
            "best_pass_GBps": best, "one_core_GBps": out["one"][2],
            "sample": f"{n} passes over the three GEMVs ({nbytes / 1e6:.1f} MB per pass) on {cores} threads, "
                      f"{out['one'][1]} passes on 1 thread; {how}"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import __graft_entry__ as ge
    pack = ge._load_module("_kd_pack", os.path.join(ge.PKG_DIR, "ggml_pack.py"))
    host_weights = build_weights(pack)
    O, eng, kind = _cpu_engine()
    cores = os.cpu_count() or 1
    eng.set_threads(cores)
    nbytes = sum(algorithmic_bytes(dt, rows, K) for (_, dt, rows, K) in GEMV_SHAPES)
    step = _cpu_pass_fn(O, eng, kind, host_weights)
    for _ in range(args.warmup):
        step()
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    val = nbytes / med / 1e9
    sample = (f"each step = one pass over the three GEMVs ({nbytes / 1e6:.1f} MB), host resident; value = median step "
              f"of {args.steps}")
    line = {
        "impl": "reference", "metric": "gguf_int8_gemv_algorithmic_GBps", "value": val, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": med * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 dots, fp32 rescale", "data": "synthetic",
        "config": {"workload": WORKLOAD, "seed": SEED},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": kind, "statistic": "median step",
                         "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------
def _graph_time_us(torch, stream, fn, iters=5, warm=3):
    """Average time of one replay of `fn` captured as a CUDA graph, CUDA events on the launch stream."""
    with torch.cuda.stream(stream):
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
        for _ in range(warm):
            g.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(iters):
            g.replay()
        b.record(stream)
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / iters


def measured_dram_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, as written by the ncu
    capture summarised under profiles/ (None when that file is absent)."""
    path = os.path.join(ROOT, "profiles", "gemv_q4k_14336x4096_dram_bytes.txt")
    if not os.path.exists(path):
        return None
    vals = {}
    for line in open(path):
        if "=" in line and not line.startswith("#"):
            k, v = line.split("=", 1)
            vals[k.strip()] = float(v.split()[0])
    if "dram__bytes_read.sum" in vals and "dram__bytes_write.sum" in vals:
        return vals["dram__bytes_read.sum"] + vals["dram__bytes_write.sum"]
    return None


def run_check_multi_rank(args):
    import torch
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    import __graft_entry__ as ge
    kd = ge.load_package()
    ms = ge._load_module("_kd_moe_bench", os.path.join(ge.PKG_DIR, "moe_stack.py"))
    res = ms.check_multi_rank(kd, dev, rank, world, layers=2, cfg=ms.StackConfig(experts=16, tokens=32, hidden=512, ffn=256, top_k=4))
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        print(f"[bench] rank {rank}/{world} on cuda:{local} ({torch.cuda.get_device_name(local)}), NCCL "
              f"{'.'.join(str(v) for v in torch.cuda.nccl.version())}, backend {dist.get_backend()}", file=sys.stderr, flush=True)

    import __graft_entry__ as ge
    kd = ge.load_package()
    host_weights = build_weights(kd.ggml_pack)
    per_set = sum(algorithmic_bytes(dt, rows, K) for (_, dt, rows, K) in GEMV_SHAPES)
    rotate = max(4, int(2 * 126e6 * 1.5 // per_set) + 1)            # > 2 x L2 of distinct bytes per step

    # device state: `rotate` copies of each matrix, inputs, outputs, staging
    sets = []
    for r in range(rotate):
        ws = []
        for (name, dt, rows, K), hw in zip(GEMV_SHAPES, host_weights):
            ws.append(kd.QuantWeight.from_numpy(hw, dt, rows, K, dev))
        sets.append(ws)
    g = torch.Generator().manual_seed(SEED)
    xs_host = [torch.randn(K, generator=g).to(torch.bfloat16).pin_memory() for (_, _, _, K) in GEMV_SHAPES]
    xs = [x.to(dev) for x in xs_host]
    ys = [torch.empty(rows, dtype=torch.float32, device=dev) for (_, _, rows, _) in GEMV_SHAPES]
    ys_host = [torch.empty(rows, dtype=torch.float32).pin_memory() for (_, _, rows, _) in GEMV_SHAPES]
    scr = [torch.empty(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device=dev)
           for (_, _, _, K) in GEMV_SHAPES]

    def one_pass():
        for ws in sets:
            for i, w in enumerate(ws):
                kd.quant_gemv(xs[i], w, ys[i], scr[i])

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        one_pass()
        torch.cuda.synchronize()
        ys_first = [y.clone() for y in ys]          # results of the plain launches (the GPU tests' path)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_pass()
    torch.cuda.synchronize()

    def replay_is_complete(g, outs, firsts):
        """Poison the outputs, replay once more, and require every row to be recomputed bit-for-bit."""
        with torch.cuda.stream(stream):
            for y in outs:
                y.fill_(float("nan"))
            g.replay()
        torch.cuda.synchronize()
        return all(torch.equal(y, f) for y, f in zip(outs, firsts))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: K steps, CUDA events on the launch stream ----------
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            graph.replay()
    barrier()
    # the K timed steps are captured together (chunks of at most 50 steps per graph), so that the host's graph
    # launches (about 25 us each, a quarter of a step) are not what is timed
    chunk = max(1, min(args.steps, 50))
    graph_chunk = graph
    if chunk > 1:
        graph_chunk = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph_chunk, stream=stream):
                for _ in range(chunk):
                    one_pass()
            graph_chunk.replay()
        torch.cuda.synchronize()
        barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(list(range(world)) if world > 1 else local, enabled=(rank == 0)) as clocks:
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(args.steps // chunk):
                graph_chunk.replay()
            for _ in range(args.steps % chunk):
                graph.replay()
            e1.record(stream)
        # the timed work is complete BEFORE the closing barrier is enqueued: its NCCL kernel would otherwise spin on a
        # few SMs next to the last timed launches (that cost 15 % at 2 to 8 ranks)
        stream.synchronize()
        barrier()
        ms_total = e0.elapsed_time(e1)
        # keep the GPU busy long enough for a few clock samples
        if ms_total < 1500:
            with torch.cuda.stream(stream):
                for _ in range(int(1500 / max(ms_total / args.steps, 1e-3))):
                    graph.replay()
            torch.cuda.synchronize()
    if not replay_is_complete(graph, ys, ys_first):
        raise RuntimeError("a replayed step did not reproduce the results of the plain launches")
    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    bytes_step = per_set * rotate
    value = world * bytes_step * args.steps / (ms_total * 1e-3) / 1e9
    launches = 3 * rotate * args.steps

    # ---- the same twelve launches grouped by shape (all Q8_0, then all Q4_K, then all Q6_K): three different
    # kernels taking turns cost more than the sum of their single-shape sequences, two do not ------------------
    def grouped_pass():
        for i in range(len(GEMV_SHAPES)):
            for ws in sets:
                kd.quant_gemv(xs[i], ws[i], ys[i], scr[i])
    pass_order = {"interleaved_us": ms_total / args.steps * 1e3,
                  "grouped_by_shape_us": _graph_time_us(torch, stream, lambda: [grouped_pass() for _ in range(10)], iters=5) / 10}

    # ---- per-kernel roofline: each shape alone, rotating copies, CUDA events -----------
    peak, peak_kind = measured_peaks()
    per_kernel = {}
    for i, (name, dt, rows, K) in enumerate(GEMV_SHAPES + [("Q4_K_4096", Q4_K, 4096, 4096)]):
        if i < 3:
            copies = [s[i] for s in sets]
            # at least 2.5 L2s of distinct weights per sweep, whatever the matrix size (four copies of the 17.8 MB
            # Q8_0 matrix would sit in the 126 MB L2)
            need = int(2.5 * 126e6 // algorithmic_bytes(dt, rows, K)) + 1
            copies = copies + [kd.QuantWeight.from_numpy(host_weights[i], dt, rows, K, dev)
                               for _ in range(max(0, need - len(copies)))]
            x, y, sc = xs[i], ys[i], scr[i]
        else:
            hw = kd.ggml_pack.synth_weight(dt, rows, K, SEED + 9, std=0.02)
            ncp = int(2.5 * 126e6 // algorithmic_bytes(dt, rows, K)) + 1
            copies = [kd.QuantWeight.from_numpy(hw, dt, rows, K, dev) for _ in range(ncp)]
            x, y, sc = xs[0], torch.empty(rows, dtype=torch.float32, device=dev), scr[0]
        reps = max(1, int(600e6 // (algorithmic_bytes(dt, rows, K) * len(copies))))
        gk = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            for w in copies:
                kd.quant_gemv(x, w, y, sc)
            torch.cuda.synchronize()
            y_first = y.clone()
            with torch.cuda.graph(gk, stream=stream):
                for _ in range(reps):
                    for w in copies:
                        kd.quant_gemv(x, w, y, sc)
            for _ in range(3):
                gk.replay()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(5):
                gk.replay()
            b.record(stream)
        torch.cuda.synchronize()
        if not replay_is_complete(gk, [y], [y_first]):
            raise RuntimeError(f"replayed {name} GEMVs did not reproduce the results of the plain launches")
        us = a.elapsed_time(b) * 1e3 / (5 * reps * len(copies))
        ab = algorithmic_bytes(dt, rows, K)
        per_kernel[f"{name}_{rows}x{K}"] = {"us_per_launch": us, "algorithmic_bytes": ab,
                                            "achieved_GBps": ab / us / 1e3, "frac": ab / us / 1e3 / peak}
    dom = per_kernel["Q4_K_14336x4096"]

    # ---- read-only streaming ceiling (the reference's benchmarks quote their GEMVs against one) ------
    big = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
    big.fill_(1)
    sink = torch.zeros(4, dtype=torch.int32, device=dev)
    ro_us = _graph_time_us(torch, stream, lambda: kd.read_probe(big, sink), iters=10)
    read_only = big.numel() / ro_us / 1e3
    del big
    # the same read-only kernel at the SIZE of the dominant GEMV (33 MB per launch, launches back to back on
    # rotating copies): what a launch that streams this few bytes can reach with its ramp and its tail
    q4 = [s[1] for s in sets]
    q4 = q4 + [kd.QuantWeight.from_numpy(host_weights[1], Q4_K, 14336, 4096, dev) for _ in range(max(0, 10 - len(q4)))]
    ro_small_us = _graph_time_us(torch, stream, lambda: [kd.read_probe(w.data, sink) for w in q4], iters=10) / len(q4)
    read_only_same_size = q4[0].data.numel() / ro_small_us / 1e3

    # ---- several matrices per launch (gate + up of a decoder share the activation row) --------------------
    multi = {}
    ab4 = algorithmic_bytes(Q4_K, 14336, 4096)
    pool = q4 + [kd.QuantWeight.from_numpy(host_weights[1], Q4_K, 14336, 4096, dev) for _ in range((-len(q4)) % 4 + 4)]
    youts = [torch.empty(14336, dtype=torch.float32, device=dev) for _ in range(4)]
    for nm in (2, 4):
        groups = [pool[i:i + nm] for i in range(0, len(pool) - nm + 1, nm)]
        us = _graph_time_us(torch, stream, lambda: [kd.quant_gemv_multi(xs[1], g_, youts[:nm], scr[1]) for g_ in groups],
                            iters=10) / (len(groups) * nm)
        multi[str(nm)] = {"us_per_matrix": us, "achieved_GBps": ab4 / us / 1e3, "frac": ab4 / us / 1e3 / peak}
    del pool

    # ---- batched sweep: 1..32 activation rows against Q4_K 14336 x 4096 (rotating copies) ------------
    by_batch = {}
    copies = q4
    N_, K_ = 14336, 4096
    paths = {1: "GEMV kernel per row", 2: "GEMV kernel per row", 4: "tcgen05 tile kernel", 8: "tcgen05 tile kernel",
             16: "mma.sync tile kernel", 32: "mma.sync tile kernel"}
    for M in (1, 2, 4, 8, 16, 32):
        X = torch.randn(M, K_, generator=torch.Generator().manual_seed(SEED + M)).to(torch.bfloat16).to(dev)
        Y = torch.empty(M, N_, dtype=torch.float32, device=dev)
        wsp = torch.zeros(kd.quant_gemm_workspace_bytes(M, K_), dtype=torch.uint8, device=dev)

        def sweep():
            for w in copies:
                kd.quant_gemm(X, w, Y, wsp)
        us = _graph_time_us(torch, stream, sweep) / len(copies)
        ab = N_ * (K_ // 256) * 144 + M * K_ * 2 + M * N_ * 4
        by_batch[str(M)] = {"us": us, "algorithmic_GBps": ab / us / 1e3, "frac": ab / us / 1e3 / peak, "path": paths[M]}
    assert kd.device_status() == 0, "a bounded device-side wait gave up"

    roofline = {"kernel": "gemv_q4k_xreg_kernel 14336x4096", "bound": "hbm", "achieved": dom["achieved_GBps"],
                "peak": peak, "peak_source": f"{peak_kind} HBM copy bandwidth (MEASURED_PEAKS.json)",
                "unit": "GB/s", "frac": dom["frac"], "frac_of_nominal_8TBps": dom["achieved_GBps"] / 8000.0,
                "read_only_ceiling_GBps": read_only, "frac_of_read_only_ceiling": dom["achieved_GBps"] / read_only,
                "read_only_same_size_GBps": read_only_same_size,
                "frac_of_read_only_same_size": dom["achieved_GBps"] / read_only_same_size,
                "matrices_per_launch": multi,
                "traffic": measured_dram_traffic(), "by_shape": per_kernel, "by_batch": by_batch,
                "pass_order": pass_order}

    # ---- end to end through the public call with host buffers --------------------------
    def e2e_pass():
        for ws in sets:
            for i, w in enumerate(ws):
                # one C-ABI call: pinned x -> device, GEMV, y -> pinned host memory
                kd.quant_gemv_host(xs_host[i], w, ys_host[i], xs[i], ys[i], scr[i])

    with torch.cuda.stream(stream):
        for _ in range(3):
            e2e_pass()
    barrier()
    steps_e2e = max(2, min(args.steps, 20))
    # (a) the calls made one by one from Python: bound by the host (ctypes call + three launches per GEMV)
    t0 = time.perf_counter()
    with torch.cuda.stream(stream):
        for _ in range(steps_e2e):
            e2e_pass()
        stream.synchronize()
    direct_s = time.perf_counter() - t0
    # (b) the same calls captured into one CUDA graph, as a decode loop would hold them: every step still moves
    # its activation rows host -> device and its result rows device -> host; wall clock around replay + synchronize
    for h in ys_host:
        h.fill_(float("nan"))
    graph_e2e = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph_e2e, stream=stream):
            for _ in range(steps_e2e):
                e2e_pass()
        graph_e2e.replay()
        stream.synchronize()
    barrier()
    t0 = time.perf_counter()
    with torch.cuda.stream(stream):
        graph_e2e.replay()
        stream.synchronize()
    e2e_s = time.perf_counter() - t0
    if not all(torch.equal(h, f.cpu()) for h, f in zip(ys_host, ys_first)):
        raise RuntimeError("the host-buffer pass did not deliver the results of the device-resident pass")
    td = torch.tensor([direct_s], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(td, op=dist.ReduceOp.MAX)
    e2e_direct = world * bytes_step * steps_e2e / float(td.item()) / 1e9
    t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_val = world * bytes_step * steps_e2e / float(t.item()) / 1e9
    h2d = rotate * sum(K * 2 for (_, _, _, K) in GEMV_SHAPES)
    d2h = rotate * sum(rows * 4 for (_, _, rows, _) in GEMV_SHAPES)
    assert kd.device_status() == 0, "a bounded device-side wait gave up"
    del sets, copies
    torch.cuda.empty_cache()

    # ---- row-split GEMV + all-gather (N > 1): what sharding a GEMV over the ranks would cost ----------
    rowsplit = None
    if world > 1:
        rowsplit = {}
        for name, dt, rows, K in (("Q4_K_14336x4096", Q4_K, 14336, 4096), ("Q5_K_131072x4096 (lm_head class)", 13, 131072, 4096)):
            hw = kd.ggml_pack.random_payload(dt, rows, K, SEED + 77)
            rb = hw.size // rows
            full = kd.QuantWeight.from_numpy(hw, dt, rows, K, dev)
            part_rows = rows // world
            part = kd.QuantWeight.from_numpy(hw.reshape(rows, rb)[rank * part_rows:(rank + 1) * part_rows].copy(), dt,
                                             part_rows, K, dev)
            x = torch.randn(K, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).to(dev)
            sc = torch.empty(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device=dev)
            y_full = torch.empty(rows, dtype=torch.float32, device=dev)
            y_part = torch.empty(part_rows, dtype=torch.float32, device=dev)
            y_all = torch.empty(rows, dtype=torch.float32, device=dev)
            kd.quant_gemv(x, full, y_full, sc)

            def split():
                kd.quant_gemv(x, part, y_part, sc)
                dist.all_gather_into_tensor(y_all, y_part)
            barrier()
            us_split = _graph_time_us(torch, stream, split, iters=20)
            us_one = _graph_time_us(torch, stream, lambda: kd.quant_gemv(x, full, y_full, sc), iters=20)
            same = bool(torch.equal(y_all, y_full))
            tt = torch.tensor([us_split], dtype=torch.float64, device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            rowsplit[name] = {"one_gpu_us": us_one, "row_split_plus_all_gather_us": float(tt.item()), "ranks": world,
                              "speedup": us_one / float(tt.item()), "results_identical": same,
                              "note": "same matrix resident in L2-sized repeats (no rotation): latency comparison"}
            del full, part
            torch.cuda.empty_cache()

    moe = None
    c4 = None
    if not args.no_moe:
        moe_bench = ge._load_module("_kd_moe_bench", os.path.join(ge.PKG_DIR, "moe_stack.py"))
        steps_m = max(2, min(args.steps, 10))
        if world > 1:
            chk = moe_bench.check_multi_rank(kd, dev, rank, world, layers=2)
            if not (chk["push"] <= 1e-3 and chk["allreduce"] <= 2.0 ** -6 and chk["device_status"] == 0):
                raise RuntimeError(f"expert-parallel stack differs from the one-rank stack: {chk}")
        moe = moe_bench.bench_moe_stack(kd, dev, rank, world, steps=steps_m, warmup=3, peak=peak, exchange="push")
        if world > 1:
            moe["correctness_vs_one_rank"] = chk
            alt = moe_bench.bench_moe_stack(kd, dev, rank, world, steps=steps_m, warmup=3, peak=peak, exchange="allreduce")
            moe["allreduce_design"] = {k: alt[k] for k in ("value", "us_per_layer", "gpu_launches_per_step")}
        else:
            small = moe_bench.StackConfig(layers=8)
            per_kind = {}
            for kind, nm in ((1, "mma.sync"), (2, "tcgen05")):
                r = moe_bench.bench_moe_stack(kd, dev, rank, world, steps=steps_m, warmup=3, peak=peak, cfg=small,
                                              tile_kind=kind)
                per_kind[nm] = r["us_per_layer"]
            moe["us_per_layer_by_tile_kernel"] = per_kind
            c4cfg = moe_bench.StackConfig(layers=2, hidden=4096, ffn=14336, experts=8, top_k=2, tokens=64)
            c4 = {"config": "8 experts, top-2, hidden 4096, FFN 14336, 64 tokens, one block = 792.7 MB of packed experts",
                  "us_per_layer": {}}
            for kind, nm in ((1, "mma.sync"), (2, "tcgen05")):
                r = moe_bench.bench_moe_stack(kd, dev, rank, world, steps=steps_m, warmup=3, peak=peak, cfg=c4cfg,
                                              tile_kind=kind)
                c4["us_per_layer"][nm] = r["us_per_layer"]
            best = min(c4["us_per_layer"].values())
            c4["hbm_frac"] = c4cfg.layer_bytes() / best / 1e3 / peak
            c4["tokens_per_s"] = 64 / (best * 1e-6)

    cpu = None
    if rank == 0 and world == 1:
        cpu = cpu_leg(host_weights, target_seconds=12.0)

    if rank == 0:
        line = {
            "metric": "gguf_int8_gemv_algorithmic_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 dots, fp32 rescale", "data": "synthetic",
            "config": {"workload": WORKLOAD, "rotate": rotate, "bytes_per_step": bytes_step, "l2": "inputs larger than L2 "
                       f"({bytes_step / 1e6:.0f} MB of distinct weights per step)", "seed": SEED,
                       "replay": "the K timed steps captured together in CUDA graphs of at most 50 steps",
                       "multi_gpu": "replicas only (GEMV); MoE stack expert-parallel"},
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "how": "kdnn_b200_quant_gemv_host per GEMV (pinned x in, pinned y out), the steps' calls captured into one "
                           "CUDA graph, wall clock around replay + synchronize",
                    "python_calls_one_by_one_GBps": e2e_direct},
            "gpu_launches": launches, "clocks": clocks.summary(), "moe_decode": moe, "moe_layer_c4": c4,
            "gemv_rowsplit": rowsplit,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_case(args):
    """One small workload on one GPU, a few hundred MB on the device and a handful of launches: the thing to
    put under a profiler (`--case gemv_q4k | gemv_q6k | gemv_q80 | gemv_q4k_pair | moe_block | moe_block_tcgen05`).
    gemv_*: 13 cold copies of the matrix, three passes over them. moe_block*: one 128-expert / top-8 / hidden
    2048 / FFN 768 block on 256 tokens, three calls."""
    import torch
    import __graft_entry__ as ge
    kd = ge.load_package()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    if args.case.startswith("gemv"):
        dt, rows, K = {"gemv_q4k": (Q4_K, 14336, 4096), "gemv_q4k_pair": (Q4_K, 14336, 4096),
                       "gemv_q6k": (Q6_K, 4096, 14336), "gemv_q80": (Q8_0, 4096, 4096)}[args.case]
        host = kd.ggml_pack.synth_weight(dt, rows, K, SEED, std=0.02)
        ws = [kd.QuantWeight.from_numpy(host, dt, rows, K, dev) for _ in range(13 if rows * K > 2e7 else 26)]
        x = torch.randn(K, generator=torch.Generator().manual_seed(SEED)).to(torch.bfloat16).to(dev)
        ys = [torch.empty(rows, dtype=torch.float32, device=dev) for _ in range(2)]
        scr = torch.zeros(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device=dev)
        for _ in range(3):
            if args.case == "gemv_q4k_pair":
                for i in range(0, len(ws) - 1, 2):
                    kd.quant_gemv_multi(x, ws[i:i + 2], ys, scr)
            else:
                for w in ws:
                    kd.quant_gemv(x, w, ys[0], scr)
        torch.cuda.synchronize()
        print(json.dumps({"case": args.case, "launches": 3 * (len(ws) // 2 if args.case == "gemv_q4k_pair" else len(ws)), "matrix_bytes": int(host.nbytes),
                          "device_status": kd.device_status()}))
        return
    ms = ge._load_module("_kd_moe_bench", os.path.join(ge.PKG_DIR, "moe_stack.py"))
    kd.tile_kind(2 if args.case.endswith("tcgen05") else 3)
    cfg = ms.StackConfig(layers=1)
    stack = ms.MoeStack(kd, dev, cfg, 0, 1)
    h0 = torch.randn(cfg.tokens, cfg.hidden, device=dev).to(torch.bfloat16)
    for _ in range(3):
        stack.forward(h0)
    torch.cuda.synchronize()
    print(json.dumps({"case": args.case, "block_calls": 3, "device_status": kd.device_status()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-moe", action="store_true")
    ap.add_argument("--check-multi-rank", action="store_true",
                    help="only compare the expert-parallel MoE stack with a one-rank run and print the errors")
    ap.add_argument("--case", default=None,
                    choices=["gemv_q4k", "gemv_q4k_pair", "gemv_q6k", "gemv_q80", "moe_block", "moe_block_tcgen05"],
                    help="run one small workload only (for a profiler) instead of the benchmark")
    args = ap.parse_args()
    if args.case:
        run_case(args)
    elif args.check_multi_rank:
        run_check_multi_rank(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
