#!/usr/bin/env python
"""Benchmark of the INT4 block-16 GEMV decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): the Qwen3-8B-shape per-layer GEMV set at M = 1 -- QKV
4096->6144, O 4096->4096, gate+up 4096->21888, down 10944->4096, LM head
4096->151643 -- in the W4A8 format (packed int4 weights, one binary16 scale per
16-element k-block, binary16 activations quantized to int8 inside the GEMV
prologue).  One step = one pass over the five matrices = five kernel launches.
Weights are seeded synthetic (random-init) values with the benchmark's
distributions; the set is 498 MB, four times the L2, so every pass streams from
HBM.

The metric is achieved HBM bandwidth: algorithmic bytes (nibbles + weight
scales + activations + outputs, each counted once) per second over all ranks.
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

from blackwell_b200 import shapes  # noqa: E402

METRIC = "int4_gemv_hbm_gbs"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
# (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes of one launch of the dominant kernel, from one
# ncu capture of a 65,536-row slice of the LM head (DRAM traffic of this kernel grows in proportion to the rows).
NCU_TRAFFIC_RATIO = 1.023
DTYPE = "int8 x int4 -> int32, f16 weight scale / f32 activation scale"
MIN_TIMED_SECONDS = 0.3  # the timed region lasts at least this long whatever --steps is (clock samples need time)


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def int8_tensor_peak_tops():
    """Dense int8 tensor-core peak used for the M >= 16 rows: twice the measured dense bf16 burst throughput (the
    int8 rate of the part is twice its bf16 rate; the driver measures bf16 only)."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return 2.0 * float(json.load(f)["bf16_tflops"]), "2 x measured bf16"
    except Exception:
        return 2.0 * FALLBACK_BF16_TFLOPS, "2 x fallback bf16"


def workload_config(world: int):
    """The `config` object, identical in both arms."""
    mats = gemv_set()
    return {"workload": "qwen3-8b-shape per-layer GEMV set, M=1, W4A8 block-16 (configs[1])",
            "matrices": [[n, N, K] for n, N, K in mats], "bytes_per_step": set_bytes(mats, 1),
            "l2": "inputs larger than L2 (498 MB set, 126 MB L2)",
            "parallelism": "tp%d" % world if world > 1 else "single"}


_ONLY = None  # (name, N override or None): restricts the set to one matrix, for profiling runs


def gemv_set(shape=shapes.QWEN3_8B):
    mats = shape.gemv_set()
    if _ONLY:
        name, n = _ONLY
        mats = [(nm, n or N, K) for nm, N, K in mats if nm == name]
    return mats


def set_bytes(mats, M=1, x_kind="f16"):
    return sum(shapes.gemv_bytes(N, K, M, 2, x_kind) for _, N, K in mats)


# ----------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._th = None

    def start(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            self.h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.nv = nv
            self.max_mhz = int(nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM))
        except Exception:
            self.nv = None
            return
        self._th = threading.Thread(target=self._run, daemon=True)
        self._th.start()

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.005)

    def stop(self):
        self._stop.set()
        if self._th:
            self._th.join(timeout=1.0)
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ----------------------------------------------------------------------------
def cpu_sample_baseline(threads: int = 0, frac: int = 8, reps: int = 1, seed: int = 900):
    """Times the oracle's scalar dequant-dot (the host port of the reference kernel) on the first 1/frac of the
    rows of each of the five matrices.  Returns (GB/s, cores, sample description, seconds)."""
    import oracle
    from blackwell_b200 import synth

    mats = gemv_set()
    work = []
    for i, (name, N, K) in enumerate(mats):
        n = max(16, N // frac)
        W, sc16, _ = synth.int4_weights(n, K, seed + i)
        x = synth.activations_f16(1, K, seed + 100 + i).astype(np.float32)
        xq, xs = oracle.quantize_int8(x)
        work.append((n, K, W, sc16, xq, xs))
    nbytes = sum(shapes.gemv_bytes(n, K, 1, 2, "f16") for n, K, *_ in work)
    used = 1
    for n, K, W, sc16, xq, xs in work:  # warm-up (page-in, thread pool)
        _, used = oracle.gemv_w4a8_f32(xq, xs, W, sc16, threads)
    t0 = time.perf_counter()
    for _ in range(reps):
        for n, K, W, sc16, xq, xs in work:
            oracle.quantize_int8(np.zeros((1, K), np.float32))  # the activation quantize step of the path
            oracle.gemv_w4a8_f32(xq, xs, W, sc16, threads)
    dt = time.perf_counter() - t0
    gbs = nbytes * reps / dt / 1e9
    sample = f"first 1/{frac} of the rows of each of the 5 matrices (M=1), {reps} pass(es), {nbytes / 1e6:.1f} MB/pass"
    return gbs, used, sample, dt


def cpu_baseline_record(frac_all: int = 8, frac_one: int = 64):
    """All-core and single-thread figures of the host port (the single-thread run takes a smaller row sample)."""
    g, cores, sample, _ = cpu_sample_baseline(0, frac_all, 2)
    g1, _, sample1, _ = cpu_sample_baseline(1, frac_one, 1)
    return {"value": g, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
            "single_thread": {"value": g1, "unit": UNIT, "cores": 1, "sample": sample1}}


def run_reference(args, rank):
    """Reference arm: the reference has no CPU implementation of this path, so its arithmetic restated on the host
    (oracle/oracle.c, scalar fp32 dequant-dot, OpenMP over rows) is timed on all host cores."""
    if rank != 0:
        return
    frac = 8
    # size the step so that warmup + steps stays within a few minutes
    gbs1, cores, sample, dt = cpu_sample_baseline(0, frac, 1)
    times = []
    for _ in range(args.warmup):
        cpu_sample_baseline(0, frac, 1)
    for _ in range(args.steps):
        g, cores, sample, dt = cpu_sample_baseline(0, frac, 1)
        times.append(dt)
    mats = gemv_set()
    nbytes = sum(shapes.gemv_bytes(max(16, N // frac), K, 1, 2, "f16") for _, N, K in mats)
    ref_gpu = None
    try:  # beside the CPU number: the reference's own CUDA kernels on this GPU, when there is one
        import torch

        if torch.cuda.is_available():
            ref_gpu = {"M%d" % mb: per_matrix_times(torch.device("cuda", 0), mb, reference_arm=True) for mb in (1, 8, 16)}
    except Exception as exc:
        ref_gpu = {"error": repr(exc)[:200]}
    t = float(np.mean(times))
    val = nbytes / t / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "reference_cuda_kernels_sm100a": ref_gpu,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------
def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    from blackwell_b200 import kernels as k
    from blackwell_b200 import synth, tp

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    mats = gemv_set()
    M = args.batch
    if args.tune:
        for kv in args.tune.split(","):
            a, b = kv.split("=")
            k.set_tuning(int(a), int(b))
    plan = tp.shard_gemv_set(mats, world, rank)

    # resident state: this rank's shard of the five matrices, activations, outputs
    state = []
    for i, sh in enumerate(plan):
        W, sc = synth.int4_weights_device(sh.n_local, sh.k_local, 500 + 17 * i + rank, device=dev)
        x = synth.activations_f16_device(M, sh.k_local, 600 + i, device=dev)
        y = torch.empty((M, sh.n_local), dtype=torch.float32, device=dev)
        state.append([sh, W, sc, x, y])
    # Exchanges for N > 1: the K-split matrices (o, down) sum their partial results across ranks -- through the
    # library's NVLink peer-load all-reduce by default, through NCCL with --exchange nccl; the row-split outputs
    # (qkv, gate_up, lm_head) stay sharded, as their consumers in the decode step read them sharded.
    coll = None
    if world > 1:
        coll = tp.Collectives(world, rank, dev, exchange=args.exchange, slot_floats=M * max(sh.N for sh in plan))
        for st in state:
            buf = coll.partial_buffer(st[0], M)
            if buf is not None:
                st[4] = buf

    def step():
        for sh, W, sc, x, y in state:
            k.gemv_w4a8_f16in(y, x, W, sc, sh.k_local, sh.n_local, M)
            if coll is not None and sh.kind == "k":
                coll.finish(sh, y)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    # One step is captured into a CUDA graph and replayed: the five launches (and the exchanges, for N > 1)
    # are then issued by the GPU front end back to back, with no per-launch host cost in the timed region.
    use_graph = not args.no_graph
    k.launch_count(reset=True)
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        launches_per_step = k.launch_count()
        run_step = graph.replay
    else:
        step()
        launches_per_step = k.launch_count()
        run_step = step
    for _ in range(3):
        run_step()
    barrier()
    # A step is one pass over the five matrices.  So that the timed region lasts long enough for the clock sampler
    # (and for the driver's own samples) whatever --steps is, every one of the K timed steps is measured as the mean
    # of `passes` back-to-back passes: the timed region holds K x passes passes and ms_per_step = time / (K x passes).
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    for _ in range(10):
        run_step()
    p1.record()
    torch.cuda.synchronize()
    est = max(p0.elapsed_time(p1) / 10 / 1e3, 1e-6)
    passes = max(1, int(np.ceil(args.min_time / (est * args.steps))))
    if world > 1:
        pt = torch.tensor([passes], dtype=torch.int64, device=dev)
        dist.all_reduce(pt, op=dist.ReduceOp.MAX)
        passes = int(pt.item())
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps * passes):
        run_step()
    e1.record()
    barrier()
    launches = launches_per_step * args.steps * passes
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    if world > 1:
        tmax = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        ms = float(tmax.item())
    assert k.device_status() == 0, "a kernel reported a bounded-wait timeout"
    assert coll is None or coll.peer is None or coll.peer.status() == 0, "a peer all-reduce gave up waiting for a rank"
    total_bytes = set_bytes(mats, M)  # whole job: the full matrices, whatever the sharding
    sec_per_step = ms / 1e3 / (args.steps * passes)
    value = total_bytes / sec_per_step / 1e9

    # ---- end to end through the public call with host buffers (pinned), copies inside the timed region
    # The caller keeps the step's activations in ONE pinned buffer and ONE device buffer (the GEMVs read views of it), so
    # that they travel in a single host-to-device copy.
    x_elems = [M * sh.k_local for sh, *_ in state]
    x_offs = [sum(x_elems[:i]) for i in range(len(state))]   # every k_local is a multiple of 32: 16-byte aligned views
    host_xcat = torch.empty(sum(x_elems), dtype=torch.float16).pin_memory()
    dev_xcat = torch.empty(sum(x_elems), dtype=torch.float16, device=dev)
    dev_x = [dev_xcat[o:o + n].view(M, sh.k_local) for o, n, (sh, *_) in zip(x_offs, x_elems, state)]
    for o, n, (_, _, _, x, _) in zip(x_offs, x_elems, state):
        host_xcat[o:o + n].copy_(x.reshape(-1).cpu())
    host_y = [torch.empty((M, sh.n_local), dtype=torch.float32).pin_memory() for sh, *_ in state]
    h2d = host_xcat.numel() * 2
    d2h = sum(h.numel() * 4 for h in host_y)

    # The caller's pipeline: inputs go up first, the largest matrix (the LM head) runs first and every result travels
    # back on a second stream while the next matrices compute, so only the last, small result's copy is exposed.
    copy_stream = torch.cuda.Stream(device=dev)
    e2e_order = sorted(range(len(state)), key=lambda i: -state[i][0].n_local * state[i][0].k_local)

    def e2e_enqueue():
        main = torch.cuda.current_stream()
        dev_xcat.copy_(host_xcat, non_blocking=True)
        for i in e2e_order:
            sh, W, sc, _, y = state[i]
            k.gemv_w4a8_f16in(y, dev_x[i], W, sc, sh.k_local, sh.n_local, M)
            if coll is not None and sh.kind == "k":
                y = coll.finish(sh, y)
            done = torch.cuda.Event()
            done.record(main)
            copy_stream.wait_event(done)
            with torch.cuda.stream(copy_stream):
                host_y[i].copy_(y, non_blocking=True)
        main.wait_stream(copy_stream)

    if use_graph:
        e2e_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(e2e_graph):
            e2e_enqueue()
        e2e_run = e2e_graph.replay
    else:
        e2e_run = e2e_enqueue

    def e2e_step():
        e2e_run()
        torch.cuda.current_stream().synchronize()  # the caller reads the result on the host every step

    for _ in range(3):
        e2e_step()
    barrier()
    e2e_n = args.steps * passes
    t0 = time.perf_counter()
    for _ in range(e2e_n):
        e2e_step()
    barrier()
    e2e_sec = (time.perf_counter() - t0) / e2e_n
    if world > 1:
        tmax = torch.tensor([e2e_sec], dtype=torch.float64, device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        e2e_sec = float(tmax.item())
    e2e_val = total_bytes / e2e_sec / 1e9

    # ---- every matrix on its own, L2-cold (rank 0, single GPU); the reference arm prints the reference's own CUDA
    # kernels on the same shapes
    per, per_batched, cfg0 = [], {}, None
    if rank == 0 and world == 1 and not args.only:
        try:
            per = per_matrix_times(dev, M)
            if M == 1:
                for mb in (8, 16):
                    per_batched["M%d" % mb] = per_matrix_times(dev, mb)
        except Exception as exc:
            per = [{"error": repr(exc)[:200]}]
        try:
            cfg0 = config0_record(dev)
        except Exception as exc:
            cfg0 = {"error": repr(exc)[:200]}
    # ---- configs[2]: the same five matrices at 2..64 sequences per call (graph replay of the set, 1 GPU)
    sweep = []
    if rank == 0 and world == 1 and not args.only and M == 1:
        try:
            sweep = batch_sweep(dev, state, mats)
        except Exception as exc:
            sweep = [{"error": repr(exc)[:200]}]
    # ---- N > 1: where the step's time goes -- the five sharded GEMVs without their exchanges, and the two exchanges alone
    # (each a CUDA graph replayed 200 times between events, max over ranks), beside the whole step
    tp_break = None
    if world > 1 and coll is not None and use_graph:
        def timed_us(fn):
            fn()
            barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            for _ in range(3):
                g.replay()
            barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(200):
                g.replay()
            a1.record()
            barrier()
            t = torch.tensor([a0.elapsed_time(a1) / 200 * 1e3], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return round(float(t.item()), 2)

        def gemvs_only():
            for sh, W, sc, x, y in state:
                k.gemv_w4a8_f16in(y, x, W, sc, sh.k_local, sh.n_local, M)

        def exchanges_only():
            for sh, W, sc, x, y in state:
                if sh.kind == "k":
                    coll.finish(sh, y)

        try:
            tp_break = {"step_us": round(sec_per_step * 1e6, 2), "gemvs_without_exchange_us": timed_us(gemvs_only),
                        "exchanges_alone_us": timed_us(exchanges_only), "exchanges_per_step": sum(1 for st in state if st[0].kind == "k"),
                        "exchange": args.exchange}
        except Exception as exc:
            tp_break = {"error": repr(exc)[:300]}
    # ---- N > 1: the values behind the scaling curve -- a small tensor-parallel decode step against the single-GPU one
    tp_par = None
    if world > 1 and not args.only:
        try:
            tp_par = tp_parity(dev, world, rank)
        except Exception as exc:
            tp_par = {"error": repr(exc)[:300]}
    if world > 1:
        barrier()

    # ---- the synthetic Qwen3-8B-shape decode step (configs[3]): batch 1 and 8, context 2048, reported beside the
    # headline; tensor-parallel over all ranks when N > 1
    decode = []
    if not args.only and not args.no_decode:
        for b in (1, 8):
            try:
                decode.append(run_decode(shapes.QWEN3_8B, b, 2048, 20, dev, world, rank, exchange=args.exchange))
            except Exception as exc:  # the headline must survive a failure of the side measurement
                decode.append({"model": shapes.QWEN3_8B.name, "batch": b, "error": repr(exc)[:200]})
        if not args.no_decode32:
            # configs[4]: Qwen3-32B-shape, batch 64, context 4096, tensor-parallel over all ranks
            try:
                decode.append(run_decode(shapes.QWEN3_32B, 64, 4096, 5, dev, world, rank, exchange=args.exchange))
            except Exception as exc:
                decode.append({"model": shapes.QWEN3_32B.name, "batch": 64, "error": repr(exc)[:200]})
    # ---- decode attention on its own (1 GPU): the binary16-cache kernel of the decode step and the reference-format
    # fp32-cache entry point, each launch over another layer of a cache larger than L2
    attention = []
    if rank == 0 and world == 1 and not args.only and not args.no_decode:
        try:
            attention = attention_records(dev)
        except Exception as exc:
            attention = [{"error": repr(exc)[:200]}]
    if rank != 0:
        return
    peak, peak_kind = measured_peak()
    # dominant kernel: gemv_w4_stream_kernel<1, half>; every launch in the timed region is one of its launches
    n_launch = launches / args.steps
    per_launch_bytes = total_bytes / world / max(n_launch, 1)
    per_launch_s = sec_per_step / max(n_launch, 1)
    achieved = per_launch_bytes / per_launch_s / 1e9
    cpu = cpu_baseline_record() if world == 1 else None
    cfg = workload_config(world)
    cfg["bytes_per_step"] = total_bytes
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": sec_per_step * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": cfg,
        "launch": "cuda graph replay, one pass per graph" if use_graph else "host launches",
        "passes_per_step": passes, "timed_region_s": ms / 1e3,
        "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "schedule": "the caller's (this bench's), not the library's: all inputs go up first in one copy, the largest "
                            "matrix (LM head) is launched first and each result is copied back on a second stream "
                            "while the next matrix runs; the host synchronises once per pass"},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": int(per_launch_bytes * NCU_TRAFFIC_RATIO), "traffic_note": "ncu capture of a 65536-row slice, scaled by rows", "peak_kind": peak_kind,
                     "kernel": "w4_stream_kernel<1,half>", "nominal_frac": achieved / 8000.0},
        "cpu_baseline": cpu,
        "config0": cfg0,
        "per_matrix": per,
        "per_matrix_batched": per_batched,
        "batch_sweep": sweep,
        "tp_parity": tp_par,
        "tp_breakdown": tp_break,
        "attention": attention,
        "decode": decode,
    }
    print(json.dumps(line), flush=True)


def _graph_us(run, reps):
    """Median-of-3 time per call of run(i), i = 0..reps-1 captured in one CUDA graph."""
    import torch

    for i in range(min(reps, 3)):
        run(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(reps):
            run(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ts = []
    for _ in range(3):
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / reps * 1e3)
    return float(np.median(ts))


def per_matrix_times(dev, M, reference_arm=False):
    """Each matrix of the set on its own, L2-cold: a CUDA graph of 24 launches rotating over enough distinct
    weight copies to exceed twice the L2.  Our arm times the W4A8 kernel (fused f16 quantize) and our kernels in the
    reference's own format (quantize_int4 + gemv_int4_batched, W4A4, fp32 scales, LM head rows padded to a
    multiple of 16 as the reference requires).  The reference arm times the reference's own CUDA kernels, rebuilt
    unchanged for sm_100a (oracle/_ref), on the same shapes in that format: the GPU kernel to beat."""
    import torch

    from blackwell_b200 import synth
    have_ref = False
    if reference_arm:
        from oracle import ref_cuda

        have_ref = ref_cuda.available()
        if not have_ref:
            return None
    else:
        from blackwell_b200 import kernels as k
    peak, _ = measured_peak()
    out = []
    for i, (name, N, K) in enumerate(gemv_set()):
        Np = (N + 15) // 16 * 16
        ncopy = int(min(24, max(2, 300e6 // (Np * K * 0.5625) + 1)))
        Ws = [synth.int4_weights_device(Np, K, 700 + 31 * i + c, device=dev) for c in range(ncopy)]
        x16 = synth.activations_f16_device(M, K, 701 + i, device=dev)
        y = torch.empty((M, Np), dtype=torch.float32, device=dev)
        rec = {"name": name, "N": N, "K": K}
        if not reference_arm:
            us = _graph_us(lambda j: k.gemv_w4a8_f16in(y, x16, Ws[j % ncopy][0], Ws[j % ncopy][1], K, N, M), 24)
            b = shapes.gemv_bytes(N, K, M, 2, "f16")
            rec.update({"us": round(us, 2), "gbs": round(b / us / 1e3, 1), "frac": round(b / us / 1e3 / peak, 3)})
        if M <= 16:
            sc32 = [w[1].float() for w in Ws]
            x32 = x16.float()
            q = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
            s_ = torch.empty((M, K // 16), dtype=torch.float32, device=dev)
            lib = ref_cuda if reference_arm else k

            def chain(j):
                lib.quantize_int4_batched(q, s_, x32, K, M)
                lib.gemv_int4_batched(y, q, s_, Ws[j % ncopy][0], sc32[j % ncopy], K, Np, M)

            b4 = shapes.gemv_bytes(Np, K, M, 4, "i4")
            u = _graph_us(chain, 24)
            rec["w4a4_fp32scale"] = {"rows": Np, "us": round(u, 2), "gbs": round(b4 / u / 1e3, 1)}
            del sc32
        out.append(rec)
        del Ws
        torch.cuda.empty_cache()
    return out


def batch_sweep(dev, state, mats):
    """The five-matrix set at M = 2..64 sequences per call: one CUDA graph of the five launches per M, replayed;
    bytes = the set's algorithmic bytes at that M.  M <= 7 runs the dp4a kernel, M >= 8 the tcgen05 kernel."""
    import torch

    from blackwell_b200 import kernels as k
    from blackwell_b200 import synth

    peak, _ = measured_peak()
    out = []
    for m in (2, 4, 8, 16, 32, 64):
        xs = [synth.activations_f16_device(m, sh.k_local, 700 + i, device=dev) for i, (sh, *_r) in enumerate(state)]
        ys = [torch.empty((m, sh.n_local), dtype=torch.float32, device=dev) for sh, *_r in state]

        def step():
            for (sh, W, sc, _x, _y), x, y in zip(state, xs, ys):
                k.gemv_w4a8_f16in(y, x, W, sc, sh.k_local, sh.n_local, m)

        step()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 20
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / reps * 1e3
        nbytes = set_bytes(mats, m)
        rec = {"M": m, "us_per_step": round(us, 1), "gbs": round(nbytes / us / 1e3, 1),
               "roofline_frac": round(nbytes / us / 1e3 / peak, 3), "status": k.device_status()}
        if m >= 16:  # also against the dense int8 tensor-core roofline (2 M N K integer operations)
            tpeak, tkind = int8_tensor_peak_tops()
            tops = sum(2.0 * m * N * K for _, N, K in mats) / us / 1e6
            rec.update({"int8_tops": round(tops, 2), "tensor_roofline_frac": round(tops / tpeak, 5),
                        "tensor_peak_tops": tpeak, "tensor_peak_kind": tkind})
        out.append(rec)
        del g, xs, ys
    return out


def config0_record(dev):
    """BASELINE.json configs[0] as its own record: one 4096 x 4096 GEMV at M = 1 in the W4A8 format (fp16 activations
    quantized to int8 by the reference's rule), L2-cold graph replay over 30 weight copies; parity of the same launch
    against the CPU oracle (outputs against the float64 dequant-dot, per-block int32 dots bit for bit); and the host
    port's time for the same call, single-thread and all cores."""
    import torch

    import oracle
    from blackwell_b200 import kernels as k
    from blackwell_b200 import synth

    N = K = 4096
    peak, kind = measured_peak()
    ncopy = 30
    Ws = [synth.int4_weights_device(N, K, 9100 + c, device=dev) for c in range(ncopy)]
    x16 = synth.activations_f16_device(1, K, 9099, device=dev)
    y = torch.empty((1, N), dtype=torch.float32, device=dev)
    us = _graph_us(lambda j: k.gemv_w4a8_f16in(y, x16, Ws[j % ncopy][0], Ws[j % ncopy][1], K, N, 1), 60)
    nbytes = shapes.gemv_bytes(N, K, 1, 2, "f16")
    # parity on host-generated operands
    W, sc16, _ = synth.int4_weights(N, K, 9001)
    xh = synth.activations_f16(1, K, 9002)
    xq, xs = oracle.quantize_int8(xh.astype(np.float32))
    Wd = torch.from_numpy(W).to(dev)
    scd = torch.from_numpy(sc16.view(np.int16)).to(dev).view(torch.float16)
    k.gemv_w4a8_f16in(y, torch.from_numpy(xh.view(np.int16)).to(dev).view(torch.float16), Wd, scd, K, N, 1)
    ref = oracle.gemv_w4a8_f64(xq, xs, W, sc16)
    got = y.cpu().numpy().astype(np.float64)
    mar = float(np.max(np.abs(got - ref)) / np.max(np.abs(ref)))
    dots = torch.empty((N, K // 16), dtype=torch.int32, device=dev)
    k.gemv_block_dots(dots, torch.from_numpy(xq).to(dev), True, Wd, K, N)
    dots_equal = bool(np.array_equal(dots.cpu().numpy(), oracle.block_dots_w4a8(W, xq[0])))
    t0 = time.perf_counter(); oracle.gemv_w4a8_f32(xq, xs, W, sc16, 1); t1 = time.perf_counter()
    _, cores = oracle.gemv_w4a8_f32(xq, xs, W, sc16, 0)
    t2 = time.perf_counter(); oracle.gemv_w4a8_f32(xq, xs, W, sc16, 0); t3 = time.perf_counter()
    return {"workload": "single INT4 GEMV, M=1, K=4096, N=4096 (configs[0])", "us": round(us, 2),
            "gbs": round(nbytes / us / 1e3, 1), "frac": round(nbytes / us / 1e3 / peak, 3), "peak_kind": kind,
            "nominal_frac": round(nbytes / us / 1e3 / 8000.0, 3), "algorithmic_bytes": nbytes,
            "parity": {"max_abs_rel_vs_f64_oracle": mar, "block_dots_bit_exact": dots_equal},
            "cpu_port": {"single_thread_us": round((t1 - t0) * 1e6, 1), "all_core_us": round((t3 - t2) * 1e6, 1),
                         "cores": cores}}


def attention_records(dev):
    """Decode attention alone, L2-cold (a CUDA graph of 24 launches rotating over the layers of one cache): time,
    K/V bytes per second and the fraction of the measured HBM peak.  `f16` is the fused tensor-core form the decode
    step uses (head norm, RoPE, KV write and int8 output included), `f32` the reference-format entry point
    (attention_decode_batched_gqa_device: fp32 cache, scalar kernel)."""
    import torch

    from blackwell_b200 import kernels as k

    peak, _ = measured_peak()
    out = []
    for kind, M, nq, nkv, ctx, layers in [("f16", 1, 32, 8, 2048, 24), ("f16", 8, 32, 8, 2048, 12),
                                          ("f16", 64, 64, 8, 4096, 3), ("f32", 1, 32, 8, 2048, 24),
                                          ("f32", 8, 32, 8, 2048, 6)]:
        max_seq = ctx + 16
        kv_layer = nkv * max_seq * 128
        dt = torch.float16 if kind == "f16" else torch.float32
        kc = torch.randn((M, layers * kv_layer), device=dev, dtype=dt) * 0.5
        vc = torch.randn((M, layers * kv_layer), device=dev, dtype=dt) * 0.5
        pos = torch.full((M,), ctx - 1, device=dev, dtype=torch.int32)
        o = torch.empty((M, nq * 128), device=dev, dtype=torch.float32)
        if kind == "f16":
            qkv = torch.randn((M, (nq + 2 * nkv) * 128), device=dev, dtype=torch.float32)
            qn, kn = torch.ones(128, device=dev), torch.ones(128, device=dev)
            oq = torch.empty((M, nq * 128), device=dev, dtype=torch.int8)
            os_ = torch.empty((M, nq * 8), device=dev, dtype=torch.float32)
            us = _graph_us(lambda j: k.attention_decode_f16kv_fused_q8(
                None, oq, os_, qkv, qn, kn, kc, vc, pos, ctx, nq, nkv, 128, max_seq, M, layers * kv_layer,
                (j % layers) * kv_layer, 1e-6, 1e6), 24)
        else:
            q = torch.randn((M, nq * 128), device=dev, dtype=torch.float32)
            us = _graph_us(lambda j: k.attention_decode_batched_gqa_device(
                o, q, kc, vc, pos, nq, nkv, 128, max_seq, M, layers * kv_layer, (j % layers) * kv_layer), 24)
        nbytes = M * nkv * ctx * 128 * 2 * kc.element_size()
        out.append({"cache": kind, "batch": M, "heads": "%d/%d" % (nq, nkv), "ctx": ctx, "us": round(us, 2),
                    "kv_gbs": round(nbytes / us / 1e3, 1), "frac": round(nbytes / us / 1e3 / peak, 3)})
        del kc, vc
        torch.cuda.empty_cache()
    return out


def tp_parity(dev, world, rank):
    """One decode step of a small Qwen3-shaped model at TP-`world` against the same step on one GPU (rank 0 holds the
    full model beside its shard): every rank slices its shard out of the full matrices of one seed.  Batch 3 runs the
    dp4a streaming kernel, batch 16 the batched kernel.  Both exchanges are checked."""
    import torch
    import torch.distributed as dist

    from blackwell_b200.decode import DecodeEngine

    shape = shapes.ModelShape("tp-parity", layers=2, hidden=1024, inter=2048, n_q_heads=8, n_kv_heads=8, head_dim=128,
                              vocab=4099)
    out = {}
    for exchange in ("peer", "nccl"):
        for batch in (3, 16):
            ctx, max_seq = 70, 96
            eng = DecodeEngine(shape, batch, max_seq, dev, seed=41, world=world, rank=rank, exchange=exchange,
                               consistent=True)
            eng.fill_cache_consistent(ctx)
            toks = [(37 * i + 5) % shape.vocab for i in range(batch)]
            eng.set_tokens(toks)
            eng.step()
            torch.cuda.synchronize()
            # gather: logits slices (padded to the largest slice), hidden state and ids of every rank
            vmax = -(-shape.vocab // world)
            pad = torch.zeros((batch, vmax), dtype=torch.float32, device=dev)
            pad[:, :eng.v_local].copy_(eng.logits)
            allp = torch.empty((world, batch, vmax), dtype=torch.float32, device=dev)
            dist.all_gather_into_tensor(allp.view(-1), pad.view(-1))
            allx = torch.empty((world,) + tuple(eng.x.shape), dtype=torch.float32, device=dev)
            dist.all_gather_into_tensor(allx.view(-1), eng.x.contiguous().view(-1))
            allt = torch.empty((world, batch), dtype=torch.int32, device=dev)
            dist.all_gather_into_tensor(allt.view(-1), eng.tokens.view(-1))
            status = 0 if eng.peer is None else eng.peer.status()
            rec = None
            if rank == 0:
                v_base, v_rem = divmod(shape.vocab, world)
                parts = [allp[r, :, :v_base + (1 if r < v_rem else 0)] for r in range(world)]
                logits_tp = torch.cat(parts, dim=1)
                one = DecodeEngine(shape, batch, max_seq, dev, seed=41, world=1, rank=0, consistent=True)
                one.fill_cache_consistent(ctx)
                one.set_tokens(toks)
                one.step()
                torch.cuda.synchronize()
                a, b = logits_tp.double(), one.logits.double()
                rel = float((a - b).abs().max() / b.abs().max())
                # ids may only differ where the single-GPU top-2 margin is inside the numerical noise
                top2 = one.logits.topk(2, dim=1).values
                clear = (top2[:, 0] - top2[:, 1]) > 1e-3 * one.logits.abs().max()
                ids_equal = bool(torch.equal(allt[0][clear], one.tokens[clear]))
                per_seq = (a - b).abs().amax(dim=1) / b.abs().max()
                rec = {"logits_max_abs_rel": rel, "seqs_within_1e-5": int((per_seq < 1e-5).sum()), "seqs": batch,
                       "ids_equal": ids_equal,
                       "ranks_bit_identical": bool(all(torch.equal(allx[0], allx[r]) and torch.equal(allt[0], allt[r])
                                                       for r in range(1, world))),
                       "status": status}
                del one
            out["%s_b%d" % (exchange, batch)] = rec
            del eng
            torch.cuda.empty_cache()
            dist.barrier()
    if rank != 0:
        return None
    # The K-split sums add in another order than one GPU does, so a hidden state differs in its last bits; where
    # that moves one activation across a rounding tie of the int8 quantize, one sequence's logits move by a whole
    # quantization step of one input (seen: 2e-3 of the largest logit at two ranks, 4e-3 at eight, where one or two of
    # 16 sequences are touched).  Everything else agrees to fp32 rounding.
    out["ok"] = bool(all(v["logits_max_abs_rel"] < 1e-2 and v["seqs_within_1e-5"] >= v["seqs"] - max(1, v["seqs"] // 4)
                         and v["ids_equal"]
                         and v["ranks_bit_identical"] and v["status"] == 0 for v in out.values()))
    return out


def run_decode(shape, batch, ctx, steps, dev, world=1, rank=0, max_seq=None, exchange="peer"):
    """Times the synthetic decode step (one CUDA graph per step) with the cache pre-filled to ``ctx``; returns a
    dict with tokens/s over all sequences and the HBM roofline fraction of the step."""
    import torch

    from blackwell_b200.decode import DecodeEngine

    max_seq = max_seq or (ctx + 64)
    eng = DecodeEngine(shape, batch, max_seq, dev, seed=3, world=world, rank=rank, exchange=exchange)
    eng.fill_cache(ctx)
    gen = torch.Generator(device="cpu")
    gen.manual_seed(11)
    eng.set_tokens(torch.randint(0, shape.vocab, (batch,), generator=gen))
    eng.step()
    torch.cuda.synchronize()
    eng.pos.fill_(ctx - 1)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        eng.step()
    for _ in range(3):
        eng.pos.fill_(ctx - 1)
        graph.replay()
    torch.cuda.synchronize()
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(steps):
        eng.pos.fill_(ctx - 1)  # every timed step attends over the same context length
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ms = float(np.median(times))
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    peak, kind = measured_peak()
    nbytes = eng.step_bytes(ctx)  # per rank
    out = {"model": shape.name, "batch": batch, "ctx": ctx, "tp": world, "ms_per_step": round(ms, 4),
           "tok_s": round(batch / (ms / 1e3), 1), "hbm_bytes_per_step_per_gpu": nbytes,
           "gbs_per_gpu": round(nbytes / ms / 1e6, 1), "roofline_frac": round(nbytes / ms / 1e6 / peak, 3),
           "peak_kind": kind, "kv": "f16", "status": 0}
    from blackwell_b200 import kernels as k

    out["status"] = k.device_status()
    if world > 1:
        out["exchange"] = eng.exchange
        if eng.peer is not None and eng.peer.status() != 0:
            out["status"] = 3  # a peer all-reduce gave up waiting for another rank
    del eng, graph
    torch.cuda.empty_cache()
    return out


def run_attention_only(args):
    """The fp16-KV decode attention kernel alone on a synthetic cache (one layer, every sequence at position CTX - 1):
    the timed loop launches it args.steps times from the host; bytes = the K and V rows read."""
    import torch

    from blackwell_b200 import kernels as k

    b, ctx, nqh, nkv = (int(v) for v in args.attn_only.split(":"))
    hd = 128
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if args.tune:
        for kv in args.tune.split(","):
            key, _, val = kv.partition("=")
            k.set_tuning(int(key), int(val))
    g = torch.Generator(device="cuda").manual_seed(0xB2000005)
    kv_batch = nkv * ctx * hd
    kc = torch.randn((b, kv_batch), generator=g, device=dev, dtype=torch.float16)
    vc = torch.randn((b, kv_batch), generator=g, device=dev, dtype=torch.float16)
    q = torch.randn((b, nqh * hd), generator=g, device=dev, dtype=torch.float32)
    out = torch.empty_like(q)
    pos = torch.full((b,), ctx - 1, device=dev, dtype=torch.int32)
    launch = lambda: k.attention_decode_f16kv(out, q, kc, vc, pos, ctx, nqh, nkv, hd, ctx, b, kv_batch, 0)
    for _ in range(max(args.warmup, 1)):
        launch()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        launch()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / args.steps * 1e3
    nbytes = 2 * b * kv_batch * 2
    return {"kernel": "attention_decode_f16kv", "batch": b, "ctx": ctx, "q_heads": nqh, "kv_heads": nkv,
            "us_per_launch": us, "kv_bytes": nbytes, "gbs": nbytes / us / 1e3, "device_status": k.device_status()}


def run_timeline(args):
    """Diagnostic, needs a library built with -DBW_GEMV_TIMELINE (BW_NVCC_EXTRA=-DBW_GEMV_TIMELINE python -m
    blackwell_b200._build -f): the small-batch GEMV kernel then stamps %globaltimer at its phase borders for its first,
    middle and last CTA.  24 launches of one matrix (NAME[:fmt], fmt = f16 or i8 activations) rotate over 24 weight
    copies in one CUDA graph; prints the mean phase durations of CTA 0 and the launch period."""
    import ctypes as C

    import torch

    from blackwell_b200 import _lib
    from blackwell_b200 import kernels as k
    from blackwell_b200 import synth

    L = _lib.load()
    if not hasattr(L, "bw_debug_set_timeline"):
        raise SystemExit("the library was built without -DBW_GEMV_TIMELINE")
    name, _, fmt = args.timeline.partition(":")
    fmt = fmt or "f16"
    N, K = next((n, kk) for nm, n, kk in shapes.QWEN3_8B.gemv_set() if nm == name)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    tl = torch.zeros(16 + 32 * 48, dtype=torch.int64, device=dev)
    L.bw_debug_set_timeline(C.c_void_p(tl.data_ptr()))
    ncopy = 24
    Ws = [synth.int4_weights_device(N, K, 700 + c, device=dev) for c in range(ncopy)]
    x16 = synth.activations_f16_device(1, K, 701, device=dev)
    xq = torch.empty((1, K), dtype=torch.int8, device=dev)
    xs = torch.empty((1, K // 16), dtype=torch.float32, device=dev)
    k.quantize_int8_f16(xq, xs, x16, K)
    y = torch.empty((1, N), dtype=torch.float32, device=dev)
    if fmt == "f16":
        run = lambda j: k.gemv_w4a8_f16in(y, x16, Ws[j % ncopy][0], Ws[j % ncopy][1], K, N, 1)
    else:
        run = lambda j: k.gemv_w4a8(y, xq, xs, Ws[j % ncopy][0], Ws[j % ncopy][1], K, N, 1)
    for j in range(3):
        run(j)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for j in range(24):
            run(j)
    g.replay()
    torch.cuda.synchronize()
    tl.zero_()
    g.replay()
    torch.cuda.synchronize()
    rec = tl.cpu().numpy()[16:].reshape(32, 3, 16)[4:24, 0, :7].astype(np.int64)
    phases = np.diff(rec, axis=1).mean(0)
    names = ["start->copies issued", "->dependency wait returns", "->activation prologue done", "->first tile landed",
             "->first tile computed", "->end"]
    return {"matrix": name, "N": N, "K": K, "activations": fmt,
            "phase_ns": {n: round(float(v)) for n, v in zip(names, phases)},
            "launch_period_ns": round(float(np.diff(rec[:, 0]).mean()))}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from the host instead of replaying "
                    "a captured CUDA graph")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode-step side measurement")
    ap.add_argument("--no-decode32", action="store_true", help="skip the 32B-shape decode side measurement")
    ap.add_argument("--decode-only", default=None, help="profiling aid: only the decode step, MODEL:BATCH:CTX "
                    "(MODEL = 8b or 32b); prints its own JSON line")
    ap.add_argument("--batch", type=int, default=1, help="profiling aid: sequences per GEMV (the headline is 1)")
    ap.add_argument("--only", default=None, help="profiling aid: run one matrix of the set, NAME or NAME:ROWS")
    ap.add_argument("--attn-only", default=None, help="profiling aid: only the fp16-KV GQA decode attention kernel, "
                    "BATCH:CTX:NQH:NKV on a synthetic cache; prints its own JSON line")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="N > 1: how the K-split partial sums "
                    "are summed across ranks (library NVLink peer-load all-reduce, or NCCL)")
    ap.add_argument("--min-time", type=float, default=MIN_TIMED_SECONDS, help="shortest timed region in seconds (each "
                    "step is timed as the mean of as many passes as that needs); 0 for profiling runs")
    ap.add_argument("--timeline", default=None, help="diagnostic: per-phase timeline of the small-batch kernel on one "
                    "matrix of the set, NAME[:f16|i8]; needs a library built with -DBW_GEMV_TIMELINE")
    ap.add_argument("--tune", default=None, help="profiling aid: comma list of key=value for bw_set_tuning")
    args = ap.parse_args()
    global _ONLY
    if args.only:
        nm, _, n = args.only.partition(":")
        _ONLY = (nm, int(n) if n else None)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        # torchrun exports OMP_NUM_THREADS=1 to every rank; the reference arm is one process that should use every host
        # core (the variable is read when the oracle's OpenMP runtime starts, which has not happened yet)
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
        run_reference(args, rank)
        return
    if args.attn_only:
        print(json.dumps(run_attention_only(args)), flush=True)
        return
    if args.timeline:
        print(json.dumps(run_timeline(args)), flush=True)
        return
    if args.decode_only:
        import torch

        if args.tune:
            from blackwell_b200 import kernels as k

            for kv in args.tune.split(","):
                key, _, val = kv.partition("=")
                k.set_tuning(int(key), int(val))
        model, b, c = args.decode_only.split(":")
        if world > 1:
            import torch.distributed as dist

            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        torch.cuda.set_device(local_rank)
        shape = shapes.QWEN3_8B if model == "8b" else shapes.QWEN3_32B
        out = run_decode(shape, int(b), int(c), args.steps, torch.device("cuda", local_rank), world, rank,
                         exchange=args.exchange)
        if rank == 0:
            print(json.dumps(out), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    if world > 1:
        import torch
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()
