#!/usr/bin/env python
"""Benchmark of the quantization hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (benchmark configuration 2): INT4 g=32 weight-only decode, W[11008,4096] stored [N,K],
X[1,4096] fp32, y = x * deq(W)^T.  One *step* = `--launches-per-step` forwards cycling through
`--copies` distinct weight sets (10 x 28.2 MB = 282 MB > 126 MB L2, so every launch streams its
weights from HBM).  Metric: achieved HBM GB/s = algorithmic bytes / time, whole job.

N > 1 (torchrun): weak scaling of a column-sharded layer — every rank holds its own
[11008,4096] column slice (N_total = 11008 * ranks) and the full-width output is assembled on every
rank per forward: the decode kernel stores its [M, 11008] slice into all ranks' outputs over NVLink
peer mappings and signals; the next forward's kernel waits for all ranks' signals in its prologue
(one NVLink round trip, no extra launch; one barrier kernel ends each step).  `--nccl`: local forward
+ NCCL all-gather + interleave instead.  value = bytes streamed by all ranks / max-over-ranks device
time.  Before anything is timed the gathered output of one forward is compared, bit for bit, with the
NCCL all-gather of the single-GPU results of the slices ("sharded_check").  `extra` then carries the
column-sharded configurations: W[28672,8192] split over the ranks (strong scaling; M = 1 and 16 on the
decode kernel, M = 128, 1024 and 8192 on the tensor cores; the kernels' epilogues store into every rank's output)
and the NanoLLaMA-INT4 generation with every linear split over the ranks.

`--impl reference` times the reference's own CPU QuantizedLinear forward (oracle/_ref, the
unmodified sources compiled for the host) on the same workload: one forward per step.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

K_DIM, N_DIM, GROUP = 4096, 11008, 32
METRIC, UNIT = "int4_g32_decode_gemv_hbm_gbs", "GB/s"


def ncu_traffic(kernel: str, m: int):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of `kernel` at batch m, as recorded by the
    committed profiler summaries: a line `traffic_bytes_per_launch <kernel> M=<m>: <bytes>` in a file of the
    profiles directory.  None when there is no such record."""
    import glob
    import re
    pat = re.compile(r"traffic_bytes_per_launch\s+" + re.escape(kernel) + r"\s+M=" + str(m) + r":\s*([0-9.eE+]+)")
    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", "*"))):
        try:
            with open(path) as f:
                hit = pat.search(f.read())
        except OSError:
            continue
        if hit:
            return float(hit.group(1))
    return None


def gemv_bytes(M: int, K: int = K_DIM, N: int = N_DIM, bits: int = 4) -> int:
    """Algorithmic bytes of one forward: packed weights + scales + x + y (fp32)."""
    w = N * K // 2 + (N * K // GROUP) * 4 if bits == 4 else N * K + 4
    return w + M * K * 4 + M * N * 4


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, period_ms: int = 50):
        self.lines, self.proc, self.thread = [], None, None
        self.cmd = ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                    "-lms", str(period_ms)]

    def start(self):
        try:
            self.proc = subprocess.Popen(self.cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True)
        self.thread.start()

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.06)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in self.lines:
            p = [s.strip() for s in l.split(",")]
            if len(p) < 7:
                continue
            try:
                sm.append(float(p[0]))
                smax.append(float(p[1]))
            except ValueError:
                continue
            for name, v in zip(names, p[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# ------------------------------------------------------------------------------------------
# reference arm: the reference's CPU implementation on the host cores
# ------------------------------------------------------------------------------------------
def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def reference_linear(M: int, native_kn: bool = False):
    """A timer for the reference's own CPU forward on all host cores.  Default: the weight as this benchmark
    stores it, W[N,K] (the reference needs dequantize + transpose + matmul for it); native_kn: the reference
    module's own layout W[K,N] (dequantize + matmul, src/quantization.cpp:199-206)."""
    import numpy as np
    import oracle
    ref = oracle.load_ref()
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((N_DIM, K_DIM)) * 0.02).astype(np.float32)
    x = rng.standard_normal((M, K_DIM)).astype(np.float32)
    if ref is not None:
        ref.set_num_threads(host_cores())          # a launcher may have exported OMP_NUM_THREADS=1
        if native_kn:
            lin = ref.linear(np.ascontiguousarray(w.T), oracle.LAYOUT_KN, 4, 0, GROUP, None)
        else:
            lin = ref.linear(w, oracle.LAYOUT_NK, 4, 0, GROUP, None)
        return "reference", ref.num_threads(), (lambda iters: lin.time_forward(x, iters, with_bias=False))
    if native_kn:
        raise RuntimeError("the compiled reference is not available")
    port = oracle.Port()                                   # the reference was never compiled here
    packed, scales = port.quantize_int4(w, GROUP)

    def run(iters):
        t0 = time.perf_counter()
        for _ in range(iters):
            port.qlinear_int4(x, packed, scales, K_DIM, N_DIM, oracle.LAYOUT_NK, GROUP, None)
        return (time.perf_counter() - t0) / iters
    return "port", host_cores(), run


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    kind, cores, timer = reference_linear(1)
    for _ in range(min(args.warmup, 3)):
        timer(1)
    t0 = time.perf_counter()
    per = timer(args.steps)
    wall = time.perf_counter() - t0
    value = gemv_bytes(1) / per / 1e9
    native = None
    try:
        _, _, timer_kn = reference_linear(1, native_kn=True)
        timer_kn(1)
        per_kn = timer_kn(max(2, min(args.steps, 10)))
        native = {"value": gemv_bytes(1) / per_kn / 1e9, "unit": UNIT, "ms_per_forward": per_kn * 1e3,
                  "what": "the same weight in the reference module's own [K,N] layout: dequantize + matmul, no transpose"}
    except Exception as e:  # noqa: BLE001
        native = {"error": f"{type(e).__name__}: {e}"[:200]}
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config2: INT4 g=32 decode, W[11008,4096] ([N,K]), X[1,4096]; one CPU forward "
                               "(dequantize + fp32 matmul, as the reference does per call) per step",
                   "M": 1, "K": K_DIM, "N": N_DIM, "group": GROUP},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": f"{args.steps} forwards of the full workload, {wall:.1f} s", "native_layout_kn": native},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
def make_graph(torch, body):
    """Captures body() (which enqueues launches on the current stream) into a CUDA graph, so that a
    replay issues them back to back without per-launch host work (a decode forward lasts ~5 us,
    less than one Python call)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        body()                                  # eager once: lazy module loading, attribute set-up
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        body()
    return graph


def time_launches(torch, fn, iters: int, inner: int = 20, warm: int = 2) -> float:
    """Average device milliseconds of one fn() call: `inner` calls per graph, `iters` replays,
    CUDA events on the launching stream."""
    graph = make_graph(torch, lambda: [fn() for _ in range(inner)])
    for _ in range(warm):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (iters * inner)


def eager_time(torch, fn, iters: int) -> float:
    """A few eager launches (profiling runs: a handful of kernels, no graph)."""
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def extras(torch, sgq, peaks, copies_w, only=None, eager=False):
    """Secondary measurements (reported, not the headline): other batch sizes, the pack kernels and
    the prefill GEMM of benchmark configuration 3."""
    out = {}
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1)

    timer = (lambda fn, iters, inner=20: eager_time(torch, fn, 3)) if eager else (lambda fn, iters, inner=20: time_launches(torch, fn, iters, inner))

    def guard(name, f):
        if only and name != only:
            return
        try:
            out[name] = f()
        except Exception as e:  # noqa: BLE001
            out[name] = {"error": f"{type(e).__name__}: {e}"[:200]}

    def gemv(M, path):
        x = torch.randn(M, K_DIM, device=dev, generator=g)
        y = torch.empty(M, N_DIM, device=dev)
        ws = sgq.Workspace(dev)
        state = {"i": 0}

        def f():
            q = copies_w[state["i"] % len(copies_w)]
            state["i"] += 1
            sgq.quantized_matmul(x, q, None, layout=sgq.LAYOUT_NK, path=path, out=y, workspace=ws)
        ms = timer(f, 20, inner=100)
        gbs = gemv_bytes(M) / ms / 1e6
        return {"ms": ms, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "path": sgq.PATH_NAMES[path]}

    for M in (1, 4, 8):
        guard(f"gemv_M{M}", lambda M=M: gemv(M, sgq.PATH_GEMV))
    guard("gemv_M16_auto", lambda: gemv(16, sgq.PATH_AUTO))
    guard("gemv_M1_simt", lambda: gemv(1, sgq.PATH_SIMT))

    def gemv_int8(M, N, K):
        # one 235 MB weight (config 5 shape) is larger than L2 by itself
        w = torch.randn(N, K, device=dev, generator=g) * 0.02
        q = sgq.quantize_int8(w, sgq.PER_TENSOR)
        del w
        x = torch.randn(M, K, device=dev, generator=g)
        y = torch.empty(M, N, device=dev)
        ws = sgq.Workspace(dev)
        f = lambda: sgq.quantized_matmul(x, q, None, layout=sgq.LAYOUT_NK, path=sgq.PATH_GEMV, out=y, workspace=ws)  # noqa: E731
        ms = timer(f, 10, inner=10)
        nbytes = N * K + 4 + M * K * 4 + M * N * 4
        return {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_measured_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"],
                "path": "gemv (int8 codes x int8 activation digits -> s32)", "launches_per_forward": 2}

    for M in (1, 16):
        guard(f"gemv_int8_tensor_M{M}_28672x8192", lambda M=M: gemv_int8(M, 28672, 8192))

    def gemv_int4_large(M, N, K):
        # config 5 shape: 147 MB of packed codes + scales, larger than L2 by itself
        w = torch.randn(N, K, device=dev, generator=g) * 0.02
        q = sgq.quantize_int4(w, GROUP)
        del w
        x = torch.randn(M, K, device=dev, generator=g)
        y = torch.empty(M, N, device=dev)
        ws = sgq.Workspace(dev)
        f = lambda: sgq.quantized_matmul(x, q, None, layout=sgq.LAYOUT_NK, path=sgq.PATH_GEMV, out=y, workspace=ws)  # noqa: E731
        ms = timer(f, 10, inner=10)
        nbytes = gemv_bytes(M, K, N)
        return {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_measured_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"], "path": "gemv"}

    for M in (1, 16):
        guard(f"gemv_int4_g32_M{M}_28672x8192", lambda M=M: gemv_int4_large(M, 28672, 8192))

    def pack(shape, bits):
        # two inputs > L2 in total for the big shape; alternate so the small one also misses L2
        ws_ = [torch.randn(shape, device=dev, generator=g) * 0.02 for _ in range(3)]
        n = ws_[0].numel()
        state = {"i": 0}

        def f():
            w = ws_[state["i"] % 3]
            state["i"] += 1
            return sgq.quantize_int4(w, GROUP) if bits == 4 else sgq.quantize_int8(w, sgq.PER_TENSOR)
        ms = timer(f, 10, inner=6)
        algo = 4.625 * n if bits == 4 else 5.0 * n
        return {"ms": ms, "gbs_algorithmic": algo / ms / 1e6, "bytes_per_element": 4.625 if bits == 4 else 5.0,
                "frac_of_measured_hbm": algo / ms / 1e6 / peaks["hbm_gbs"]}

    for shape in ((4096, 4096), (11008, 4096)):
        guard(f"pack_int4_g32_{shape[0]}x{shape[1]}", lambda s=shape: pack(s, 4))
        guard(f"pack_int8_tensor_{shape[0]}x{shape[1]}", lambda s=shape: pack(s, 8))

    def gemm(N, path, bits=None, layout=None, M=2048, K=4096):
        layout = sgq.LAYOUT_NK if layout is None else layout
        x = torch.randn(M, K, device=dev, generator=g)
        w = torch.randn((N, K) if layout == sgq.LAYOUT_NK else (K, N), device=dev, generator=g) * 0.02
        bits = bits or (8 if path == sgq.PATH_TC_I8 else 4)
        q = sgq.quantize_int4(w, GROUP) if bits == 4 else sgq.quantize_int8(w, sgq.PER_TENSOR)
        y = torch.empty(M, N, device=dev)
        ws = sgq.Workspace(dev)
        f = lambda: sgq.quantized_matmul(x, q, None, layout=layout, path=path, out=y, workspace=ws)  # noqa: E731
        ms = timer(f, 5, inner=4)
        tf = 2.0 * M * N * K / ms / 1e9
        return {"ms": ms, "tflops": tf, "frac_of_measured_bf16_burst": tf / peaks["bf16_tflops"],
                "frac_of_nominal_bf16_2250": tf / 2250.0, "path": sgq.PATH_NAMES[path],
                "includes": "activation conversion/quantization kernel + GEMM"
                            + (" + per-forward expansion of the [K,N] weight to bf16 [N,K]" if layout == sgq.LAYOUT_KN else "")}

    def int8_tensor_peak():
        # Denominator for the W8A8 lines: the vendor library's int8 x int8 -> int32 GEMM (cuBLASLt through
        # torch._int_mm) on 8192^3, timed the same way; a library call used only as a measured peak.
        n = 8192
        a = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8)
        b = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8).t()
        f = lambda: torch._int_mm(a, b)  # noqa: E731
        ms = timer(f, 5, inner=4)
        return {"ms": ms, "tops": 2.0 * n ** 3 / ms / 1e9, "what": "torch._int_mm (cuBLASLt s8*s8->s32), 8192^3"}

    guard("int8_tensor_peak_measured", int8_tensor_peak)
    i8_peak = (out.get("int8_tensor_peak_measured") or {}).get("tops")

    for N in (4096, 11008):
        guard(f"prefill_bf16_2048x4096x{N}", lambda N=N: gemm(N, sgq.PATH_TC_BF16))
        guard(f"prefill_bf16_int8w_2048x4096x{N}", lambda N=N: gemm(N, sgq.PATH_TC_BF16, bits=8))
        guard(f"prefill_i8_2048x4096x{N}", lambda N=N: gemm(N, sgq.PATH_TC_I8))
        guard(f"prefill_bf16_layout_kn_2048x4096x{N}", lambda N=N: gemm(N, sgq.PATH_TC_BF16, layout=sgq.LAYOUT_KN))
        r = out.get(f"prefill_i8_2048x4096x{N}")
        if i8_peak and r and "tflops" in r:
            r["frac_of_measured_int8"] = r["tflops"] / i8_peak
    # configuration 5's batch sweep on the tensor cores (M = 1 and 16 are the decode lines above); the largest is
    # 3.85 TFLOP per forward with a 470 MB expanded weight
    for M5 in (128, 1024, 8192):
        guard(f"prefill_bf16_{M5}x8192x28672", lambda M5=M5: gemm(28672, sgq.PATH_TC_BF16, M=M5, K=8192))
    status = sgq.device_status()
    out["device_status_word"] = status
    return out


def sharded_extras(torch, sgq, sh, dist, dev, rank: int, world: int, peaks):
    """N > 1: the column-sharded configurations.  W[28672,8192] (benchmark configuration 5) split by rows over
    the ranks (strong scaling: the same total work at every N), M = 1 and 16, full-width output assembled on
    every rank per forward by the fused exchange; and the NanoLLaMA-INT4 generation (configuration 4) with every
    linear split over the ranks.  Every rank takes part; times are the maximum over the ranks."""
    out = {}
    N, K = 28672, 8192
    n0, n1 = sh.shard_bounds(N, world, rank)
    g = torch.Generator(device=dev).manual_seed(99 + rank)
    slice_bytes = (n1 - n0) * K // 2 + (n1 - n0) * K // GROUP * 4
    copies = max(2, min(12, int(300e6 // slice_bytes) + 1))          # rotate so that every forward streams from HBM
    qs = [sgq.quantize_int4(torch.randn(n1 - n0, K, device=dev, generator=g) * 0.02, GROUP) for _ in range(copies)]
    for M in (1, 16):
        try:
            ex = sh.PeerExchange(M, N, dev)
            lins = [sh.PeerShardedLinear(q, None, N, ex, deferred=True) for q in qs]
            x = torch.randn(M, K, device=dev, generator=g)
            inner = 48
            graph = make_graph(torch, lambda: ([lins[i % copies](x) for i in range(inner)], ex.barrier()))
            for _ in range(2):
                graph.replay()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            us = float(t.item()) / (10 * inner) * 1e3
            nbytes = gemv_bytes(M, K, N)
            out[f"sharded_int4_g32_M{M}_28672x8192"] = {
                "us_per_forward": us, "aggregate_gbs": nbytes / us / 1e3, "n_local": n1 - n0, "weight_copies": copies,
                "frac_of_measured_hbm_all_gpus": nbytes / us / 1e3 / (world * peaks["hbm_gbs"]), "scaling": "strong",
                "exchange": "peer stores from the decode kernel, wait in the next forward's prologue"}
            del ex, lins, graph
        except Exception as e:  # noqa: BLE001
            out[f"sharded_int4_g32_M{M}_28672x8192"] = {"error": f"{type(e).__name__}: {e}"[:300]}
        torch.cuda.synchronize()
        dist.barrier()
    # the prefill sizes of the same sweep: every rank runs its slice on the tensor cores and the GEMM's epilogue
    # stores the tiles into every rank's full-width output; a barrier kernel ends each forward (eager launches,
    # CUDA events, max over ranks)
    for M in (128, 1024, 8192):
        try:
            ex = sh.PeerExchange(M, N, dev, n_buffers=1)
            lin = sh.PeerShardedLinear(qs[0], None, N, ex)
            x = torch.randn(M, K, device=dev, generator=g)
            for _ in range(3):
                lin(x)
            torch.cuda.synchronize()
            dist.barrier()
            reps = 5
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                lin(x)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item()) / reps
            tf = 2.0 * M * N * K / ms / 1e9
            out[f"sharded_prefill_bf16_{M}x8192x28672"] = {
                "ms": ms, "tflops_all_gpus": tf, "frac_of_measured_bf16_burst_all_gpus": tf / (world * peaks["bf16_tflops"]),
                "n_local": n1 - n0, "scaling": "strong", "exchange": "peer stores from the GEMM's epilogue + barrier kernel"}
            del lin, x, ex
        except Exception as e:  # noqa: BLE001
            out[f"sharded_prefill_bf16_{M}x8192x28672"] = {"error": f"{type(e).__name__}: {e}"[:300]}
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.empty_cache()
    del qs
    torch.cuda.empty_cache()
    try:
        out["nanollama_int4_config4_sharded"] = nanollama_case(torch, sgq, dev, reps=2, warm=1, rank=rank, world=world, dist=dist)
    except Exception as e:  # noqa: BLE001
        out["nanollama_int4_config4_sharded"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    return out


def nanollama_case(torch, sgq, dev, *, reps: int, warm: int, rank: int = 0, world: int = 1, dist=None,
                   batch: int = 8, prompt_len: int = 512, n_new: int = 128):
    """benchmark configuration 4: NanoLLaMA-INT4 (dim 2048, 16 blocks, 16 heads, SwiGLU 5632, vocab 32000,
    random init), batch 8, uniform random token ids, 512-token prefill + 128 greedy decode steps.
    One generation = prefill (tcgen05 bf16 path) + first token + 127 decode steps (decode kernel, one
    CUDA graph replay per step on one GPU; eager with NCCL all-gathers when column-sharded).
    The prompt comes from pinned host memory and the generated tokens go back to it inside the
    timed region, so every figure here is end to end."""
    import importlib
    nl = importlib.import_module("sgq_b200.nanollama")
    cfg = nl.NanoLlamaConfig()
    model = nl.NanoLlamaInt4(cfg, dev, batch, seed=1234, rank=rank, world=world)
    gen = torch.Generator().manual_seed(4321)
    prompt_h = torch.randint(0, cfg.vocab, (batch, prompt_len), generator=gen).pin_memory()
    prompt_d = torch.empty(batch, prompt_len, dtype=torch.int64, device=dev)
    out_h = torch.empty(batch, n_new, dtype=torch.int64).pin_memory()
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    t_prefill = t_decode = t_total = 0.0
    first = None
    for it in range(warm + reps):
        if dist:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1, e2 = ev(), ev(), ev()
        e0.record()
        prompt_d.copy_(prompt_h, non_blocking=True)
        logits = model.prefill(prompt_d)
        toks = torch.empty(batch, n_new, dtype=torch.int64, device=dev)
        model._argmax(logits)
        toks[:, 0].copy_(model.tok)
        if model._graph is None:
            model.capture_decode_graph()          # first (warm-up) generation only
        e1.record()
        for s in range(1, n_new):
            model._graph.replay()
            toks[:, s].copy_(model.tok)
        out_h.copy_(toks, non_blocking=True)
        e2.record()
        torch.cuda.synchronize()
        if first is None:
            first = out_h.clone()
        elif not torch.equal(first, out_h):
            raise RuntimeError("greedy generation is not reproducible from run to run")
        if it >= warm:
            tp, td = e0.elapsed_time(e1), e1.elapsed_time(e2)
            if dist:
                t = torch.tensor([tp, td], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                tp, td = float(t[0]), float(t[1])
            t_prefill += tp
            t_decode += td
            t_total += tp + td
    status = sgq.device_status()
    n_lin = 4 * cfg.n_layers + 1
    w_bytes = sum(2 * (q.q.qdata.numel() + 4 * q.q.scales.numel()) // 2 for L in model.layers for q in (L["qkv"], L["wo"], L["gu"], L["down"]))
    w_bytes += model.lm_head.q.qdata.numel() + 4 * model.lm_head.q.scales.numel()
    return {
        "tokens_per_s_decode": batch * (n_new - 1) * reps / (t_decode * 1e-3),
        "tokens_per_s_prefill": batch * prompt_len * reps / (t_prefill * 1e-3),
        "tokens_per_s_generation": batch * n_new * reps / (t_total * 1e-3),
        "ms_prefill": t_prefill / reps, "us_per_decode_step": t_decode / reps / (n_new - 1) * 1e3,
        "ms_per_generation": t_total / reps, "launches_per_decode_step": model.launches_per_decode_step,
        "quantized_linears_per_step": n_lin, "packed_weight_bytes_per_gpu": int(w_bytes),
        "weight_stream_gbs_decode": w_bytes * (n_new - 1) * reps / (t_decode * 1e-3) / 1e9,
        "h2d_bytes": batch * prompt_len * 8, "d2h_bytes": batch * n_new * 8, "device_status_word": status,
        "batch": batch, "prompt_len": prompt_len, "new_tokens": n_new, "kv_cache": "fp32",
        "prefill_path": "tc_bf16 (auto)", "decode_path": "gemv (auto)",
        "launch": "one CUDA graph replay per decode step" + ("" if world == 1 else "; column slices exchanged by peer stores from this "
                  "library's kernels + a barrier kernel per exchange (4 per block + logits), NCCL only in the prompt pass"),
    }


def run_nanollama(args):
    """`--workload nanollama`: the config-4 line (tokens/s), 1 GPU or column-sharded over the ranks."""
    import torch
    from __graft_entry__ import load_package
    sgq = load_package()
    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    r = nanollama_case(torch, sgq, dev, reps=max(1, args.steps), warm=max(1, args.warmup), rank=rank, world=world, dist=dist)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        line = {"metric": "nanollama_int4_generation_tokens_per_s", "value": r["tokens_per_s_generation"], "unit": "tokens/s",
                "n_gpus": world, "steps": max(1, args.steps), "warmup": max(1, args.warmup), "ms_per_step": r["ms_per_generation"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "INT4 g=32 weights; bf16 x bf16 -> fp32 prefill, u8 x s8 -> s32 decode; fp32 everything else",
                "data": "synthetic",
                "config": {"workload": "config4: NanoLLaMA-INT4 dim 2048, 16 blocks, 16 heads, SwiGLU 5632, vocab 32000; batch 8, "
                                       "512-token prefill + 128 greedy decode steps"
                                       + (f"; every linear column-sharded over {world} GPUs" if world > 1 else ""),
                           "l2": "packed weights + KV cache (1.8 GB) > 126 MB L2", "step": "one whole generation"},
                "e2e": {"value": r["tokens_per_s_generation"], "unit": "tokens/s", "h2d_bytes_per_step": r["h2d_bytes"],
                        "d2h_bytes_per_step": r["d2h_bytes"]},
                "gpu_launches": r["launches_per_decode_step"] * 127 * max(1, args.steps), "clocks": clocks, "detail": r}
        print(json.dumps(line), flush=True)
    if dist:
        dist.destroy_process_group()


def run_ours(args):
    import torch
    from __graft_entry__ import load_package
    sgq = load_package()
    rank, local_rank, world = dist_env()
    if world != args.gpus and world > 1:
        args.gpus = world
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    peaks = measured_peaks()
    sgq.set_stream_overlap(0 if args.no_overlap else args.overlap_mode)     # consecutive forwards overlap their prologue and first weight tiles
    M, copies, lps = args.M, args.copies, args.launches_per_step
    if args.only:
        # profiling aid: run one secondary case a few times, eagerly, and print it
        g0 = torch.Generator(device=dev).manual_seed(1234)
        ws0 = [sgq.quantize_int4(torch.randn(N_DIM, K_DIM, device=dev, generator=g0) * 0.02, GROUP) for _ in range(copies)]
        print(json.dumps({"only": args.only, **extras(torch, sgq, peaks, ws0, only=args.only, eager=not args.only_graph)}), flush=True)
        return

    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    weights = []
    for _ in range(copies):
        w = torch.randn(N_DIM, K_DIM, device=dev, generator=g) * 0.02
        weights.append(sgq.quantize_int4(w, GROUP))
        del w
    x = torch.randn(M, K_DIM, device=dev, generator=g)
    y_local = torch.empty(M, N_DIM, device=dev)
    ws = sgq.Workspace(dev)
    path = sgq.PATH_GEMV if M <= 16 else sgq.PATH_AUTO
    sharded = None
    if world > 1:
        import importlib
        sh = importlib.import_module("sgq_b200.sharding")
        exchange = None
        if not (args.nccl or M > 16):
            # fused all-gather: the decode kernel stores its slice into every rank's output (peer stores), then one
            # barrier kernel; two alternating output sets, shared by all layers of this shape
            ok = torch.ones(1, device=dev)
            try:
                exchange = sh.PeerExchange(M, world * N_DIM, dev)
            except Exception as e:  # noqa: BLE001  (no peer mapping on this box: every rank falls back together)
                sys.stderr.write(f"[bench] rank {rank}: peer exchange unavailable ({type(e).__name__}: {e}); using NCCL\n")
                ok.zero_()
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if float(ok.item()) == 0.0:
                exchange, args.nccl = None, True
        if exchange is None:
            # one column-sharded layer per weight set: local slice through the C ABI, NCCL all-gather, interleave
            args.nccl = True
            sharded = [sh.cuda_sharded_linear(q, None, world * N_DIM, path=path) for q in weights]
        else:
            # deferred exchange: a forward stores its slices into every rank's output and signals; the NEXT forward
            # waits for all ranks in its prologue (one NVLink round trip, no second launch)
            sharded = [sh.PeerShardedLinear(q, None, world * N_DIM, exchange, deferred=True) for q in weights]
    if world > 1 and args.nccl and lps > 200:
        lps = 200                   # eager NCCL launches: keep a step short
    last = {}

    def forward(i):
        if sharded:
            last["y"] = sharded[i % copies](x)          # every layer writes the same [M, world*N] output buffer shape
        else:
            sgq.quantized_matmul(x, weights[i % copies], None, layout=sgq.LAYOUT_NK, path=path, out=y_local, workspace=ws)

    def drain():
        """Ends a sequence of deferred exchanges: after this barrier the last outputs are whole on every rank."""
        if sharded and exchange is not None:
            exchange.barrier()

    # ---- N > 1: the gathered output must equal the single-GPU results of the slices, bit for bit
    sharded_check = None
    if world > 1:
        forward(0)
        drain()
        torch.cuda.synchronize()
        y_sharded = last["y"].clone()
        sgq.quantized_matmul(x, weights[0], None, layout=sgq.LAYOUT_NK, path=path, out=y_local, workspace=ws)
        parts = [torch.empty_like(y_local) for _ in range(world)]
        dist.all_gather(parts, y_local)                  # NCCL as the checker only
        ok = torch.tensor([1.0 if torch.equal(y_sharded, torch.cat(parts, dim=1)) else 0.0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        sharded_check = "ok" if float(ok.item()) == 1.0 else "MISMATCH"
        if sharded_check != "ok":
            if rank == 0:
                print(json.dumps({"metric": METRIC, "n_gpus": world, "sharded_check": sharded_check,
                                  "error": "gathered output differs from the single-GPU results of the slices"}), flush=True)
            dist.destroy_process_group()
            sys.exit(3)

    # collectives are launched eagerly: capturing a thousand NCCL calls into one graph buys nothing
    # (the all-gather latency dominates a sharded decode forward) and is fragile across NCCL versions
    use_graph = not args.no_graph and (world == 1 or not args.nccl)
    if use_graph:
        try:
            graph = make_graph(torch, lambda: ([forward(i) for i in range(lps)], drain()))
        except Exception as e:  # noqa: BLE001  (e.g. a collective that cannot be captured)
            sys.stderr.write(f"[bench] CUDA graph capture failed ({type(e).__name__}: {e}); launching eagerly\n")
            use_graph = False
            torch.cuda.synchronize()

    def step(s):
        if use_graph:
            graph.replay()
        else:
            for i in range(lps):
                forward(s * lps + i)
            drain()

    for s in range(args.warmup):
        step(s)
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(args.steps):
        step(s)
    e1.record()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    ms_total = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if dist:
        dist.all_reduce(ms_total, op=dist.ReduceOp.MAX)
    ms_total = float(ms_total.item())
    launches = args.steps * lps
    bytes_per_launch = gemv_bytes(M)
    value = world * launches * bytes_per_launch / (ms_total * 1e-3) / 1e9
    launch_ms = ms_total / launches
    achieved = bytes_per_launch / (launch_ms * 1e-3) / 1e9 if world == 1 else None

    # ---- end to end through the public call with HOST buffers (pinned), copies inside the timed region
    e2e = None
    if not args.no_e2e:
        xh = torch.randn(M, K_DIM).pin_memory()
        yh = torch.empty(M, (world if world > 1 else 1) * N_DIM).pin_memory()
        e2e_steps = max(1, min(args.steps, 20))

        def e2e_forward(i):
            x.copy_(xh, non_blocking=True)
            forward(i)
            if sharded and exchange is not None:
                drain()                                  # the copy below reads this forward's gathered output
            yh.copy_(last["y"] if sharded else y_local, non_blocking=True)
        # One GPU: the copies run on streams of their own with four buffers each way, so the transfer of forward
        # i + 1 overlaps the kernel of forward i; every forward still gets its x from pinned host memory and
        # returns its y there inside the timed region.  (The serial form is timed as well and reported beside it.)
        pipelined = None
        if use_graph and world == 1:
            NB = 4                                               # buffers each way
            x2 = [torch.empty_like(x) for _ in range(NB)]
            y2 = [torch.empty_like(y_local) for _ in range(NB)]
            yh2 = [torch.empty(M, N_DIM).pin_memory() for _ in range(NB)]
            cin, cout = torch.cuda.Stream(), torch.cuda.Stream()
            x_ready = [torch.cuda.Event() for _ in range(NB)]
            k_done = [torch.cuda.Event() for _ in range(NB)]
            y_done = [torch.cuda.Event() for _ in range(NB)]

            def pipelined_body():
                main = torch.cuda.current_stream()
                cin.wait_stream(main)
                cout.wait_stream(main)
                for i in range(lps):
                    b = i % NB
                    with torch.cuda.stream(cin):
                        if i >= NB:
                            cin.wait_event(k_done[b])            # forward i - NB has read x2[b]
                        x2[b].copy_(xh, non_blocking=True)
                        x_ready[b].record(cin)
                    main.wait_event(x_ready[b])
                    if i >= NB:
                        main.wait_event(y_done[b])               # the copy of forward i - NB's result has left y2[b]
                    sgq.quantized_matmul(x2[b], weights[i % copies], None, layout=sgq.LAYOUT_NK, path=path, out=y2[b], workspace=ws)
                    k_done[b].record(main)
                    with torch.cuda.stream(cout):
                        cout.wait_event(k_done[b])
                        yh2[b].copy_(y2[b], non_blocking=True)
                        y_done[b].record(cout)
                main.wait_stream(cin)
                main.wait_stream(cout)
            try:
                pipelined = make_graph(torch, pipelined_body)
            except Exception as e:  # noqa: BLE001
                sys.stderr.write(f"[bench] pipelined e2e graph capture failed ({type(e).__name__}: {e}); serial form only\n")
                pipelined = None
                torch.cuda.synchronize()
        e2e_graph = None
        if use_graph:
            try:
                e2e_graph = make_graph(torch, lambda: ([e2e_forward(i) for i in range(lps)], drain()))
            except Exception as e:  # noqa: BLE001
                sys.stderr.write(f"[bench] e2e graph capture failed ({type(e).__name__}: {e}); launching eagerly\n")
                torch.cuda.synchronize()

        def e2e_step(s):
            if e2e_graph is not None:
                e2e_graph.replay()
            else:
                for i in range(lps):
                    e2e_forward(s * lps + i)
                drain()
        for s in range(3):
            e2e_step(s)
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for s in range(e2e_steps):
            e2e_step(s)
        f1.record()
        torch.cuda.synchronize()
        t = torch.tensor([f0.elapsed_time(f1)], device=dev)
        if dist:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
        e2e = {"value": world * e2e_steps * lps * bytes_per_launch / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": lps * M * K_DIM * 4, "d2h_bytes_per_step": lps * M * world * N_DIM * 4,
               "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
               "note": "weights are resident layer parameters; per forward x comes from pinned host memory and y returns to it"}
        if pipelined is not None:
            for _ in range(3):
                pipelined.replay()
            torch.cuda.synchronize()
            yh2[(lps - 1) % NB].zero_()
            f0.record()
            for _ in range(e2e_steps):
                pipelined.replay()
            f1.record()
            torch.cuda.synchronize()
            p_ms = f0.elapsed_time(f1)
            # the last forward's result must be in host memory and equal to the one the serial form left there
            same = bool(torch.equal(yh2[(lps - 1) % NB], yh))        # (both forms end a replay with forward lps - 1 on the same weight set)
            e2e = {"value": e2e_steps * lps * bytes_per_launch / (p_ms * 1e-3) / 1e9, "unit": UNIT,
                   "h2d_bytes_per_step": lps * M * K_DIM * 4, "d2h_bytes_per_step": lps * M * N_DIM * 4,
                   "steps": e2e_steps, "ms_per_step": p_ms / e2e_steps, "result_matches_serial_form": same,
                   "serial": {"value": e2e["value"], "ms_per_step": e2e["ms_per_step"]},
                   "note": "weights are resident layer parameters; per forward x comes from pinned host memory and y returns to "
                           "it; the copies of forward i+1 overlap the kernel of forward i (copy streams, four buffers each way); "
                           "`serial` is the same loop with copy, kernel and copy strictly one after the other"}

    status = sgq.device_status()
    extra_sharded = None
    if world > 1 and not args.no_extras and not args.nccl:
        del sharded, weights
        torch.cuda.empty_cache()
        extra_sharded = sharded_extras(torch, sgq, sh, dist, dev, rank, world, peaks)
        weights = []
    if rank != 0:
        if dist:
            dist.destroy_process_group()
        return

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        try:
            kind, cores, timer = reference_linear(M)
            t1 = timer(1)
            iters = max(2, min(400, int(10.0 / max(t1, 1e-4))))
            t0 = time.perf_counter()
            per = timer(iters)
            cpu = {"value": gemv_bytes(M) / per / 1e9, "unit": UNIT, "cores": cores, "kind": kind,
                   "sample": f"{iters} CPU forwards of the same W[11008,4096], M={M} workload "
                             f"({time.perf_counter() - t0:.1f} s); each dequantizes the whole weight, as the reference does",
                   "ms_per_forward": per * 1e3}
            try:        # the same weight in the reference module's own [K,N] layout (no transpose before the matmul)
                _, _, timer_kn = reference_linear(M, native_kn=True)
                timer_kn(1)
                per_kn = timer_kn(max(2, min(40, int(4.0 / max(t1, 1e-4)))))
                cpu["native_layout_kn"] = {"value": gemv_bytes(M) / per_kn / 1e9, "unit": UNIT, "ms_per_forward": per_kn * 1e3}
            except Exception as e:  # noqa: BLE001
                cpu["native_layout_kn"] = {"error": f"{type(e).__name__}: {e}"[:200]}
        except Exception as e:  # noqa: BLE001
            cpu = {"error": f"{type(e).__name__}: {e}"[:200]}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u8 x s8 -> s32 (INT4 codes x int8 activation digits), fp32 group scales", "data": "synthetic",
        "config": {"workload": f"config2: INT4 g=32 decode GEMV, W[{N_DIM},{K_DIM}] stored [N,K], X[{M},{K_DIM}] fp32"
                               + (f"; column-sharded, N_total={world * N_DIM}, "
                                  + ("NCCL all-gather of output slices per forward" if args.nccl else
                                     "output slices stored into every GPU's output by the decode kernel (NVLink peer stores), "
                                     "signal at its end, wait in the next forward's prologue; one barrier kernel per step")
                                  if world > 1 else ""),
                   "M": M, "K": K_DIM, "N_per_gpu": N_DIM, "group": GROUP, "launches_per_step": lps, "weight_copies": copies,
                   "l2": f"rotating {copies} weight sets ({copies * gemv_bytes(0) / 1e6:.0f} MB) > 126 MB L2",
                   "path": sgq.PATH_NAMES[path], "bytes_per_launch": bytes_per_launch,
                   "launch": "one CUDA graph replay per step" if use_graph else "eager launches",
                   "stream_overlap": (f"mode {args.overlap_mode}: programmatic dependent launch, a forward's first weight tiles are "
                                      "fetched while the previous forward finishes") if not args.no_overlap else "off"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": (achieved / peaks["hbm_gbs"]) if achieved else None,
                     "traffic": args.traffic if args.traffic is not None else ncu_traffic("gemv_int4_nk_kernel", M) if world == 1 else None,
                     "peak_source": peaks["source"], "kernel": "gemv_int4_nk_kernel",
                     "launch_us": launch_ms * 1e3},
        "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches + (args.steps if world > 1 else 0), "clocks": clocks,
        "device_status_word": status,
    }
    if sharded_check is not None:
        line["sharded_check"] = sharded_check
    if extra_sharded is not None:
        line["extra"] = extra_sharded
    if world == 1 and not args.no_extras:
        line["extra"] = extras(torch, sgq, peaks, weights)
        del weights
        try:
            line["extra"]["nanollama_int4_config4"] = nanollama_case(torch, sgq, dev, reps=3, warm=2)
        except Exception as e:  # noqa: BLE001
            line["extra"]["nanollama_int4_config4"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    print(json.dumps(line), flush=True)
    if dist:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemv", choices=["gemv", "nanollama"],
                    help="gemv: the config-2 headline (default); nanollama: the config-4 tokens/s line")
    ap.add_argument("--M", type=int, default=1)
    ap.add_argument("--copies", type=int, default=10)
    ap.add_argument("--launches-per-step", type=int, default=1000)
    ap.add_argument("--traffic", type=float, default=None, help="ncu dram bytes per launch to report instead of the recorded figure")
    ap.add_argument("--only", default=None, help="run just this secondary case (a key of `extra`), eagerly")
    ap.add_argument("--only-graph", action="store_true", help="with --only: time graph replays instead of a few eager launches")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-overlap", action="store_true", help="launch without programmatic dependent launch")
    ap.add_argument("--overlap-mode", type=int, default=1, choices=[1, 2],
                    help="1: overlapped launches; 2: overlapped launches with the two-CTAs-per-SM form of the decode kernel")
    ap.add_argument("--nccl", action="store_true", help="N > 1: exchange output slices with an NCCL all-gather instead of peer stores")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "nanollama":
        if args.steps == 100 and args.warmup == 5:      # the gemv defaults: one generation is ~0.2 s
            args.steps, args.warmup = 5, 2
        run_nanollama(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
