#!/usr/bin/env python
"""Benchmark of the dense-contraction hot path on N B200s of one node.

Headline workload (BASELINE config 1): bf16 GEMM M=N=K=8192, A[M,K] and B[K,N] ~ N(0,1)/sqrt(K)
rounded to bf16, fp32 accumulation, bf16 output.  A "step" is one GEMM launch.  With N>1 GPUs the
weight columns are split (rank r owns B[:, r*N/G:(r+1)*N/G] and the matching columns of C, A is
replicated), so the total work is fixed ("strong" scaling) and no data-path collective runs.

`value` is the whole-job TFLOP/s with operands resident in HBM; `e2e` is the same metric through
the public launcher API with HOST buffers (pinned host -> device copies of A and B and a
device -> host read of C inside the timed region).  `roofline` compares the kernel with the
measured cuBLAS bf16 peak of this pool; `cpu_baseline` times the CPU oracle (a port of the
reference's `cpu_gemm`) on a bounded slab.  `extra` reports FMHA forward (BASELINE config 2,
8 x 32 x 4096 x 128, sharded by batch x head) measured the same way.

`--impl reference` times the reference's own CPU implementation of the path (the oracle port of
`cpu_gemm`; the reference's GPU path needs a Rust toolchain and NVIDIA's `tileiras`, neither of
which exists here) on all host threads, each step a bounded row slab of the same GEMM.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "TFLOP/s (GEMM 8192^3 bf16, fp32 accumulate)"
M = N = K = 8192
FALLBACK_BF16_TFLOPS = 1590.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of gemm_tc_pair_kernel: 316.7 MB measured
# by ncu on a 4096x4096x8192 case (256 tiles), scaled by tiles processed to the 1024 tiles of
# 8192^3 (profiles/gemm_bf16_pair.md).  The full-size launch is not captured under ncu.
GEMM_DRAM_TRAFFIC_BYTES = int(316.7e6 * 4)


SUSTAINED_BF16_TFLOPS = None


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            d = json.load(fh)
        global SUSTAINED_BF16_TFLOPS
        SUSTAINED_BF16_TFLOPS = float(d.get("bf16_tflops_sustained", 0.0)) or None
        return float(d["bf16_tflops"]), float(d.get("hbm_gbs", 0.0)), "measured"
    except (OSError, ValueError, KeyError):
        return FALLBACK_BF16_TFLOPS, 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.lines = []
        self.proc = None
        self.thread = None

    def start(self):
        # NVML polled in-process every millisecond when the binding is there (a timed region of a few
        # milliseconds falls between two nvidia-smi samples); nvidia-smi otherwise.  Read-only queries.
        self.nvml_rows = []
        self._stop = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self.gpu)
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return
        except Exception:
            self._nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _poll_nvml(self):
        n = self._nvml
        while not self._stop:
            try:
                sm = n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)
                reasons = n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                power = n.nvmlDeviceGetPowerUsage(self._handle) / 1000.0
                self.nvml_rows.append((time.monotonic(), sm, reasons, power))
            except Exception:
                pass
            time.sleep(0.001)

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.monotonic(), line.strip()))

    def _stop_nvml(self, t0: float, t1: float):
        n = self._nvml
        self._stop = True
        self.thread.join(timeout=2)
        try:
            smax = n.nvmlDeviceGetMaxClockInfo(self._handle, n.NVML_CLOCK_SM)
        except Exception:
            smax = None
        rows = [r for r in self.nvml_rows if t0 <= r[0] <= t1] or self.nvml_rows
        bits = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}
        reasons = sorted(name for name, bit in bits.items() if any(r[2] & bit for r in rows))
        return {"sm_mhz": statistics.median([r[1] for r in rows]) if rows else None, "sm_max_mhz": smax,
                "reasons": reasons, "samples": len(rows), "source": "nvml, 1 ms poll",
                "sm_mhz_min": min((r[1] for r in rows), default=None),
                "power_w_max": max((r[3] for r in rows), default=None)}

    def stop(self, t0: float, t1: float):
        if getattr(self, "_nvml", None) is not None:
            return self._stop_nvml(t0, t1)
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [l for (t, l) in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or [l for _, l in self.lines]
        for line in rows:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi -lms 100"}


# ------------------------------------------------------------------------------------------
# CPU arms (the only place besides tests/smoke where the oracle runs)
# ------------------------------------------------------------------------------------------
def _cpu_slab_inputs(rows: int):
    import torch
    from cutile_rs_b200 import workloads
    g = torch.Generator().manual_seed(workloads.SEED_BASE + 1)
    s = 1.0 / math.sqrt(K)
    a = (torch.randn(rows, K, generator=g) * s).to(torch.bfloat16).float().numpy()
    b = (torch.randn(K, N, generator=g) * s).to(torch.bfloat16).float().numpy()
    return a, b


def cpu_gemm_rate(target_seconds: float, threads: int):
    """Times the oracle's cpu_gemm on a row slab of the 8192^3 problem sized to ~target_seconds."""
    from oracle import oracle
    threads = threads or oracle.max_threads()
    a, b = _cpu_slab_inputs(max(threads, 8) * 8)
    probe_rows = max(threads, 8)
    t0 = time.perf_counter()
    oracle.cpu_gemm(a[:probe_rows], b, threads=threads)
    per_row = (time.perf_counter() - t0) / probe_rows
    rows = int(min(max(target_seconds / max(per_row, 1e-9), probe_rows), a.shape[0]))
    rows -= rows % max(threads, 1) if rows >= threads else 0
    rows = max(rows, 1)
    t0 = time.perf_counter()
    oracle.cpu_gemm(a[:rows], b, threads=threads)
    dt = time.perf_counter() - t0
    return {"tflops": 2.0 * rows * N * K / dt / 1e12, "rows": rows, "seconds": dt, "threads": threads}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import oracle
    threads = oracle.max_threads()
    steps, warmup = args.steps, args.warmup
    budget = 150.0 / max(steps + warmup, 1)
    a, b = _cpu_slab_inputs(max(threads, 8) * 4)
    probe_rows = max(threads, 8)
    t0 = time.perf_counter()
    oracle.cpu_gemm(a[:probe_rows], b, threads=threads)
    per_row = (time.perf_counter() - t0) / probe_rows
    rows = int(min(max(budget / max(per_row, 1e-9), 1), a.shape[0]))
    if rows >= threads:
        rows -= rows % threads
    for _ in range(warmup):
        oracle.cpu_gemm(a[:rows], b, threads=threads)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.cpu_gemm(a[:rows], b, threads=threads)
    dt = time.perf_counter() - t0
    tflops = 2.0 * rows * N * K * steps / dt / 1e12
    sample = f"rows [0,{rows}) of the 8192^3 bf16-rounded GEMM per step, naive f32 triple loop"
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": dt / steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "gemm_bf16_8192x8192x8192", "layout": "A[M,K] B[K,N] row-major",
                   "note": "reference's host-side cpu_gemm (oracle port) on host cores; the "
                           "reference's GPU path cannot be built here (no Rust toolchain, no tileiras)"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    from cutile_rs_b200 import _lib, api, launch, sharding, workloads

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; the product has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    _lib.check(lib.b200tile_init(local_rank))
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- operands: A replicated, B and C column-sharded; generated once, outside timing ----
    n0, n1 = sharding.split_range(N, world, rank, 256)
    a_host, b_host = workloads.gemm_bf16_inputs(M, N, K)
    b_host = b_host[:, n0:n1].contiguous()
    n_local = n1 - n0
    x = api.copy_host_to_device(a_host)
    y = api.copy_host_to_device(b_host)
    z = api.zeros([M, n_local], "bf16")
    # the reference's published configuration: tile 256x256x64 on CTA pairs (num_cta_in_cga = 2)
    bm, bn = 256, 256
    generics = ["bf16", str(bm), str(bn), "64"]
    opts = launch.CompileOptions(num_cta_in_cga=2, occupancy=1)

    def step():
        launch.gemm(z.partition([bm, bn]), x, y).generics(generics).compile_options(opts).async_on(stream)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    barrier()
    t_begin = time.monotonic()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    t_end = time.monotonic()
    total_ms = sharding.max_over_ranks(e0.elapsed_time(e1), dev)
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    ms_per_step = total_ms / args.steps
    flops = workloads.gemm_flops(M, N, K)
    value = flops / (ms_per_step * 1e-3) / 1e12
    _lib.check(lib.b200tile_status(stream.cuda_stream, __import__("ctypes").byref(_lib.StatusC())))

    # ---- end to end through the public API with host buffers ----
    a_pin, b_pin = api.pin(a_host), api.pin(b_host)
    c_pin = torch.empty((M, n_local), dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(min(args.steps, 5), 1)

    # one call of the public API per step: B up, A up in 1024-row slabs, each slab multiplied on arrival and
    # its C rows sent back while the next slab is in flight (uploads, MMA and downloads on three streams)
    host_gemm = api.HostGemm(M, n_local, K, "bf16")

    def e2e_step():
        host_gemm(a_pin, b_pin, c_pin, stream)

    def e2e_serial_step():
        xa = api.copy_host_to_device(a_pin, stream=stream)
        yb = api.copy_host_to_device(b_pin, stream=stream)
        (zz, _, _) = launch.gemm(z.partition([bm, bn]), xa, yb).generics(generics) \
            .compile_options(opts).async_on(stream)
        c_pin.copy_(zz.unpartition().storage, non_blocking=True)

    e2e_serial_step()
    barrier()
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_serial_step()
    e1.record(stream)
    barrier()
    e2e_serial_ms = sharding.max_over_ranks(e0.elapsed_time(e1), dev) / e2e_steps
    e2e_step()
    barrier()
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e1.record(stream)
    barrier()
    e2e_ms = sharding.max_over_ranks(e0.elapsed_time(e1), dev) / e2e_steps
    e2e_value = flops / (e2e_ms * 1e-3) / 1e12
    h2d = (a_pin.numel() + b_pin.numel()) * 2 * world
    d2h = c_pin.numel() * 2 * world

    # ---- FMHA forward (config 2), sharded by batch x head, reported as `extra` ----
    extra = {}
    if not args.no_fmha:
        import ctypes
        B_, H_, S_, D_ = 8, 32, 4096, 128
        p0, p1 = sharding.split_range(B_ * H_, world, rank, 1)
        nb = p1 - p0
        g = torch.Generator(device="cuda").manual_seed(workloads.SEED_BASE + 2 + rank)
        q = torch.randn(nb, S_, D_, generator=g, device=dev).bfloat16()
        kk = torch.randn(nb, S_, D_, generator=g, device=dev).bfloat16()
        v = torch.randn(nb, S_, D_, generator=g, device=dev).bfloat16()
        o = torch.empty_like(q)
        I2 = ctypes.c_int64 * 2
        st = I2(S_ * D_, D_)
        for causal in (False, True):
            def fstep():
                _lib.check(lib.b200tile_fmha_fwd(b"bf16", q.data_ptr(), kk.data_ptr(), v.data_ptr(), o.data_ptr(),
                                                 1, nb, nb, S_, S_, D_, st, st, st, st, 1.0 / math.sqrt(D_),
                                                 int(causal), 0, stream.cuda_stream))
            for _ in range(3):
                fstep()
            barrier()
            e0.record(stream)
            iters = 10
            for _ in range(iters):
                fstep()
            e1.record(stream)
            barrier()
            fms = sharding.max_over_ranks(e0.elapsed_time(e1), dev) / iters
            ftf = workloads.fmha_flops(B_, H_, S_, D_, causal) / (fms * 1e-3) / 1e12
            extra["fmha_fwd_causal" if causal else "fmha_fwd_noncausal"] = {
                "tflops": ftf, "tflops_per_gpu": ftf / world, "ms": fms,
                "config": f"bf16 b{B_} h{H_} s{S_} d{D_}, (b*h) split over {world} GPU(s)"}
        # the same non-causal shape through the generated-launcher mirror with the CTA-pair configuration
        # (CompileOptions(num_cta_in_cga=2): persistent pairs, alternating softmax warpgroups)
        qd, kd, vd = (api.from_torch(t_.view(1, nb, S_, D_)) for t_ in (q, kk, v))
        od = api.from_torch(o).partition([1, 128, D_])
        fopts = launch.CompileOptions(num_cta_in_cga=2)

        def pstep():
            nonlocal od
            (od, *_r) = launch.fmha(od, qd, kd, vd, 1.0 / math.sqrt(D_), 0, 1, causal=False) \
                .compile_options(fopts).async_on(stream)
        for _ in range(3):
            pstep()
        barrier()
        e0.record(stream)
        for _ in range(10):
            pstep()
        e1.record(stream)
        barrier()
        fms = sharding.max_over_ranks(e0.elapsed_time(e1), dev) / 10
        ftf = workloads.fmha_flops(B_, H_, S_, D_, False) / (fms * 1e-3) / 1e12
        extra["fmha_fwd_noncausal_cta_pairs"] = {
            "tflops": ftf, "tflops_per_gpu": ftf / world, "ms": fms,
            "config": "same shape, CompileOptions(num_cta_in_cga=2), through the launcher"}
        del q, kk, v, o, qd, kd, vd, od

        # ---- block-scaled GEMMs (configs 3 and 4), weight rows (N) split over the ranks ----
        from cutile_rs_b200 import quant

        def timed(fn, iters=10):
            for _ in range(3):
                fn()
            barrier()
            e0.record(stream)
            for _ in range(iters):
                fn()
            e1.record(stream)
            barrier()
            return sharding.max_over_ranks(e0.elapsed_time(e1), dev) / iters

        g = torch.Generator(device="cuda").manual_seed(workloads.SEED_BASE + 3)
        m8, n8, k8 = 8192, 28672, 8192
        r0, r1 = sharding.split_range(n8, world, rank, 256)
        xq, xs = quant.quant_fp8_block(torch.randn(m8, k8, device=dev, generator=g), 1, 128)
        yq, ys = quant.quant_fp8_block(torch.randn(r1 - r0, k8, device=dev, generator=g), 128, 128)
        z8 = torch.empty(m8, r1 - r0, dtype=torch.bfloat16, device=dev)

        def f8step():
            _lib.check(lib.b200tile_linear_fp8_blk128(xq.data_ptr(), yq.data_ptr(), xs.data_ptr(), ys.data_ptr(),
                                                      z8.data_ptr(), b"bf16", m8, r1 - r0, k8, k8, k8, r1 - r0,
                                                      k8 // 128, k8 // 128, 1.0, stream.cuda_stream))
        ms8 = timed(f8step, 5)
        tf8 = workloads.gemm_flops(m8, n8, k8) / (ms8 * 1e-3) / 1e12
        extra["gemm_fp8_blk128"] = {"tflops": tf8, "tflops_per_gpu": tf8 / world, "ms": ms8,
                                    "pct_of_nominal_fp8_peak_4500": 100.0 * tf8 / world / 4500.0,
                                    "config": f"e4m3 M{m8} N{n8} K{k8}, fp32 scales 1x128 / 128x128, bf16 out, "
                                              f"N split over {world} GPU(s)"}
        # the same shape with the hardware's own fp8 block scaling (MXFP8: e8m0 scale per 32 elements), the
        # reference's fp8 path (cutile-examples/examples/mxfp8.rs:34-64): no promotion pass on CUDA cores
        xm, xms = quant.quant_mxfp8(torch.randn(m8, k8, device=dev, generator=g))
        ym, yms = quant.quant_mxfp8(torch.randn(r1 - r0, k8, device=dev, generator=g))
        wsm = lib.b200tile_linear_mxfp8_workspace_bytes(m8, r1 - r0, k8)
        wsb8 = torch.empty(wsm, dtype=torch.uint8, device=dev)

        def mx8step():
            _lib.check(lib.b200tile_linear_mxfp8(xm.data_ptr(), ym.data_ptr(), xms.data_ptr(), yms.data_ptr(),
                                                 z8.data_ptr(), b"bf16", m8, r1 - r0, k8, k8, k8, r1 - r0, k8 // 32,
                                                 k8 // 32, 1.0, wsb8.data_ptr(), wsm, stream.cuda_stream))
        msm = timed(mx8step, 5)
        tfm = workloads.gemm_flops(m8, n8, k8) / (msm * 1e-3) / 1e12
        extra["gemm_mxfp8"] = {"tflops": tfm, "tflops_per_gpu": tfm / world, "ms": msm,
                               "pct_of_nominal_fp8_peak_4500": 100.0 * tfm / world / 4500.0,
                               "config": f"MXFP8 (e4m3, e8m0 scale per 32) M{m8} N{n8} K{k8}, bf16 out, N split over "
                                         f"{world} GPU(s); includes the per-call scale re-layout"}
        del xm, xms, ym, yms, wsb8
        del xq, xs, yq, ys, z8
        n4, k4 = 14336, 4096
        r0, r1 = sharding.split_range(n4, world, rank, 256)
        yp, ysc, gy = quant.quant_nvfp4(torch.randn(r1 - r0, k4, device=dev, generator=g))
        for m4 in (4096, 16):
            xp, xsc, gx = quant.quant_nvfp4(torch.randn(m4, k4, device=dev, generator=g))
            z4 = torch.empty(m4, r1 - r0, dtype=torch.bfloat16, device=dev)
            wsb = lib.b200tile_linear_nvfp4_workspace_bytes(m4, r1 - r0, k4)
            ws = torch.empty(wsb, dtype=torch.uint8, device=dev)

            def f4step():
                _lib.check(lib.b200tile_linear_nvfp4(xp.data_ptr(), yp.data_ptr(), xsc.data_ptr(), ysc.data_ptr(),
                                                     z4.data_ptr(), b"bf16", m4, r1 - r0, k4, k4 // 2, k4 // 2,
                                                     r1 - r0, k4 // 16, k4 // 16, gx * gy, ws.data_ptr(), wsb, -1,
                                                     stream.cuda_stream))
            ms4 = timed(f4step, 10)
            tf4 = workloads.gemm_flops(m4, n4, k4) / (ms4 * 1e-3) / 1e12
            nbytes = (m4 * k4 // 2 + m4 * k4 // 16 + n4 * k4 // 2 + n4 * k4 // 16 + m4 * n4 * 2)
            entry = {"tflops": tf4, "tflops_per_gpu": tf4 / world, "ms": ms4,
                     "pct_of_nominal_fp4_peak_9000": 100.0 * tf4 / world / 9000.0,
                     "algorithmic_gbs": nbytes / (ms4 * 1e-3) / 1e9,
                     "config": f"NVFP4 M{m4} N{n4} K{k4}, e4m3 scale per 16, bf16 out, N split over {world} "
                               "GPU(s); includes the per-call re-layout of the weight scales"}
            if m4 <= 128:
                # decode: weight scales laid out once (they are constants of the model), then one kernel per call
                cfg = 0
                need = lib.b200tile_nvfp4_weight_scales_bytes(r1 - r0, k4, cfg)
                prep = torch.empty(need, dtype=torch.uint8, device=dev)
                _lib.check(lib.b200tile_nvfp4_prepare_weight_scales(ysc.data_ptr(), r1 - r0, k4, k4 // 16, cfg,
                                                                    prep.data_ptr(), need, stream.cuda_stream))

                def f4prep():
                    _lib.check(lib.b200tile_linear_nvfp4_prepared(xp.data_ptr(), yp.data_ptr(), xsc.data_ptr(),
                                                                  prep.data_ptr(), z4.data_ptr(), b"bf16", m4, r1 - r0,
                                                                  k4, k4 // 2, k4 // 2, r1 - r0, k4 // 16, gx * gy, cfg,
                                                                  stream.cuda_stream))
                msp = timed(f4prep, 20)
                entry["prepared_weight_scales"] = {
                    "us": msp * 1e3, "algorithmic_gbs": nbytes / (msp * 1e-3) / 1e9,
                    "frac_of_measured_hbm": nbytes / (msp * 1e-3) / 1e9 / world / measured_peaks()[1]}
            extra[f"gemm_nvfp4_m{m4}"] = entry
        del xp, xsc, yp, ysc, z4, ws

        # ---- split-KV GQA decode attention + merge: K/V heads split over the ranks ----
        HKV, GRP, SKV, DD = 8, 4, 65536, 128
        h0, h1 = sharding.split_range(HKV, world, rank, 1)
        hl = h1 - h0
        if hl > 0:
            ns = max(1, lib.b200tile_num_sms() // hl)
            nbuf = 4   # rotate K/V sets (268 MB each at 8 heads) so that no launch finds its keys in L2
            qd = torch.randn(hl, GRP, DD, generator=g, device=dev).bfloat16()
            kds = [torch.randn(hl, SKV, DD, generator=g, device=dev).bfloat16() for _ in range(nbuf)]
            vds = [torch.randn(hl, SKV, DD, generator=g, device=dev).bfloat16() for _ in range(nbuf)]
            attp = torch.empty(hl, ns * GRP, DD, dtype=torch.bfloat16, device=dev)
            lsep = torch.empty(hl, ns * GRP, dtype=torch.float32, device=dev)
            od = torch.empty_like(qd)
            posd = torch.tensor([SKV - 1], dtype=torch.int32, device=dev)
            turn = [0]

            def dstep():
                i = turn[0] = (turn[0] + 1) % nbuf
                _lib.check(lib.b200tile_fmha_decode_gqa_split(
                    b"bf16", qd.data_ptr(), kds[i].data_ptr(), vds[i].data_ptr(), attp.data_ptr(), lsep.data_ptr(),
                    od.data_ptr(), posd.data_ptr(), hl, GRP, DD, SKV, 128, ns, 1.0 / math.sqrt(DD), I2(GRP * DD, DD),
                    I2(SKV * DD, DD), I2(SKV * DD, DD), I2(ns * GRP * DD, DD), ns * GRP, I2(GRP * DD, DD),
                    stream.cuda_stream))
            msd = timed(dstep, 20)
        else:
            barrier(); barrier()
            msd = sharding.max_over_ranks(0.0, dev)
        kv_bytes = 2 * HKV * SKV * DD * 2
        gbs = kv_bytes / (msd * 1e-3) / 1e9
        extra["fmha_decode_gqa_split_merge"] = {
            "gbs": gbs, "gbs_per_gpu": gbs / world, "us": msd * 1e3,
            "frac_of_measured_hbm": gbs / world / measured_peaks()[1],
            "config": f"bf16 kv_heads {HKV} group {GRP} D {DD} s_kv {SKV}, BN 128, splits = SMs / local heads, "
                      f"split pass + merge per step, kv heads split over {world} GPU(s), K/V sets rotated (inputs > L2)"}

        # ---- residual add + RMSNorm (HBM-bound neighbour of the linear layers), token rows split over the ranks;
        # two sets of tensors are alternated so that nothing is served from L2 (2 x 1.07 GB at one GPU)
        NT, NH = 16384, 8192
        t0_, t1_ = sharding.split_range(NT, world, rank, 1)
        nt = t1_ - t0_
        sets = []
        for i_ in range(2):
            g = torch.Generator(device="cuda").manual_seed(workloads.SEED_BASE + 11 + i_)
            sets.append((torch.randn(nt, NH, device=dev, generator=g).half(),
                         torch.randn(nt, NH, device=dev, generator=g).half(),
                         torch.empty(nt, NH, device=dev, dtype=torch.float16),
                         torch.empty(nt, NH, device=dev, dtype=torch.float16)))
        wn = torch.ones(NH, device=dev, dtype=torch.float16)
        flip = [0]

        def nstep():
            r_, x_, o_, ro_ = sets[flip[0] & 1]
            flip[0] += 1
            _lib.check(lib.b200tile_add_rms_norm(b"f16", r_.data_ptr(), x_.data_ptr(), wn.data_ptr(), o_.data_ptr(),
                                                 ro_.data_ptr(), nt, NH, NH, NH, NH, NH, 1e-5, stream.cuda_stream))
        msn = timed(nstep, 20)
        nbytes = 4.0 * NT * NH * 2
        gbn = nbytes / (msn * 1e-3) / 1e9
        extra["add_rms_norm_f16"] = {
            "gbs": gbn, "gbs_per_gpu": gbn / world, "us": msn * 1e3,
            "frac_of_measured_hbm": gbn / world / measured_peaks()[1],
            "config": f"f16 {NT} tokens x {NH}, read residual + x, write out + residual_out (algorithmic bytes), "
                      f"token rows split over {world} GPU(s), two tensor sets alternated (inputs > L2)"}
        del sets

        # ---- rotary position embedding over [tokens, heads, D]; token rows split over the ranks, two sets alternated
        RT, RH, RD = 32768, 32, 128
        t0_, t1_ = sharding.split_range(RT, world, rank, 1)
        rt = t1_ - t0_
        rsets = [(torch.randn(rt, RH, RD, device=dev).half(), torch.empty(rt, RH, RD, device=dev, dtype=torch.float16))
                 for _ in range(2)]
        inv_f = (1.0 / 10000.0 ** (torch.arange(0, RD, 2, dtype=torch.float32, device=dev) / RD)).contiguous()
        I2r = ctypes.c_int64 * 2
        rst = I2r(RH * RD, RD)
        rflip = [0]

        def rstep():
            x_, o_ = rsets[rflip[0] & 1]
            rflip[0] += 1
            _lib.check(lib.b200tile_rope_seq(b"f16", x_.data_ptr(), inv_f.data_ptr(), o_.data_ptr(), rt, RH, RD, rst, rst,
                                             t0_, None, stream.cuda_stream))
        msr = timed(rstep, 20)
        gbr = 2.0 * RT * RH * RD * 2 / (msr * 1e-3) / 1e9
        extra["rope_seq_f16"] = {
            "gbs": gbr, "gbs_per_gpu": gbr / world, "us": msr * 1e3,
            "frac_of_measured_hbm": gbr / world / measured_peaks()[1],
            "config": f"f16 {RT} tokens x {RH} heads x {RD}, one read + one write per element, token rows split over "
                      f"{world} GPU(s), two tensor sets alternated (inputs > L2)"}
        del rsets

        # ---- QK norm + rotary embedding + KV-cache write in one pass (prefill block of 16384 tokens, 32 + 8 heads);
        # token rows split over the ranks; 403 MB of reads and writes per launch at one GPU (> L2)
        QT, QH, KVH = 16384, 32, 8
        t0_, t1_ = sharding.split_range(QT, world, rank, 1)
        qt = t1_ - t0_
        qq = torch.randn(qt, QH, RD, device=dev).half()
        qk_ = torch.randn(qt, KVH, RD, device=dev).half()
        qv = torch.randn(qt, KVH, RD, device=dev).half()
        qo_ = torch.empty_like(qq)
        kc_ = torch.empty(KVH, qt, RD, device=dev, dtype=torch.float16)
        vc_ = torch.empty(KVH, qt, RD, device=dev, dtype=torch.float16)
        wq_ = torch.ones(RD, device=dev, dtype=torch.float16)

        def qstep():
            _lib.check(lib.b200tile_qk_norm_rope_kv(b"f16", qq.data_ptr(), qk_.data_ptr(), qv.data_ptr(), wq_.data_ptr(),
                                                    wq_.data_ptr(), inv_f.data_ptr(), qo_.data_ptr(), kc_.data_ptr(),
                                                    vc_.data_ptr(), 1e-6, 0, None, qt, QH, KVH, RD, qt, QH * RD,
                                                    KVH * RD, KVH * RD, QH * RD, stream.cuda_stream))
        msq = timed(qstep, 20)
        gbq = 2.0 * QT * (QH + 2 * KVH) * RD * 2 / (msq * 1e-3) / 1e9
        extra["qk_norm_rope_kv_prefill"] = {
            "gbs": gbq, "gbs_per_gpu": gbq / world, "us": msq * 1e3,
            "frac_of_measured_hbm": gbq / world / measured_peaks()[1],
            "config": f"f16 {QT} tokens, {QH} q heads + {KVH} kv heads x {RD}: read q, k, v; write q_out, k_cache, v_cache; "
                      f"token rows split over {world} GPU(s)"}
        del qq, qk_, qv, qo_, kc_, vc_

        # ---- LM head fused with the block argmax (decode: one hidden vector against the vocabulary matrix), the
        # vocabulary rows split over the ranks; 1.05 GB of weights at one GPU (> L2), read once
        LV, LK = 128256, 4096
        v0_, v1_ = sharding.split_range(LV, world, rank, 64)
        lv = v1_ - v0_
        lw = (torch.randn(lv, LK, device=dev) / 64).half()
        lh = torch.randn(LK, device=dev).half()
        lbm = torch.empty((lv + 63) // 64, device=dev, dtype=torch.float32)
        lbi = torch.empty((lv + 63) // 64, device=dev, dtype=torch.int32)
        ltok = torch.empty(1, device=dev, dtype=torch.int32)

        def lstep():
            _lib.check(lib.b200tile_lm_head_argmax_blocks(b"f16", lw.data_ptr(), lh.data_ptr(), lbm.data_ptr(),
                                                          lbi.data_ptr(), lv, LK, LK, stream.cuda_stream))
            _lib.check(lib.b200tile_argmax_reduce_blocks(lbm.data_ptr(), lbi.data_ptr(), ltok.data_ptr(),
                                                         (lv + 63) // 64, stream.cuda_stream))
        msl = timed(lstep, 20)
        gbl = 2.0 * LV * LK / (msl * 1e-3) / 1e9
        extra["lm_head_argmax_f16"] = {
            "gbs": gbl, "gbs_per_gpu": gbl / world, "us": msl * 1e3,
            "frac_of_measured_hbm": gbl / world / measured_peaks()[1],
            "config": f"f16 vocabulary {LV} x hidden {LK}: fused matrix-vector product + block argmax, then the reduction "
                      f"over blocks (two launches per step); vocabulary rows split over {world} GPU(s)"}
        del lw

        # ---- SiLU(gate) * up as a kernel of its own (the unfused SwiGLU step), token rows split over the ranks;
        # 3 x 235 MB per launch at one GPU (> L2)
        ST, SI = 8192, 14336
        t0_, t1_ = sharding.split_range(ST, world, rank, 1)
        st_ = t1_ - t0_
        sg = torch.randn(st_, SI, device=dev).half()
        su = torch.randn(st_, SI, device=dev).half()
        so = torch.empty_like(sg)

        def sstep():
            _lib.check(lib.b200tile_silu_mul_2d(b"f16", so.data_ptr(), sg.data_ptr(), su.data_ptr(), st_, SI, SI, SI, SI,
                                                stream.cuda_stream))
        mss = timed(sstep, 20)
        gbs_ = 3.0 * ST * SI * 2 / (mss * 1e-3) / 1e9
        extra["silu_mul_2d_f16"] = {
            "gbs": gbs_, "gbs_per_gpu": gbs_ / world, "us": mss * 1e3,
            "frac_of_measured_hbm": gbs_ / world / measured_peaks()[1],
            "config": f"f16 {ST} x {SI}: two reads and one write per element, token rows split over {world} GPU(s)"}
        del sg, su, so

        # ---- the reference's published protocol, as far as this library goes: f16 all-ones operands, 5 warm-up
        # launches, median over 10 samples of 3 back-to-back launches between stream syncs, host clock
        # (cutile-benchmarks/paper/sec5_exp1_safety_overhead/rust/gemm/src/main.rs:629-631,1289-1322).
        # The accumulator here stays fp32 (the reference's run used f16 accumulation).
        if world == 1:
            ones_a = torch.ones(M, K, dtype=torch.float16, device=dev)
            ones_b = torch.ones(K, N, dtype=torch.float16, device=dev)
            ones_c = torch.empty(M, N, dtype=torch.float16, device=dev)

            def ones_step():
                _lib.check(lib.b200tile_gemm(b"f16", 0, ones_a.data_ptr(), ones_b.data_ptr(), ones_c.data_ptr(), 1, M,
                                             N, K, K, N, N, 0, 0, 0, 0, 2, 8, 0, stream.cuda_stream))
            for _ in range(5):
                ones_step()
            torch.cuda.synchronize()
            samples = []
            for _ in range(10):
                t0 = time.perf_counter()
                for _ in range(3):
                    ones_step()
                torch.cuda.synchronize()
                samples.append((time.perf_counter() - t0) / 3)
            samples.sort()
            med = 0.5 * (samples[4] + samples[5])
            ok_ones = bool((ones_c[::997, ::991].float() == float(K)).all().item())
            extra["gemm_f16_ones_published_protocol"] = {
                "tflops": flops / med / 1e12, "median_us": med * 1e6, "result_is_k_everywhere": ok_ones,
                "published_reference_tflops": 2068.88,
                "config": "f16 all-ones 8192^3, tile 256x256x64 on CTA pairs, grouped-M 8; fp32 accumulation here, "
                          "f16 accumulation in the published run (other GPU, CUDA 13.2, locked 1830 MHz target)"}
            del ones_a, ones_b, ones_c

        # ---- this kernel and cuBLAS (torch.matmul, a library call used only as a yardstick) in alternating
        # blocks of 16 launches on the same operands: under a sustained load both sit on the 1 kW cap, so a
        # back-to-back comparison in one thermal state says more than two separate bursts
        if world == 1:
            a_t, b_t, c_t = x.storage, y.storage, torch.empty((M, n_local), dtype=torch.bfloat16, device=dev)
            for _ in range(3):          # library initialisation and heuristics stay outside the timing
                torch.matmul(a_t, b_t, out=c_t)
            torch.cuda.synchronize()
            ours, theirs = [], []
            for _ in range(6):
                for lst, fn in ((ours, step), (theirs, lambda: torch.matmul(a_t, b_t, out=c_t))):
                    e0.record(stream)
                    for _ in range(16):
                        fn()
                    e1.record(stream)
                    torch.cuda.synchronize()
                    lst.append(flops / (e0.elapsed_time(e1) / 16 * 1e-3) / 1e12)
            extra["gemm_bf16_vs_cublas_interleaved"] = {
                "this_kernel_tflops": sum(ours) / len(ours), "cublas_tflops": sum(theirs) / len(theirs),
                "this_kernel_blocks": ours, "cublas_blocks": theirs,
                "config": "8192^3 bf16, 6 alternating blocks of 16 launches each, CUDA events per block"}

            # ---- the library's fp8 GEMM (cuBLASLt through torch._scaled_mm, one scale per tensor) as a
            # yardstick for the block-scaled kernels above: it does less (no block scales) on the same
            # power-capped part
            try:
                a8 = torch.randn(M, K, device=dev).to(torch.float8_e4m3fn)
                b8 = torch.randn(N, K, device=dev).to(torch.float8_e4m3fn).t()
                one = torch.ones((), device=dev)

                def lib8():
                    return torch._scaled_mm(a8, b8, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
                for _ in range(3):
                    lib8()
                torch.cuda.synchronize()
                e0.record(stream)
                for _ in range(16):
                    lib8()
                e1.record(stream)
                torch.cuda.synchronize()
                extra["library_fp8_gemm_yardstick"] = {
                    "tflops": 2.0 * M * N * K / (e0.elapsed_time(e1) / 16 * 1e-3) / 1e12,
                    "config": "8192^3 e4m3 x e4m3 -> bf16, per-tensor scales, torch._scaled_mm, 16 launches"}
                del a8, b8
            except Exception as exc:  # the private API may differ between torch builds
                extra["library_fp8_gemm_yardstick"] = {"unavailable": str(exc)[:200]}

    peak, hbm_peak, peak_src = measured_peaks()
    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            r = cpu_gemm_rate(12.0, 0)
            cpu = {"value": r["tflops"], "unit": "TFLOP/s", "cores": r["threads"], "kind": "port",
                   "sample": f"rows [0,{r['rows']}) of the same 8192^3 GEMM ({r['seconds']:.1f} s), "
                             "oracle port of the reference's cpu_gemm"}
        per_gpu = value / world
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "gemm_bf16_8192x8192x8192", "layout": "A[M,K] B[K,N] row-major, fp32 acc",
                       "tile": f"{bm}x{bn}x64 per CTA pair (cta_group::2), 6-stage TMA ring, persistent, grouped-M 8",
                       "parallelism": f"N-split x{world}" if world > 1 else "single GPU",
                       "l2": "operands 403 MB per step exceed the 126 MB L2; no flush between steps"},
            "per_gpu_tflops": per_gpu,
            "pct_of_nominal_peak_2250": 100.0 * per_gpu / 2250.0,
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s",
                         "frac": per_gpu / peak, "traffic": GEMM_DRAM_TRAFFIC_BYTES,
                         "peak_source": f"{peak_src} cuBLAS bf16 burst",
                         "peak_sustained": SUSTAINED_BF16_TFLOPS,
                         "frac_of_sustained": (per_gpu / SUSTAINED_BF16_TFLOPS) if SUSTAINED_BF16_TFLOPS else None,
                         "note": "the MMA-issuing thread measures 1048 cycles per 1024 tensor-pipe cycles of work "
                                 "(cycle accounting of the diagnostic trace build); the SM clock under the 1 kW cap sets the rest"},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "api": "api.HostGemm (b200tile_gemm_host): pinned host A, B, C; pipelined in 1024-row slabs",
                    "serial_copy_launch_copy_ms": e2e_serial_ms,
                    "gpu_launches_per_step": -(-M // 1024)},
            "gpu_launches": args.steps * world,
            "clocks": clocks,
            "extra": extra,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-fmha", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 and world == 1:
        # convenience: re-launch under torchrun so that `python bench.py --gpus N` works by itself
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29531", os.path.abspath(__file__)] + sys.argv[1:]
        return subprocess.call(cmd)
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
