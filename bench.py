#!/usr/bin/env python
"""Benchmark of the dense-contraction hot path on N B200s of one node.

Headline workload: bf16 GEMM M=N=K=8192, A[M,K] and B[K,N] ~ N(0,1)/sqrt(K)
rounded to bf16, fp32 accumulation, bf16 output.  A "step" is one GEMM launch.  With N>1 GPUs the
weight columns are split (rank r owns B[:, r*N/G:(r+1)*N/G] and the matching columns of C, A is
replicated), so the total work is fixed ("strong" scaling) and no data-path collective runs.

`value` is the whole-job TFLOP/s with operands resident in HBM; `e2e` is the same metric through
the public launcher API with HOST buffers (pinned host -> device copies of A and B and a
device -> host read of C inside the timed region).  `roofline` compares the kernel with the
measured cuBLAS bf16 peak of this pool; `cpu_baseline` times the CPU oracle (a port of the
reference's `cpu_gemm`) on a bounded slab.  The other workloads of the path (FMHA forward 8 x 32 x 4096 x
128 non-causal and causal, the fp8 block-scaled GEMM 8192 x 28672 x 8192, the NVFP4 GEMM 4096 / 16 x 14336 x
4096 and the f32 512^3 GEMM) are measured the same way and reported as `by_config` entries inside `roofline`,
`cpu_baseline` and `e2e`; `extra` holds compact figures for the neighbouring kernels.

`--case <kernel> ...` runs one kernel a few times on a small problem (what the `ncu` summaries under profiles/
were captured on); see `run_case`.

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
# dram__bytes_read.sum + dram__bytes_write.sum per launch of gemm_tc_pair_kernel<., ., 512> on the full-size 8192^3
# problem: 984.2 MB + 146.2 MB, a one-pass ncu capture of two launches of `bench.py --case gemm --m 8192 --n 8192
# --k 8192 --config 3` (profiles/gemm_bf16_pair.md); the 256-wide tile's figure, scaled from a quarter-size capture,
# was 1.27 GB.
GEMM_DRAM_TRAFFIC_BYTES = 984_226_816 + 146_217_728


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
            time.sleep(0.002)

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
                "reasons": reasons, "samples": len(rows), "source": "nvml, 2 ms poll",
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
NOMINAL_BF16, NOMINAL_FP8, NOMINAL_FP4 = 2250.0, 4500.0, 9000.0   # dense TFLOP/s per GPU (fp8 / fp4 = 2x / 4x bf16)


class Ctx:
    """What every workload of the GPU arm needs: the library, the stream, the ranks and a device timer."""

    def __init__(self, lib, stream, dev, world, rank):
        import torch
        self.lib, self.stream, self.dev, self.world, self.rank = lib, stream, dev, world, rank
        self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.launches = 0

    def barrier(self):
        import torch
        import torch.distributed as dist
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(self, fn, iters, warm=3):
        """ms per call: CUDA events on the launching stream, barrier + synchronize on both sides, max over ranks."""
        from cutile_rs_b200 import sharding
        for _ in range(warm):
            fn()
        self.barrier()
        self.e0.record(self.stream)
        for _ in range(iters):
            fn()
        self.e1.record(self.stream)
        self.barrier()
        return sharding.max_over_ranks(self.e0.elapsed_time(self.e1), self.dev) / iters


def _roof(bound, achieved, peak, unit, ms, source, **more):
    d = {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
         "frac": (achieved / peak) if peak else None, "ms": ms, "peak_source": source}
    d.update(more)
    return d


def _pin_like(t):
    import torch
    return torch.empty(t.shape, dtype=t.dtype).pin_memory()


def bench_fmha(ctx, by, cpu_by, e2e_by, do_cpu):
    """FMHA forward bf16 8 x 32 x 4096 x 128 (b x h split over the ranks), non-causal and causal."""
    import ctypes
    import torch
    from cutile_rs_b200 import _lib, api, sharding, workloads
    lib, stream, dev, world = ctx.lib, ctx.stream, ctx.dev, ctx.world
    peak, _, src = measured_peaks()
    B_, H_, S_, D_ = 8, 32, 4096, 128
    p0, p1 = sharding.split_range(B_ * H_, world, ctx.rank, 1)
    nb = p1 - p0
    g = torch.Generator(device="cuda").manual_seed(workloads.SEED_BASE + 2 + ctx.rank)
    q = torch.randn(nb, S_, D_, generator=g, device=dev).bfloat16()
    k = torch.randn(nb, S_, D_, generator=g, device=dev).bfloat16()
    v = torch.randn(nb, S_, D_, generator=g, device=dev).bfloat16()
    o = torch.empty_like(q)
    st = (ctypes.c_int64 * 2)(S_ * D_, D_)
    scale = 1.0 / math.sqrt(D_)
    qh, kh, vh, oh = q.cpu().pin_memory(), k.cpu().pin_memory(), v.cpu().pin_memory(), _pin_like(o)
    for causal in (False, True):
        name = "fmha_causal" if causal else "fmha_noncausal"

        def fstep():
            _lib.check(lib.b200tile_fmha_fwd(b"bf16", q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), 1, nb, nb,
                                             S_, S_, D_, st, st, st, st, scale, int(causal), 0, stream.cuda_stream))
        ms = ctx.timed(fstep, 10)
        flops = workloads.fmha_flops(B_, H_, S_, D_, causal)
        tf = flops / (ms * 1e-3) / 1e12 / world
        by[name] = _roof("tensor", tf, peak, "TFLOP/s", ms, f"{src} cuBLAS bf16 burst", frac_of_nominal_2250=tf / NOMINAL_BF16)

        # end to end: api.HostFmha, eight groups of (batch, head) problems uploaded / attended / downloaded on three streams
        plan = api.HostFmha(nb, S_, D_, "bf16", causal=causal, group=max(1, nb // 8))

        def estep():
            plan(qh, kh, vh, oh, scale, stream)
        ems = ctx.timed(estep, 3, warm=1)
        del plan
        e2e_by[name] = {"value": flops / (ems * 1e-3) / 1e12, "unit": "TFLOP/s", "ms": ems,
                        "h2d_bytes_per_step": 3 * B_ * H_ * S_ * D_ * 2, "d2h_bytes_per_step": B_ * H_ * S_ * D_ * 2,
                        "note": "api.HostFmha: pinned host Q, K, V, O; pipelined in eight groups of problems"}
        ctx.launches += 13 + 4 * 8
        if do_cpu:
            from oracle import oracle
            nbh, rows = 4, 256
            qf = q[:nbh].float().cpu().numpy().reshape(1, nbh, S_, D_)
            kf = k[:nbh].float().cpu().numpy().reshape(1, nbh, S_, D_)
            vf = v[:nbh].float().cpu().numpy().reshape(1, nbh, S_, D_)
            thr = oracle.max_threads()
            t0 = time.perf_counter()
            oracle.fmha_ref_cpu(qf, kf, vf, scale, causal=causal, bh=(0, nbh), rows=(S_ - rows, S_), threads=thr)
            dt = time.perf_counter() - t0
            rf = nbh * rows * 4.0 * S_ * D_ / (2.0 if causal else 1.0)
            cpu_by[name] = {"value": rf / dt / 1e12, "unit": "TFLOP/s", "cores": thr, "kind": "port",
                            "sample": f"fmha_ref_cpu port, {nbh} (b,h) x last {rows} query rows, {dt:.1f} s"}
    # the CTA-pair configuration of the same non-causal shape, through the launcher mirror
    from cutile_rs_b200 import api, launch
    qd, kd, vd = (api.from_torch(t_.view(1, nb, S_, D_)) for t_ in (q, k, v))
    od = [api.from_torch(o).partition([1, 128, D_])]
    fopts = launch.CompileOptions(num_cta_in_cga=2)

    def pstep():
        (od[0], *_r) = launch.fmha(od[0], qd, kd, vd, scale, 0, 1, causal=False).compile_options(fopts).async_on(stream)
    pms = ctx.timed(pstep, 10)
    ctx.launches += 13
    return {"fmha_noncausal_cta_pairs": {"tflops_per_gpu": workloads.fmha_flops(B_, H_, S_, D_, False) / (pms * 1e-3) / 1e12 / world,
                                         "ms": pms}}


def bench_fp8(ctx, by, cpu_by, e2e_by, do_cpu):
    """fp8 e4m3 GEMM 8192 x 28672 x 8192 with fp32 scales per 1x128 / 128x128 block (weight rows split over the ranks),
    and the same shape as MXFP8 (e8m0 scale per 32, applied by the tensor core)."""
    import torch
    from cutile_rs_b200 import _lib, api, quant, sharding, workloads
    lib, stream, dev, world = ctx.lib, ctx.stream, ctx.dev, ctx.world
    g = torch.Generator(device="cuda").manual_seed(workloads.SEED_BASE + 3)
    m8, n8, k8 = 8192, 28672, 8192
    r0, r1 = sharding.split_range(n8, world, ctx.rank, 256)
    nl = r1 - r0
    xq, xs = quant.quant_fp8_block(torch.randn(m8, k8, device=dev, generator=g), 1, 128)
    yq, ys = quant.quant_fp8_block(torch.randn(nl, k8, device=dev, generator=g), 128, 128)
    z8 = torch.empty(m8, nl, dtype=torch.bfloat16, device=dev)

    def f8step():
        _lib.check(lib.b200tile_linear_fp8_blk128(xq.data_ptr(), yq.data_ptr(), xs.data_ptr(), ys.data_ptr(), z8.data_ptr(),
                                                  b"bf16", m8, nl, k8, k8, k8, nl, k8 // 128, k8 // 128, 1.0,
                                                  stream.cuda_stream))
    ms = ctx.timed(f8step, 5)
    flops = workloads.gemm_flops(m8, n8, k8)
    tf = flops / (ms * 1e-3) / 1e12 / world
    by["fp8_blk128"] = _roof("tensor", tf, NOMINAL_FP8, "TFLOP/s", ms, "nominal dense fp8 = 2 x 2250 (no measured fp8 peak)")
    hx, hy, hxs, hys, hz = xq.cpu().pin_memory(), yq.cpu().pin_memory(), xs.cpu().pin_memory(), ys.cpu().pin_memory(), _pin_like(z8)

    # end to end: api.HostRowPipeline, weights first, then 1024-row slabs uploaded / multiplied / downloaded on three streams
    pipe = api.HostRowPipeline(m8, 1024)

    def f8rows(a0, a1, s_):
        _lib.check(lib.b200tile_linear_fp8_blk128(xq[a0:].data_ptr(), yq.data_ptr(), xs[a0:].data_ptr(), ys.data_ptr(),
                                                  z8[a0:].data_ptr(), b"bf16", a1 - a0, nl, k8, k8, k8, nl, k8 // 128,
                                                  k8 // 128, 1.0, s_.cuda_stream))

    def estep():
        pipe([(hy, yq), (hys, ys)], [(hx, xq), (hxs, xs)], [(z8, hz)], f8rows, stream)
    ems = ctx.timed(estep, 3, warm=1)
    e2e_by["fp8_blk128"] = {"value": flops / (ems * 1e-3) / 1e12, "unit": "TFLOP/s", "ms": ems,
                            "h2d_bytes_per_step": world * (hx.numel() + hxs.numel() * 4) + n8 * k8 + (n8 // 128) * (k8 // 128) * 4,
                            "d2h_bytes_per_step": m8 * n8 * 2,
                            "note": "api.HostRowPipeline: all operands uploaded, pipelined in 1024-row slabs"}
    ctx.launches += 8 + 4 * 8
    if do_cpu:
        from oracle import oracle
        rows, cols = 16, 2048
        thr = oracle.max_threads()
        xqn, xsn = hx[:128].numpy().view("uint8"), hxs[:128].numpy()
        yqn, ysn = hy[:cols].numpy().view("uint8"), hys[:cols // 128].numpy()
        t0 = time.perf_counter()
        xa = oracle.dequant_fp8_block(xqn, xsn, 1, 128)[:rows]
        ya = oracle.dequant_fp8_block(yqn, ysn, 128, 128)
        oracle.cpu_gemm_nt(xa, ya, threads=thr)
        dt = time.perf_counter() - t0
        cpu_by["fp8_blk128"] = {"value": 2.0 * rows * cols * k8 / dt / 1e12, "unit": "TFLOP/s", "cores": thr, "kind": "port",
                                "sample": f"dequantise + cpu_gemm port on C[0:{rows}, 0:{cols}], K={k8}, {dt:.1f} s"}
    del hx, hy, hxs, hys, hz
    # MXFP8 on the same shape
    xm, xms = quant.quant_mxfp8(torch.randn(m8, k8, device=dev, generator=g))
    ym, yms = quant.quant_mxfp8(torch.randn(nl, k8, device=dev, generator=g))
    wsm = lib.b200tile_linear_mxfp8_workspace_bytes(m8, nl, k8)
    wsb8 = torch.empty(wsm, dtype=torch.uint8, device=dev)

    def mx8step():
        _lib.check(lib.b200tile_linear_mxfp8(xm.data_ptr(), ym.data_ptr(), xms.data_ptr(), yms.data_ptr(), z8.data_ptr(),
                                             b"bf16", m8, nl, k8, k8, k8, nl, k8 // 32, k8 // 32, 1.0, wsb8.data_ptr(), wsm,
                                             stream.cuda_stream))
    msm = ctx.timed(mx8step, 5)
    ctx.launches += 8 * 2
    tfm = flops / (msm * 1e-3) / 1e12 / world
    by["mxfp8"] = _roof("tensor", tfm, NOMINAL_FP8, "TFLOP/s", msm, "nominal dense fp8 = 2 x 2250 (no measured fp8 peak)",
                        how="typed entry point (scale pre-pass + CTA-pair GEMM), e8m0 scale per 32")
    hx, hy, hxs, hys, hz = xm.cpu().pin_memory(), ym.cpu().pin_memory(), xms.cpu().pin_memory(), yms.cpu().pin_memory(), _pin_like(z8)

    def mx8rows(a0, a1, s_):
        _lib.check(lib.b200tile_linear_mxfp8(xm[a0:].data_ptr(), ym.data_ptr(), xms[a0:].data_ptr(), yms.data_ptr(),
                                             z8[a0:].data_ptr(), b"bf16", a1 - a0, nl, k8, k8, k8, nl, k8 // 32, k8 // 32,
                                             1.0, wsb8.data_ptr(), wsm, s_.cuda_stream))

    def emstep():
        pipe([(hy, ym), (hys, yms)], [(hx, xm), (hxs, xms)], [(z8, hz)], mx8rows, stream)
    emm = ctx.timed(emstep, 3, warm=1)
    ctx.launches += 4 * 2 * 8
    e2e_by["mxfp8"] = {"value": flops / (emm * 1e-3) / 1e12, "unit": "TFLOP/s", "ms": emm,
                       "h2d_bytes_per_step": world * (hx.numel() + hxs.numel()) + n8 * k8 + n8 * k8 // 32,
                       "d2h_bytes_per_step": m8 * n8 * 2,
                       "note": "api.HostRowPipeline: all operands uploaded, pipelined in 1024-row slabs"}
    if do_cpu:
        from oracle import oracle
        rows, cols = 16, 2048
        thr = oracle.max_threads()
        t0 = time.perf_counter()
        xa = oracle.dequant_mxfp8(hx[:rows].numpy(), hxs[:rows].numpy())
        ya = oracle.dequant_mxfp8(hy[:cols].numpy(), hys[:cols].numpy())
        oracle.cpu_gemm_nt(xa, ya, threads=thr)
        dt = time.perf_counter() - t0
        cpu_by["mxfp8"] = {"value": 2.0 * rows * cols * k8 / dt / 1e12, "unit": "TFLOP/s", "cores": thr, "kind": "port",
                           "sample": f"dequantise + cpu_gemm port on C[0:{rows}, 0:{cols}], K={k8}, {dt:.1f} s"}
    del hx, hy, hxs, hys, hz
    return {"gemm_mxfp8_8192x28672x8192": {"tflops_per_gpu": tfm, "ms": msm, "frac_of_nominal_4500": tfm / NOMINAL_FP8}}


def bench_nvfp4(ctx, by, cpu_by, e2e_by, do_cpu):
    """NVFP4 GEMM N=14336, K=4096 at M=4096 and the decode shape M=16 (weight rows split over the ranks), through the
    reference's own kernel name: b200tile_launch("linear_tile", ...)."""
    import torch
    from cutile_rs_b200 import _lib, api, launch, quant, sharding, workloads
    lib, stream, dev, world = ctx.lib, ctx.stream, ctx.dev, ctx.world
    _, hbm_peak, src = measured_peaks()
    g = torch.Generator(device="cuda").manual_seed(workloads.SEED_BASE + 4)
    n4, k4 = 14336, 4096
    r0, r1 = sharding.split_range(n4, world, ctx.rank, 256)
    nl = r1 - r0
    yp, ysc, gy = quant.quant_nvfp4(torch.randn(nl, k4, device=dev, generator=g))
    y, sy = api.from_torch(yp, "f4e2m1fnx2"), api.from_torch(ysc, "f8e4m3fn")
    extra = {}
    for m4 in (4096, 16):
        name = f"nvfp4_m{m4}"
        xp, xsc, gx = quant.quant_nvfp4(torch.randn(m4, k4, device=dev, generator=g))
        x, sx = api.from_torch(xp, "f4e2m1fnx2"), api.from_torch(xsc, "f8e4m3fn")
        z4 = torch.empty(m4, nl, dtype=torch.bfloat16, device=dev)
        zp = [api.from_torch(z4).partition([16, 128])]
        alpha = gx * gy

        # The generic call is captured once and replayed (CUDA graph): the launcher mirror's Python costs ~100 us per
        # call, more than the kernel at decode sizes and on the shards of a multi-GPU run.
        cap = torch.cuda.Stream()
        cap.wait_stream(stream)
        (zp[0], *_r) = launch.linear_tile(zp[0], x, y, sx, sy, alpha).sync_on(cap)   # the capture stream's scratch
        graph = [launch.linear_tile(zp[0], x, y, sx, sy, alpha).graph_on(cap)]
        if m4 <= 128:
            # decode: first with the per-call weight-scale pre-pass, then with the weight scales (constants of the
            # model) laid out once and registered: the same generic call then runs one kernel.
            extra["nvfp4_m16_unregistered_weight_scales_us"] = ctx.timed(lambda: graph[0].launch(), 20) * 1e3
            prep = launch.nvfp4_prepare_weight_scales(sy, nl, k4, 0)
            launch.nvfp4_register_weight_scales(sy, nl, k4, prep, 0)
            torch.cuda.synchronize()
            graph[0] = launch.linear_tile(zp[0], x, y, sx, sy, alpha).graph_on(cap)
            ctx.launches += 23 * 2 + 3

        def f4step():
            graph[0].launch()
        ms = ctx.timed(f4step, 20 if m4 <= 128 else 10)
        ctx.launches += 23 if m4 <= 128 else 13 * 2
        chain_how = None
        if m4 <= 128:
            # A serving step runs its linear layers back to back, each over its own weights: 16 calls of one captured
            # graph over 6 weight matrices (6 x 33.5 MB on one GPU, more than L2), time per call.  The decode-sized
            # kernel is launched with programmatic stream serialisation, so a call sets itself up and starts streaming
            # its (registered, i.e. constant) weights while its predecessor drains.
            extra["nvfp4_m16_single_call_graph_replay_us"] = ms * 1e3
            sets = [(y, sy, prep, gy)]
            for _ in range(5):
                yp_i, ysc_i, gy_i = quant.quant_nvfp4(torch.randn(nl, k4, device=dev, generator=g))
                y_i, sy_i = api.from_torch(yp_i, "f4e2m1fnx2"), api.from_torch(ysc_i, "f8e4m3fn")
                prep_i = launch.nvfp4_prepare_weight_scales(sy_i, nl, k4, 0)
                launch.nvfp4_register_weight_scales(sy_i, nl, k4, prep_i, 0)
                sets.append((y_i, sy_i, prep_i, gy_i))
            torch.cuda.synchronize()
            calls = 16

            def record(r):
                for j in range(calls):
                    w = sets[j % len(sets)]
                    r(launch.linear_tile(zp[0], x, w[0], sx, w[1], gx * w[3]))
            chain = launch.CudaGraph.scope(cap, record)
            ms = ctx.timed(lambda: chain.launch(), 10) / calls
            ctx.launches += 13 * calls
            chain_how = (f"{calls} generic linear_tile calls of one captured decode step over {len(sets)} weight matrices "
                         f"({len(sets) * (nl * k4 // 2 + nl * k4 // 16) / 1e6:.0f} MB, more than L2), registered weight scales; "
                         "time per call")
        flops = workloads.gemm_flops(m4, n4, k4)
        nbytes = (m4 * k4 // 2 + m4 * k4 // 16 + n4 * k4 // 2 + n4 * k4 // 16 + m4 * n4 * 2)
        if m4 <= 128:
            gbs = nbytes / (ms * 1e-3) / 1e9 / world
            by[name] = _roof("hbm", gbs, hbm_peak, "GB/s", ms, f"{src} copy bandwidth", algorithmic_bytes=nbytes,
                             tflops=flops / (ms * 1e-3) / 1e12 / world,
                             how=chain_how)
        else:
            tf = flops / (ms * 1e-3) / 1e12 / world
            by[name] = _roof("tensor", tf, NOMINAL_FP4, "TFLOP/s", ms, "nominal dense fp4 = 4 x 2250 (no measured fp4 peak)",
                             how="generic linear_tile call (scale pre-pass + GEMM), CUDA-graph replay")
        hx, hxs, hy, hys, hz = xp.cpu().pin_memory(), xsc.cpu().pin_memory(), yp.cpu().pin_memory(), ysc.cpu().pin_memory(), _pin_like(z4)

        def estep():
            xp.copy_(hx, non_blocking=True)
            xsc.copy_(hxs, non_blocking=True)
            if m4 > 128:                 # decode: the weights stay resident, as they do in serving
                yp.copy_(hy, non_blocking=True)
                ysc.copy_(hys, non_blocking=True)
            f4step()
            hz.copy_(z4, non_blocking=True)
        ems = ctx.timed(estep, 5, warm=1)
        ctx.launches += 6 * 2
        e2e_by[name] = {"value": flops / (ems * 1e-3) / 1e12, "unit": "TFLOP/s", "ms": ems,
                        "h2d_bytes_per_step": world * (hx.numel() + hxs.numel()) + (0 if m4 <= 128 else n4 * k4 // 2 + n4 * k4 // 16),
                        "d2h_bytes_per_step": m4 * n4 * 2,
                        "note": "weights resident, CUDA-graph replay" if m4 <= 128 else "all operands uploaded, CUDA-graph replay"}
        if do_cpu:
            from oracle import oracle
            rows, cols = min(m4, 64), 2048
            thr = oracle.max_threads()
            t0 = time.perf_counter()
            xa = oracle.dequant_nvfp4(hx[:rows].numpy(), hxs[:rows].numpy())
            ya = oracle.dequant_nvfp4(hy[:cols].numpy(), hys[:cols].numpy())
            oracle.cpu_gemm_nt(xa, ya, alpha=alpha, threads=thr)
            dt = time.perf_counter() - t0
            cpu_by[name] = {"value": 2.0 * rows * cols * k4 / dt / 1e12, "unit": "TFLOP/s", "cores": thr, "kind": "port",
                            "sample": f"dequantise + cpu_gemm port on C[0:{rows}, 0:{cols}], K={k4}, {dt:.1f} s"}
        if m4 <= 128:
            for w in sets:
                launch.nvfp4_unregister_weight_scales(w[1])
    # MXFP4 (the same packed operands with power-of-two scales per 32 elements) at M = 4096, typed entry point
    m4 = 4096
    xq, xqs = quant.quant_mxfp4(torch.randn(m4, k4, device=dev, generator=g))
    yq, yqs = quant.quant_mxfp4(torch.randn(nl, k4, device=dev, generator=g))
    zq = torch.empty(m4, nl, dtype=torch.bfloat16, device=dev)
    need = lib.b200tile_linear_mxfp4_workspace_bytes(m4, nl, k4)
    wsq = torch.empty(need, dtype=torch.uint8, device=dev)

    def mx4step():
        _lib.check(lib.b200tile_linear_mxfp4(xq.data_ptr(), yq.data_ptr(), xqs.data_ptr(), yqs.data_ptr(), zq.data_ptr(),
                                             b"bf16", m4, nl, k4, k4 // 2, k4 // 2, nl, k4 // 32, k4 // 32, 1.0,
                                             wsq.data_ptr(), need, stream.cuda_stream))
    msq = ctx.timed(mx4step, 10)
    ctx.launches += 13 * 2        # scale pre-pass + CTA-pair GEMM per call
    tfq = workloads.gemm_flops(m4, n4, k4) / (msq * 1e-3) / 1e12 / world
    extra["gemm_mxfp4_4096x14336x4096"] = {"tflops_per_gpu": tfq, "ms": msq, "frac_of_nominal_9000": tfq / NOMINAL_FP4}
    return extra


def bench_f32(ctx, by, cpu_by, e2e_by, do_cpu):
    """f32 GEMM 512^3, the reference's CPU-runnable configuration: exact fp32 arithmetic on the CUDA cores (replicas
    only: every rank runs the whole problem)."""
    import torch
    from cutile_rs_b200 import api, launch, workloads
    stream = ctx.stream
    a, b = workloads.gemm_f32_inputs(512, 512, 512)
    x, y = api.copy_host_to_device(a), api.copy_host_to_device(b)
    z = [api.zeros([512, 512]).partition([64, 64])]
    gen = ["f32", "64", "64", "16"]

    # captured once and replayed: the launcher mirror's Python costs more per call than this kernel runs
    cap = torch.cuda.Stream()
    cap.wait_stream(stream)
    (z[0], *_r) = launch.gemm(z[0], x, y).generics(gen).sync_on(cap)
    graph = launch.gemm(z[0], x, y).generics(gen).graph_on(cap)

    def step():
        graph.launch()
    ms = ctx.timed(step, 20)
    flops = workloads.gemm_flops(512, 512, 512)
    by["f32_512"] = _roof("none", flops / (ms * 1e-3) / 1e9, None, "GFLOP/s", ms,
                          "correctness configuration: bit-exact fp32, no tensor path, no roofline claim",
                          how="generic gemm launcher, CUDA-graph replay")
    ap, bp = api.pin(a), api.pin(b)
    cp = torch.empty(512, 512).pin_memory()

    def estep():
        xa = api.copy_host_to_device(ap, stream=stream)
        yb = api.copy_host_to_device(bp, stream=stream)
        (zz, _, _) = launch.gemm(z[0], xa, yb).generics(gen).async_on(stream)
        cp.copy_(zz.unpartition().storage, non_blocking=True)
    ems = ctx.timed(estep, 10, warm=2)
    ctx.launches += 23 + 12
    e2e_by["f32_512"] = {"value": flops / (ems * 1e-3) / 1e9, "unit": "GFLOP/s", "ms": ems,
                         "h2d_bytes_per_step": 2 * 512 * 512 * 4, "d2h_bytes_per_step": 512 * 512 * 4}
    if do_cpu:
        from oracle import oracle
        an, bn = a.numpy(), b.numpy()
        t0 = time.perf_counter()
        oracle.cpu_gemm(an, bn, threads=1)
        t1 = time.perf_counter() - t0
        thr = oracle.max_threads()
        t0 = time.perf_counter()
        oracle.cpu_gemm(an, bn, threads=thr)
        tn = time.perf_counter() - t0
        cpu_by["f32_512"] = {"value": flops / tn / 1e9, "unit": "GFLOP/s", "cores": thr, "kind": "port",
                             "sample": f"cpu_gemm port on the whole 512^3 problem: {tn * 1e3:.1f} ms on {thr} threads, "
                                       f"{t1 * 1e3:.1f} ms single-threaded as written"}


def bench_neighbours(ctx):
    """Compact figures for the other kernels on and around the path (numbers only; shapes in the names)."""
    import ctypes
    import torch
    from cutile_rs_b200 import _lib, launch, sharding, workloads
    lib, stream, dev, world, rank = ctx.lib, ctx.stream, ctx.dev, ctx.world, ctx.rank
    hbm = measured_peaks()[1]
    I2 = ctypes.c_int64 * 2
    out = {}
    g = torch.Generator(device="cuda").manual_seed(workloads.SEED_BASE + 9)

    # split-KV GQA decode attention + merge, K/V heads split over the ranks, K/V sets rotated (inputs > L2)
    HKV, GRP, SKV, DD = 8, 4, 65536, 128
    h0, h1 = sharding.split_range(HKV, world, rank, 1)
    hl = h1 - h0
    if hl > 0:
        ns = max(1, lib.b200tile_num_sms() // hl)
        nbuf = 4
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
        msd = ctx.timed(dstep, 20)
        del kds, vds
    else:
        ctx.barrier()
        ctx.barrier()
        msd = sharding.max_over_ranks(0.0, dev)
    gbs = 2 * HKV * SKV * DD * 2 / (msd * 1e-3) / 1e9 / world
    out["decode_attn_8kvh_x4_65536_d128"] = {"gbs_per_gpu": gbs, "us": msd * 1e3, "frac_of_measured_hbm": gbs / hbm}
    ctx.launches += 23 * 2

    # MoE grouped GEMM: 64 experts x 512 tokens x 4096 x 7168 bf16 (experts split over the ranks)
    E, GM, GN, GK = 64, 512, 4096, 7168
    e0_, e1_ = sharding.split_range(E, world, rank, 1)
    ne = e1_ - e0_
    ga = torch.randn(ne, GM, GK, device=dev, generator=g).bfloat16() / 8
    gb = torch.randn(ne, GK, GN, device=dev, generator=g).bfloat16() / 8
    gc = torch.empty(ne, GM, GN, device=dev, dtype=torch.bfloat16)
    tabs = launch.group_gemm_tables(list(ga), list(gb), list(gc))
    need = lib.b200tile_group_gemm_workspace_bytes(ne)
    gws = torch.empty(need + 128, dtype=torch.uint8, device=dev)
    gwp = (gws.data_ptr() + 127) // 128 * 128

    def gstep():
        _lib.check(lib.b200tile_group_gemm(b"bf16", *(t_.cu_deviceptr() for t_ in tabs), ne, 256, gwp, need,
                                           stream.cuda_stream))
    msg = ctx.timed(gstep, 5)
    tfg = 2.0 * E * GM * GN * GK / (msg * 1e-3) / 1e12 / world
    out["group_gemm_64x512x4096x7168"] = {"tflops_per_gpu": tfg, "ms": msg, "frac_of_nominal_2250": tfg / NOMINAL_BF16}
    ctx.launches += 8 * 2
    del ga, gb, gc

    # residual add + RMSNorm, token rows split over the ranks, two tensor sets alternated (inputs > L2)
    NT, NH = 16384, 8192
    t0_, t1_ = sharding.split_range(NT, world, rank, 1)
    nt = t1_ - t0_
    sets = [(torch.randn(nt, NH, device=dev, generator=g).half(), torch.randn(nt, NH, device=dev, generator=g).half(),
             torch.empty(nt, NH, device=dev, dtype=torch.float16), torch.empty(nt, NH, device=dev, dtype=torch.float16))
            for _ in range(2)]
    wn = torch.ones(NH, device=dev, dtype=torch.float16)
    flip = [0]

    def nstep():
        r_, x_, o_, ro_ = sets[flip[0] & 1]
        flip[0] += 1
        _lib.check(lib.b200tile_add_rms_norm(b"f16", r_.data_ptr(), x_.data_ptr(), wn.data_ptr(), o_.data_ptr(),
                                             ro_.data_ptr(), nt, NH, NH, NH, NH, NH, 1e-5, stream.cuda_stream))
    msn = ctx.timed(nstep, 20)
    gbn = 4.0 * NT * NH * 2 / (msn * 1e-3) / 1e9 / world
    out["add_rms_norm_16384x8192"] = {"gbs_per_gpu": gbn, "us": msn * 1e3, "frac_of_measured_hbm": gbn / hbm}
    ctx.launches += 23
    del sets

    # rotary embedding and the fused QK-norm + RoPE + KV-cache write, token rows split over the ranks
    RT, RH, RD = 32768, 32, 128
    t0_, t1_ = sharding.split_range(RT, world, rank, 1)
    rt = t1_ - t0_
    rsets = [(torch.randn(rt, RH, RD, device=dev).half(), torch.empty(rt, RH, RD, device=dev, dtype=torch.float16))
             for _ in range(2)]
    inv_f = (1.0 / 10000.0 ** (torch.arange(0, RD, 2, dtype=torch.float32, device=dev) / RD)).contiguous()
    rst = I2(RH * RD, RD)
    rflip = [0]

    def rstep():
        x_, o_ = rsets[rflip[0] & 1]
        rflip[0] += 1
        _lib.check(lib.b200tile_rope_seq(b"f16", x_.data_ptr(), inv_f.data_ptr(), o_.data_ptr(), rt, RH, RD, rst, rst,
                                         t0_, None, stream.cuda_stream))
    msr = ctx.timed(rstep, 20)
    gbr = 2.0 * RT * RH * RD * 2 / (msr * 1e-3) / 1e9 / world
    out["rope_seq_32768x32x128"] = {"gbs_per_gpu": gbr, "us": msr * 1e3, "frac_of_measured_hbm": gbr / hbm}
    ctx.launches += 23
    del rsets
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
    msq = ctx.timed(qstep, 20)
    gbq = 2.0 * QT * (QH + 2 * KVH) * RD * 2 / (msq * 1e-3) / 1e9 / world
    out["qk_norm_rope_kv_16384tok"] = {"gbs_per_gpu": gbq, "us": msq * 1e3, "frac_of_measured_hbm": gbq / hbm}
    ctx.launches += 23
    del qq, qk_, qv, qo_, kc_, vc_

    # LM head fused with the block argmax (vocabulary rows split over the ranks)
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
    msl = ctx.timed(lstep, 20)
    gbl = 2.0 * LV * LK / (msl * 1e-3) / 1e9 / world
    out["lm_head_argmax_128256x4096"] = {"gbs_per_gpu": gbl, "us": msl * 1e3, "frac_of_measured_hbm": gbl / hbm}
    ctx.launches += 23 * 2
    del lw

    # SiLU(gate) * up as a kernel of its own
    ST, SI = 8192, 14336
    t0_, t1_ = sharding.split_range(ST, world, rank, 1)
    st_ = t1_ - t0_
    sg = torch.randn(st_, SI, device=dev).half()
    su = torch.randn(st_, SI, device=dev).half()
    so = torch.empty_like(sg)

    def sstep():
        _lib.check(lib.b200tile_silu_mul_2d(b"f16", so.data_ptr(), sg.data_ptr(), su.data_ptr(), st_, SI, SI, SI, SI,
                                            stream.cuda_stream))
    mss = ctx.timed(sstep, 20)
    gbs_ = 3.0 * ST * SI * 2 / (mss * 1e-3) / 1e9 / world
    out["silu_mul_8192x14336"] = {"gbs_per_gpu": gbs_, "us": mss * 1e3, "frac_of_measured_hbm": gbs_ / hbm}
    ctx.launches += 23
    return out


def bench_single_gpu_yardsticks(ctx, step, flops, x, y, n_local):
    """1-GPU only: the reference's published timing protocol on all-ones f16 operands, and library kernels
    (cuBLAS through torch.matmul, cuBLASLt fp8 through torch._scaled_mm) as yardsticks on the same box."""
    import torch
    from cutile_rs_b200 import _lib
    lib, stream, dev = ctx.lib, ctx.stream, ctx.dev
    out = {}
    ones_a = torch.ones(M, K, dtype=torch.float16, device=dev)
    ones_b = torch.ones(K, N, dtype=torch.float16, device=dev)
    ones_c = torch.empty(M, N, dtype=torch.float16, device=dev)

    # 5 warm-up launches, median over 10 samples of 3 back-to-back launches between stream syncs, host clock
    # (cutile-benchmarks/paper/sec5_exp1_safety_overhead/rust/gemm/src/main.rs:629-631,1289-1322); once with
    # fp32 accumulators and once with the f16 accumulators of the published kernel (benches/gemm.rs:20-41)
    for key, cfg, acc in (("gemm_f16_ones_published_protocol", 3, "fp32"),
                          ("gemm_f16_ones_published_protocol_f16_accumulators", 4, "f16, as in the published run")):
        def ones_step():
            _lib.check(lib.b200tile_gemm(b"f16", 0, ones_a.data_ptr(), ones_b.data_ptr(), ones_c.data_ptr(), 1, M, N, K,
                                         K, N, N, 0, 0, 0, 0, cfg, 8, 0, stream.cuda_stream))
        ones_c.fill_(float("nan"))
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
        out[key] = {
            "tflops": flops / med / 1e12, "median_us": med * 1e6, "published_reference_tflops": 2068.88,
            "result_is_k_everywhere": bool((ones_c[::997, ::991].float() == float(K)).all().item()),
            "tile": "256x512 per CTA pair", "accumulator": acc}
        ctx.launches += 35
    del ones_a, ones_b, ones_c
    a_t, b_t, c_t = x.storage, y.storage, torch.empty((M, n_local), dtype=torch.bfloat16, device=dev)
    for _ in range(3):          # library initialisation and heuristics stay outside the timing
        torch.matmul(a_t, b_t, out=c_t)
    torch.cuda.synchronize()
    ours, theirs = [], []
    for _ in range(6):
        for lst, fn in ((ours, step), (theirs, lambda: torch.matmul(a_t, b_t, out=c_t))):
            ctx.e0.record(stream)
            for _ in range(16):
                fn()
            ctx.e1.record(stream)
            torch.cuda.synchronize()
            lst.append(flops / (ctx.e0.elapsed_time(ctx.e1) / 16 * 1e-3) / 1e12)
    ctx.launches += 96
    out["gemm_bf16_vs_cublas_interleaved_blocks_of_16"] = {"this_kernel_tflops": sum(ours) / len(ours),
                                                           "cublas_tflops": sum(theirs) / len(theirs)}
    try:
        a8 = torch.randn(M, K, device=dev).to(torch.float8_e4m3fn)
        b8 = torch.randn(N, K, device=dev).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=dev)

        def lib8():
            return torch._scaled_mm(a8, b8, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        for _ in range(3):
            lib8()
        torch.cuda.synchronize()
        ctx.e0.record(stream)
        for _ in range(16):
            lib8()
        ctx.e1.record(stream)
        torch.cuda.synchronize()
        out["library_fp8_per_tensor_gemm_8192_yardstick_tflops"] = 2.0 * M * N * K / (ctx.e0.elapsed_time(ctx.e1) / 16 * 1e-3) / 1e12
    except Exception as exc:  # the private API may differ between torch builds
        out["library_fp8_per_tensor_gemm_8192_yardstick_tflops"] = f"unavailable: {str(exc)[:80]}"
    return out


def run_gpu_arm(args):
    import ctypes
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
    ctx = Ctx(lib, stream, dev, world, rank)
    barrier = ctx.barrier
    peak, hbm_peak, peak_src = measured_peaks()

    # ---- operands: A replicated, B and C column-sharded; generated once, outside timing ----
    n0, n1 = sharding.split_range(N, world, rank, 256)
    a_host, b_host = workloads.gemm_bf16_inputs(M, N, K)
    b_host = b_host[:, n0:n1].contiguous()
    n_local = n1 - n0
    x = api.copy_host_to_device(a_host)
    y = api.copy_host_to_device(b_host)
    z = api.zeros([M, n_local], "bf16")
    # CTA pairs (num_cta_in_cga = 2, the reference's published cluster setting) on the 256 x 512 tile: two N = 256
    # MMAs per k-step share the A operand, three quarters of the 256 x 256 tile's bytes per FLOP.  Shards whose
    # 512-wide tiles do not fill whole waves of the 74 pairs (8192 x 4096 / 2048 / 1024 at 2 / 4 / 8 GPUs) take the
    # 256 x 256 tile, whose partial last wave the pair kernel splits along K over all pairs (stream-K).
    wide_tiles = (n_local // 512) * (M // 256)
    bm, bn = 256, (512 if wide_tiles / (-(-wide_tiles // 74) * 74) >= 0.95 else 256)
    generics = ["bf16", str(bm), str(bn), "64"]
    opts = launch.CompileOptions(num_cta_in_cga=2, occupancy=1)

    # the launcher object is built once (partition, generics, options), as a serving loop would; a step is its launch
    gemm_op = launch.gemm(z.partition([bm, bn]), x, y).generics(generics).compile_options(opts)

    def step():
        gemm_op.async_on(stream)

    warmup = max(args.warmup, 3)
    step()                      # first launch: attribute set-up, scratch, lazy module load
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    barrier()
    # the warm-up steps come directly before the timed ones (no idle gap in between, in which the GPU would drop
    # its clocks and the first timed launches would pay for ramping them up again)
    for _ in range(warmup):
        step()
    barrier()
    t_begin = time.monotonic()
    ctx.e0.record(stream)
    for _ in range(args.steps):
        step()
    ctx.e1.record(stream)
    barrier()
    t_end = time.monotonic()
    total_ms = sharding.max_over_ranks(ctx.e0.elapsed_time(ctx.e1), dev)
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    ms_per_step = total_ms / args.steps
    flops = workloads.gemm_flops(M, N, K)
    value = flops / (ms_per_step * 1e-3) / 1e12
    ctx.launches += 1 + warmup + args.steps
    _lib.check(lib.b200tile_status(stream.cuda_stream, ctypes.byref(_lib.StatusC())))

    # ---- the same launch repeated for about two seconds: the rate under the power cap (the timed region above
    # is a burst of a few milliseconds) ----
    n_sus = 20 if args.no_sustained else int(min(max(2000.0 / ms_per_step, 100), 20000))
    sampler2 = ClockSampler(local_rank)
    if rank == 0:
        sampler2.start()
    t_s0 = time.monotonic()
    sus_ms = ctx.timed(step, n_sus, warm=0)
    t_s1 = time.monotonic()
    sus_clocks = sampler2.stop(t_s0, t_s1) if rank == 0 else None
    ctx.launches += n_sus
    sus_tf = flops / (sus_ms * 1e-3) / 1e12 / world

    # ---- end to end through the public API with host buffers ----
    e2e_steps = max(min(args.steps, 5), 1)
    if world == 1:
        a_pin, b_pin = api.pin(a_host), api.pin(b_host)
        c_pin = torch.empty((M, n_local), dtype=torch.bfloat16).pin_memory()
        # one call of the public API per step: B up, A up in 1024-row slabs, each slab multiplied on arrival and
        # its C rows sent back while the next slab is in flight (uploads, MMA and downloads on three streams)
        host_gemm = api.HostGemm(M, n_local, K, "bf16")

        def e2e_step():
            host_gemm(a_pin, b_pin, c_pin, stream)
        e2e_api = "api.HostGemm (b200tile_gemm_host): pinned host A, B, C; upload / multiply / download pipelined in 1024-row slabs"
        e2e_launches = -(-M // 1024)
    else:
        # A crosses PCIe once per box: every rank uploads M/G rows and an NCCL all-gather over NVLink completes A
        # in every rank's HBM; B and C stay column-sharded (no data-path collective in the GEMM itself)
        rows0, rows1 = rank * (M // world), (rank + 1) * (M // world)
        a_pin = api.pin(a_host[rows0:rows1].contiguous())
        b_pin = api.pin(b_host)
        c_pin = torch.empty((M, n_local), dtype=torch.bfloat16).pin_memory()
        host_gemm = sharding.ShardedHostGemm(M, n_local, K, "bf16")

        def e2e_step():
            host_gemm(a_pin, b_pin, c_pin, stream)
        e2e_api = ("sharding.ShardedHostGemm: each rank uploads M/G rows of A and its B columns from pinned host memory, "
                   "NCCL all-gather of A over NVLink, b200tile_gemm, download of its C columns; pipelined over "
                   f"{host_gemm.chunks} row chunks")
        e2e_launches = host_gemm.chunks
    e2e_ms = ctx.timed(e2e_step, e2e_steps, warm=1)
    ctx.launches += (e2e_steps + 1) * e2e_launches
    e2e_value = flops / (e2e_ms * 1e-3) / 1e12
    h2d = M * K * 2 + K * N * 2
    d2h = M * N * 2
    del host_gemm

    by = {"gemm_bf16_8192": _roof("tensor", value / world, peak, "TFLOP/s", ms_per_step, f"{peak_src} cuBLAS bf16 burst",
                                  frac_of_nominal_2250=value / world / NOMINAL_BF16)}
    cpu_by, e2e_by, extra = {}, {}, {}
    e2e_by["gemm_bf16_8192"] = {"value": e2e_value, "unit": "TFLOP/s", "ms": e2e_ms, "h2d_bytes_per_step": h2d,
                                "d2h_bytes_per_step": d2h}
    do_cpu = world == 1 and rank == 0 and not args.no_cpu_baseline
    if not args.no_fmha:
        extra.update(bench_fmha(ctx, by, cpu_by, e2e_by, do_cpu))
        extra.update(bench_fp8(ctx, by, cpu_by, e2e_by, do_cpu))
        extra.update(bench_nvfp4(ctx, by, cpu_by, e2e_by, do_cpu) or {})
        bench_f32(ctx, by, cpu_by, e2e_by, do_cpu)
        extra.update(bench_neighbours(ctx))
        if world == 1:
            extra.update(bench_single_gpu_yardsticks(ctx, step, flops, x, y, n_local))
        else:
            # the replicated-result option: NCCL all-gather of the C column shards (+ the local re-layout) and of
            # the attention output slabs, timed by themselves
            c_loc = z.storage
            ag_ms = ctx.timed(lambda: sharding.all_gather_columns(c_loc), 5)
            o_loc = torch.empty((256 // world, 4096, 128), dtype=torch.bfloat16, device=dev)
            ao_ms = ctx.timed(lambda: sharding.all_gather_problems(o_loc), 5)
            extra["all_gather_replicated_result"] = {
                "gemm_c_columns_ms": ag_ms, "gemm_c_bytes_per_rank": c_loc.numel() * 2,
                "gemm_step_plus_gather_ms": ms_per_step + ag_ms,
                "fmha_o_problems_ms": ao_ms, "fmha_o_bytes_per_rank": o_loc.numel() * 2}
    _lib.check(lib.b200tile_status(stream.cuda_stream, ctypes.byref(_lib.StatusC())))

    if rank == 0:
        cpu = None
        if do_cpu:
            r = cpu_gemm_rate(12.0, 0)
            cpu = {"value": r["tflops"], "unit": "TFLOP/s", "cores": r["threads"], "kind": "port",
                   "sample": f"rows [0,{r['rows']}) of the same 8192^3 GEMM ({r['seconds']:.1f} s), "
                             "oracle port of the reference's cpu_gemm",
                   "by_config": cpu_by}
        per_gpu = value / world
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "gemm_bf16_8192x8192x8192", "layout": "A[M,K] B[K,N] row-major, fp32 acc",
                       "tile": f"{bm}x{bn} per CTA pair (cta_group::2), " + ("4 stages of 64-deep" if bn == 512 else "3 stages of 128-deep") +
                               " k slabs (TMA ring), persistent, grouped-M 8",
                       "parallelism": f"N-split x{world}" if world > 1 else "single GPU",
                       "l2": "operands 403 MB per step exceed the 126 MB L2; no flush between steps"},
            "per_gpu_tflops": per_gpu,
            "pct_of_nominal_peak_2250": 100.0 * per_gpu / NOMINAL_BF16,
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s",
                         "frac": per_gpu / peak, "traffic": GEMM_DRAM_TRAFFIC_BYTES,
                         "peak_source": f"{peak_src} cuBLAS bf16 burst",
                         "sustained": {"achieved": sus_tf, "launches": n_sus, "seconds": sus_ms * n_sus * 1e-3,
                                       "peak_sustained": SUSTAINED_BF16_TFLOPS,
                                       "frac_of_sustained": (sus_tf / SUSTAINED_BF16_TFLOPS) if SUSTAINED_BF16_TFLOPS else None,
                                       "sm_mhz": (sus_clocks or {}).get("sm_mhz"), "reasons": (sus_clocks or {}).get("reasons")},
                         "by_config": by},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "api": e2e_api,
                    "gpu_launches_per_step": e2e_launches * world, "by_config": e2e_by},
            "gpu_launches": ctx.launches * world,
            "clocks": clocks,
            "extra": extra,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


# ------------------------------------------------------------------------------------------
# Single-kernel cases (profiler captures)
# ------------------------------------------------------------------------------------------
def run_case(argv) -> int:
    """One kernel a few times on a small case, for profiler captures and quick timing (`bench.py --case <kernel> ...`).
    The default sizes keep the operands above the 126 MB L2 (so DRAM counters mean something) and the device
    footprint far below a few GB (so a multi-pass capture ends by itself).  With the diagnostic build
    (B200_VARIANT=trace B200_NVCC_EXTRA=-DB200TILE_TRACE cutile_rs_b200/csrc/build.sh) and
    B200TILE_LIB=cutile_rs_b200/libb200tile_trace.so, `--trace` prints where the MMA-issuing thread (and one softmax
    lane) of one CTA spent its cycles."""
    import ctypes
    import torch
    from cutile_rs_b200 import _lib
    ap = argparse.ArgumentParser(prog="bench.py --case")
    ap.add_argument("kernel", choices=["gemm", "fmha", "decode", "nvfp4", "fp8", "group", "norm", "qkrope"])
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--config", type=int, default=-1)
    ap.add_argument("--layout", type=int, default=0)
    ap.add_argument("--group-m", type=int, default=0, help="gemm: tile rows per band of the tile order (0 = the library's default, 8)")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--causal", type=int, default=0)
    ap.add_argument("--group", type=int, default=4)
    ap.add_argument("--splits", type=int, default=18)
    ap.add_argument("--bn", type=int, default=128)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--pair", type=int, default=0, help="fmha: 1 = the CTA-pair configuration")
    ap.add_argument("--ones", action="store_true", help="gemm: all-ones operands instead of random ones")
    ap.add_argument("--trace", action="store_true", help="print the cycle counters of a trace build")
    args = ap.parse_args(argv)
    if args.pair:
        os.environ["B200TILE_FMHA_PAIR"] = str(args.pair)

    torch.cuda.set_device(0)
    lib = _lib.load()
    _lib.check(lib.b200tile_init(0))
    stream = torch.cuda.current_stream()
    g = torch.Generator(device="cuda").manual_seed(1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.kernel == "gemm":
        m, n, k = args.m, args.n, args.k
        tdt, name = (torch.float16, b"f16") if args.config == 4 else (torch.bfloat16, b"bf16")   # config 4: f16 accumulators
        a = (torch.randn(m, k, device="cuda", generator=g) / math.sqrt(k)).to(tdt)
        b = (torch.randn((n, k) if args.layout else (k, n), device="cuda", generator=g) / math.sqrt(k)).to(tdt)
        if args.ones:   # the published benchmark's inputs: far fewer bit flips, so less power and higher clocks
            a.fill_(1.0)
            b.fill_(1.0)
        c = torch.empty(m, n, dtype=tdt, device="cuda")

        def run():
            _lib.check(lib.b200tile_gemm(name, args.layout, a.data_ptr(), b.data_ptr(), c.data_ptr(), 1, m, n,
                                         k, k, b.stride(0), n, 0, 0, 0, 0, args.config, args.group_m, 0, stream.cuda_stream))
        flops = 2.0 * m * n * k
    elif args.kernel == "nvfp4":
        m, n, k = args.m, args.n, args.k
        xp = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, device="cuda", generator=g)
        yp = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda", generator=g)
        xs = torch.full((m, k // 16), 0x38, dtype=torch.uint8, device="cuda")    # e4m3 1.0
        ys = torch.full((n, k // 16), 0x38, dtype=torch.uint8, device="cuda")
        z = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        wsb = lib.b200tile_linear_nvfp4_workspace_bytes(m, n, k)
        ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")

        def run():
            _lib.check(lib.b200tile_linear_nvfp4(xp.data_ptr(), yp.data_ptr(), xs.data_ptr(), ys.data_ptr(),
                                                 z.data_ptr(), b"bf16", m, n, k, k // 2, k // 2, n, k // 16, k // 16,
                                                 1.0, ws.data_ptr(), wsb, args.config, stream.cuda_stream))
        flops = 2.0 * m * n * k
    elif args.kernel == "fp8":
        from cutile_rs_b200 import quant
        m, n, k = args.m, args.n, args.k
        xq, xs = quant.quant_fp8_block(torch.randn(m, k, device="cuda", generator=g), 1, 128)
        yq, ys = quant.quant_fp8_block(torch.randn(n, k, device="cuda", generator=g), 128, 128)
        z = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")

        def run():
            _lib.check(lib.b200tile_linear_fp8_blk128(xq.data_ptr(), yq.data_ptr(), xs.data_ptr(), ys.data_ptr(), z.data_ptr(),
                                                      b"bf16", m, n, k, k, k, n, k // 128, k // 128, 1.0, stream.cuda_stream))
        flops = 2.0 * m * n * k
    elif args.kernel == "group":
        from cutile_rs_b200 import launch
        e, m, n, k = args.batch, args.m, args.n, args.k      # --batch experts of m x n x k
        ga = (torch.randn(e, m, k, device="cuda", generator=g) / 8).bfloat16()
        gb = (torch.randn(e, k, n, device="cuda", generator=g) / 8).bfloat16()
        gc = torch.empty(e, m, n, device="cuda", dtype=torch.bfloat16)
        tabs = launch.group_gemm_tables(list(ga), list(gb), list(gc))

        def run():
            _lib.check(lib.b200tile_group_gemm(b"bf16", *(t_.cu_deviceptr() for t_ in tabs), e, 256, None, 0,
                                               stream.cuda_stream))
        flops = 2.0 * e * m * n * k
    elif args.kernel == "norm":
        rows, n = args.m, args.n
        r = torch.randn(rows, n, device="cuda", generator=g).half()
        x = torch.randn(rows, n, device="cuda", generator=g).half()
        w = torch.ones(n, device="cuda", dtype=torch.float16)
        o, ro = torch.empty_like(x), torch.empty_like(x)

        def run():
            _lib.check(lib.b200tile_add_rms_norm(b"f16", r.data_ptr(), x.data_ptr(), w.data_ptr(), o.data_ptr(),
                                                 ro.data_ptr(), rows, n, n, n, n, n, 1e-5, stream.cuda_stream))
        flops = 4.0 * rows * n * 2     # bytes, reported below as GB/s
    elif args.kernel == "qkrope":
        t, qh, kvh, d = args.m, args.heads, max(args.heads // 4, 1), args.head_dim
        q = torch.randn(t, qh, d, device="cuda", generator=g).half()
        k = torch.randn(t, kvh, d, device="cuda", generator=g).half()
        v = torch.randn(t, kvh, d, device="cuda", generator=g).half()
        w = torch.ones(d, device="cuda", dtype=torch.float16)
        f = (1.0 / 10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32, device="cuda") / d)).contiguous()
        qo = torch.empty_like(q)
        kc = torch.empty(kvh, t, d, device="cuda", dtype=torch.float16)
        vc = torch.empty_like(kc)

        def run():
            _lib.check(lib.b200tile_qk_norm_rope_kv(b"f16", q.data_ptr(), k.data_ptr(), v.data_ptr(), w.data_ptr(),
                                                    w.data_ptr(), f.data_ptr(), qo.data_ptr(), kc.data_ptr(),
                                                    vc.data_ptr(), 1e-6, 0, None, t, qh, kvh, d, t, qh * d, kvh * d,
                                                    kvh * d, qh * d, stream.cuda_stream))
        flops = 2.0 * t * (qh + 2 * kvh) * d * 2     # bytes
    elif args.kernel == "decode":
        h, grp, s, d, ns = args.heads, args.group, args.seq, args.head_dim, args.splits
        q = torch.randn(h, grp, d, device="cuda", generator=g).bfloat16()
        kk = torch.randn(h, s, d, device="cuda", generator=g).bfloat16()
        v = torch.randn(h, s, d, device="cuda", generator=g).bfloat16()
        att = torch.empty(h, ns * grp, d, dtype=torch.bfloat16, device="cuda")
        lse = torch.empty(h, ns * grp, dtype=torch.float32, device="cuda")
        o = torch.empty_like(q)
        pos = torch.tensor([s - 1], dtype=torch.int32, device="cuda")
        i2 = ctypes.c_int64 * 2

        def run():
            _lib.check(lib.b200tile_fmha_decode_gqa_split(
                b"bf16", q.data_ptr(), kk.data_ptr(), v.data_ptr(), att.data_ptr(), lse.data_ptr(), o.data_ptr(),
                pos.data_ptr(), h, grp, d, s, args.bn, ns, 1.0 / math.sqrt(d), i2(grp * d, d), i2(s * d, d),
                i2(s * d, d), i2(ns * grp * d, d), ns * grp, i2(grp * d, d), stream.cuda_stream))
        flops = 4.0 * s * d * h * grp
        print(f"decode: K+V bytes per launch {2 * h * s * d * 2}")
    else:
        bsz, h, s, d = args.batch, args.heads, args.seq, args.head_dim
        q = torch.randn(bsz * h, s, d, device="cuda", generator=g).bfloat16()
        kk = torch.randn(bsz * h, s, d, device="cuda", generator=g).bfloat16()
        v = torch.randn(bsz * h, s, d, device="cuda", generator=g).bfloat16()
        o = torch.empty_like(q)
        st = (ctypes.c_int64 * 2)(s * d, d)

        def run():
            _lib.check(lib.b200tile_fmha_fwd(b"bf16", q.data_ptr(), kk.data_ptr(), v.data_ptr(), o.data_ptr(),
                                             bsz, h, h, s, s, d, st, st, st, st, 1.0 / math.sqrt(d),
                                             args.causal, 0, stream.cuda_stream))
        flops = 4.0 * s * s * d * h * bsz / (2 if args.causal else 1)
    run()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.iters
    status = _lib.StatusC()
    _lib.check(lib.b200tile_status(stream.cuda_stream, ctypes.byref(status)))
    if args.kernel in ("norm", "qkrope"):
        print(f"{args.kernel}: {ms * 1e3:.1f} us/launch, {flops / ms / 1e6:.0f} GB/s of algorithmic bytes")
    else:
        print(f"{args.kernel}: {ms:.4f} ms/launch, {flops / ms / 1e9:.1f} TFLOP/s")
    if args.trace:
        _print_trace(lib, args)
    return 0


def _print_trace(lib, args) -> None:
    import ctypes
    if not hasattr(lib, "b200tile_trace_read"):
        raise SystemExit("--trace needs the diagnostic build (see the module docstring)")
    out = (ctypes.c_longlong * 20)()
    which = {"gemm": b"gemm_pair", "fmha": b"fmha_alt" if args.pair else b"fmha",
             "nvfp4": b"block_scaled_pair" if args.config == 3 else b"block_scaled", "group": b"grouped"}.get(args.kernel)
    if which is None or lib.b200tile_trace_read(which, out):
        raise SystemExit("no trace for this kernel")
    v = list(out)
    if args.kernel == "group":
        n = max(v[4], 1)
        print(f"MMA warp of one CTA per 64-deep stage (4 MMAs = 540 tensor cycles): stage-full waits {v[1] / n:.0f}, fence + issue "
              f"+ commit {v[2] / n:.0f}, accumulator waits {v[0] / n:.0f}; total {v[5] / n:.0f} cycles per stage ({n} stages); "
              f"SM clock inside the kernel {1e3 * v[5] / max(v[6], 1):.0f} MHz")
        return
    if args.kernel == "gemm" and v[13] > v[8] > 0:
        t0 = v[8]
        print("time line of that CTA, us after its entry: set-up done %.2f, first operands landed %.2f, last commit "
              "issued %.2f, first epilogue warp done %.2f, about to leave %.2f"
              % tuple((v[i] - t0) / 1e3 for i in (9, 10, 11, 12, 13)))
    if args.kernel == "nvfp4":
        n = max(v[5], 1)
        print(f"MMA thread of one CTA per stage (4 block-scaled MMAs): stage + scale waits {v[2] / n:.0f}, "
              f"MMA issue {v[3] / n:.0f}, commit {v[4] / n:.0f}, accumulator waits {v[0] / n:.0f}; "
              f"total {v[6] / n:.0f} cycles per stage ({n} stages); "
              f"SM clock inside the kernel {1e3 * v[6] / max(v[7], 1):.0f} MHz")
        w = max(v[14], 1)
        if args.config == 3:
            print(f"scale-writer warp per stage: stage-full wait {v[10] / w:.0f}, loads + store issue {v[11] / w:.0f}, "
                  f"store completion {v[12] / w:.0f}, region wait {v[13] / w:.0f}; total {v[15] / w:.0f}")
        else:
            print(f"scale-writer warp per stage: stage-full wait {v[10] / w:.0f}, region wait + loads + store issue "
                  f"{v[11] / w:.0f}, store completion {v[12] / w:.0f}, hand-off {v[13] / w:.0f}; total {v[15] / w:.0f}")
        if args.config == 3:
            tl = (ctypes.c_longlong * 40)()
            if lib.b200tile_trace_read(b"block_scaled_pair_timeline", tl) == 0:
                print("time lines of 8 consecutive stages (cycles after the producer saw the first slot free): "
                      "slot free / copies issued / landed / scales ready seen by the MMA warp / committed")
                for g in range(8):
                    print("   " + " ".join(f"{tl[5 * g + e] - tl[0]:6d}" for e in range(5)))
        pn = max(v[19], 1)
        print(f"TMA producer per stage: stage-empty wait {v[17] / pn:.0f}, issue of the copies {v[18] / pn:.0f}")
        return
    if args.kernel == "gemm":
        stages, tiles = max(v[4], 1), max(v[5], 1)
        print(f"MMA thread of one CTA pair, per 128-deep stage (8 MMAs 256x256x16 = 1024 tensor cycles): "
              f"wait full {v[1] / stages:.0f}, issue {v[2] / stages:.0f}, commits {v[3] / stages:.0f}; "
              f"accumulator waits {v[0] / tiles:.0f} per tile; total {v[6] / stages:.0f} cycles per stage "
              f"({stages} stages, {tiles} tiles); SM clock inside the kernel {1e3 * v[6] / max(v[7], 1):.0f} MHz")
    else:
        n, m = max(v[6], 1), max(v[16], 1)
        names = ["K/V waits", "P waits", "P.V issue", "Q.K issue", "S commits", "release commits"]
        if args.pair:
            names = ["V waits", "P waits", "P.V issue", "K waits (Q.K thread)", "free-S waits (Q.K thread)", "release commits"]
        print("MMA thread per key tile (both query tiles): " +
              ", ".join(f"{nm} {v[i] / n:.0f}" for i, nm in enumerate(names)) + f"; total {v[7] / n:.0f} ({n} key tiles); SM clock inside the kernel {1e3 * v[7] / max(v[8], 1):.0f} MHz")
        if args.pair:
            t = (ctypes.c_longlong * 20)()
            if lib.b200tile_trace_read(b"fmha_alt_t", t) == 0:
                t = list(t)
                t0 = min(x for x in t if x > 0)
                for wg in range(2):
                    print(f"warpgroup {wg} tiles 10..14 (scores loaded, P handed over), cycles: " +
                          " ".join(f"({t[wg * 10 + 2 * i] - t0}, {t[wg * 10 + 2 * i + 1] - t0})" for i in range(5)))
        names = ["S wait", "TMEM load", "max+rescale", "exp2 loop", "store wait", "hand-off"]
        print("softmax lane per key tile: " + ", ".join(f"{nm} {v[10 + i] / m:.0f}" for i, nm in enumerate(names)) +
              f"; total {v[17] / m:.0f}")



def main():
    if len(sys.argv) > 1 and sys.argv[1] == "--case":
        return run_case(sys.argv[2:])
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-fmha", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sustained", action="store_true",
                    help="shorten the two-second repetition of the headline launch to 20 launches (launch-list captures)")
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
