"""Runs one kernel a few times on a small case, for profiler captures and quick timing.

    python -m cutile_rs_b200.profile_case gemm --m 4096 --n 4096 --k 8192 --iters 3
    python -m cutile_rs_b200.profile_case fmha --batch 1 --heads 16 --seq 4096 --causal 0 --iters 3
    python -m cutile_rs_b200.profile_case decode --heads 8 --group 4 --seq 65536 --splits 18 --iters 3
    python -m cutile_rs_b200.profile_case nvfp4 --m 4096 --n 14336 --k 4096 --iters 3
    python -m cutile_rs_b200.profile_case norm --m 8192 --n 8192 --iters 3      # residual add + RMSNorm, rows x N
    python -m cutile_rs_b200.profile_case qkrope --m 16384 --heads 32 --iters 3 # QK norm + RoPE + KV write, tokens

With the diagnostic build (B200_VARIANT=trace B200_NVCC_EXTRA=-DB200TILE_TRACE csrc/build.sh) and
B200TILE_LIB=cutile_rs_b200/libb200tile_trace.so, ``--trace`` prints where the MMA-issuing thread
(and one softmax lane) of one CTA spent its cycles:

    B200TILE_LIB=cutile_rs_b200/libb200tile_trace.so python -m cutile_rs_b200.profile_case gemm \
        --m 8192 --n 8192 --k 8192 --config 2 --iters 5 --trace

The default sizes keep the operands above the 126 MB L2 (so DRAM counters mean something) and the
device footprint far below a few GB (so a multi-pass capture ends by itself).
"""
from __future__ import annotations

import argparse
import ctypes
import math

import torch

from . import _lib


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "fmha", "decode", "nvfp4", "norm", "qkrope"])
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--config", type=int, default=-1)
    ap.add_argument("--layout", type=int, default=0)
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
    args = ap.parse_args()
    if args.pair:
        import os
        os.environ["B200TILE_FMHA_PAIR"] = str(args.pair)

    torch.cuda.set_device(0)
    lib = _lib.load()
    _lib.check(lib.b200tile_init(0))
    stream = torch.cuda.current_stream()
    g = torch.Generator(device="cuda").manual_seed(1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.kernel == "gemm":
        m, n, k = args.m, args.n, args.k
        a = (torch.randn(m, k, device="cuda", generator=g) / math.sqrt(k)).bfloat16()
        b = (torch.randn((n, k) if args.layout else (k, n), device="cuda", generator=g) / math.sqrt(k)).bfloat16()
        if args.ones:   # the published benchmark's inputs: far fewer bit flips, so less power and higher clocks
            a.fill_(1.0)
            b.fill_(1.0)
        c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")

        def run():
            _lib.check(lib.b200tile_gemm(b"bf16", args.layout, a.data_ptr(), b.data_ptr(), c.data_ptr(), 1, m, n,
                                         k, k, b.stride(0), n, 0, 0, 0, 0, args.config, 0, 0, stream.cuda_stream))
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


def _print_trace(lib, args) -> None:
    if not hasattr(lib, "b200tile_trace_read"):
        raise SystemExit("--trace needs the diagnostic build (see the module docstring)")
    out = (ctypes.c_longlong * 20)()
    which = {"gemm": b"gemm_pair", "fmha": b"fmha_alt" if args.pair else b"fmha",
             "nvfp4": b"block_scaled"}.get(args.kernel)
    if which is None or lib.b200tile_trace_read(which, out):
        raise SystemExit("no trace for this kernel")
    v = list(out)
    if args.kernel == "nvfp4":
        n = max(v[5], 1)
        print(f"MMA thread of one CTA per stage (4 block-scaled MMAs): stage + scale waits {v[2] / n:.0f}, "
              f"MMA issue {v[3] / n:.0f}, commit {v[4] / n:.0f}; total {v[6] / n:.0f} cycles per stage ({n} stages); "
              f"SM clock inside the kernel {1e3 * v[6] / max(v[7], 1):.0f} MHz")
        w = max(v[14], 1)
        print(f"scale-writer warp per stage: stage-full wait {v[10] / w:.0f}, region wait + loads + store issue "
              f"{v[11] / w:.0f}, store completion {v[12] / w:.0f}, hand-off {v[13] / w:.0f}; total {v[15] / w:.0f}")
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


if __name__ == "__main__":
    main()
