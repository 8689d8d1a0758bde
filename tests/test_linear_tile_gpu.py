"""The reference's block-scaled `linear_tile` kernels under their own name: `b200tile_launch("linear_tile", ...)`
with the parameter list and generics of cutile-examples/examples/nvfp4.rs:37-76 and mxfp8.rs:34-64, driven
through the launcher mirror exactly as the examples drive the generated launcher."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from cutile_rs_b200 import _lib, api, launch, quant, workloads  # noqa: E402
from cutile_rs_b200.tensor import KernelLaunchError  # noqa: E402

FP4_TOL = 3e-2   # relative Frobenius error of the block-scaled GEMMs against the fp32 dequantised reference


def _stream():
    return torch.cuda.current_stream()


def _status_ok(lib):
    st = _lib.StatusC()
    _lib.check(lib.b200tile_status(_stream().cuda_stream, st))
    assert st.code == 0


def test_nvfp4_example_known_answer(b200):
    # nvfp4.rs:97-151: BM = BN = 16, BK = 64, M = N = 16, K = 128, nibbles 0x2 (1.0), scales 0x38 (1.0) -> 128.0
    bm = bn = 16
    bk, m, n, k = 64, 16, 16, 128
    x = api.from_torch(torch.full((m, k // 2), 0x22, dtype=torch.uint8, device="cuda"), "f4e2m1fnx2")
    y = api.from_torch(torch.full((n, k // 2), 0x22, dtype=torch.uint8, device="cuda"), "f4e2m1fnx2")
    xs = api.from_torch(torch.full((m, k // 16), 0x38, dtype=torch.uint8, device="cuda"), "f8e4m3fn")
    ys = api.from_torch(torch.full((n, k // 16), 0x38, dtype=torch.uint8, device="cuda"), "f8e4m3fn")
    z = api.zeros([m, n], "f32").partition([bm, bn])
    generics = [str(bm), str(bn), str(bk), str(bk // 2), str(bk // 16)]
    (z, x2, _y, _xs, _ys, _alpha) = launch.linear_tile(z, x, y, xs, ys, 1.0).generics(generics).sync_on(_stream())
    assert x2 is x
    got = z.unpartition().to_host()
    assert torch.all((got - float(k)).abs() <= 1e-3)
    # the same call with inferred generics
    z2 = api.zeros([m, n], "f32").partition([bm, bn])
    launch.linear_tile(z2, x, y, xs, ys, 0.5).sync_on(_stream())
    assert torch.all((z2.unpartition().to_host() - 0.5 * k).abs() <= 1e-3)
    _status_ok(b200)


def test_mxfp8_example_known_answer(b200):
    # mxfp8.rs:83-135: BM = BN = 16, BK = 64, M = N = 16, K = 128, fp8 0x38 (1.0), E8M0 0x7F (1.0) -> 128.0
    bm = bn = 16
    bk, m, n, k = 64, 16, 16, 128
    x = api.from_torch(torch.full((m, k), 0x38, dtype=torch.uint8, device="cuda"), "f8e4m3fn")
    y = api.from_torch(torch.full((n, k), 0x38, dtype=torch.uint8, device="cuda"), "f8e4m3fn")
    xs = api.from_torch(torch.full((m, k // 32), 0x7F, dtype=torch.uint8, device="cuda"), "f8e8m0fnu")
    ys = api.from_torch(torch.full((n, k // 32), 0x7F, dtype=torch.uint8, device="cuda"), "f8e8m0fnu")
    z = api.zeros([m, n], "f32").partition([bm, bn])
    generics = [str(bm), str(bn), str(bk), str(bk // 32)]
    (z, *_rest) = launch.linear_tile(z, x, y, xs, ys, 1.0).generics(generics).sync_on(_stream())
    assert torch.all((z.unpartition().to_host() - float(k)).abs() <= 1e-3)
    _status_ok(b200)


@pytest.mark.parametrize("fmt,m,n,k", [("nvfp4", 200, 328, 320), ("mxfp8", 200, 328, 384)])
def test_random_operands_match_oracle(b200, oracle, fmt, m, n, k):
    a, b = workloads.gemm_normal_inputs(m, n, k, config_index=6)
    if fmt == "nvfp4":
        xp, xs, ga = quant.quant_nvfp4(a)
        yp, ys, gb = quant.quant_nvfp4(b)
        alpha, dt, st = ga * gb, "f4e2m1fnx2", "f8e4m3fn"
        ref = oracle.cpu_gemm_nt(oracle.dequant_nvfp4(xp.numpy(), xs.numpy()), oracle.dequant_nvfp4(yp.numpy(), ys.numpy()),
                                 alpha=alpha, threads=0)
    else:
        xp, xs = quant.quant_mxfp8(a)
        yp, ys = quant.quant_mxfp8(b)
        alpha, dt, st = 0.25, "f8e4m3fn", "f8e8m0fnu"
        ref = oracle.cpu_gemm_nt(oracle.dequant_mxfp8(xp.numpy(), xs.numpy()), oracle.dequant_mxfp8(yp.numpy(), ys.numpy()),
                                 alpha=alpha, threads=0)
    x, y = api.from_torch(xp.cuda(), dt), api.from_torch(yp.cuda(), dt)
    sx, sy = api.from_torch(xs.cuda(), st), api.from_torch(ys.cuda(), st)
    z = api.from_torch(torch.full((m, n), float("nan"), device="cuda")).partition([64, 64])
    launch.linear_tile(z, x, y, sx, sy, alpha).sync_on(_stream())
    got = z.unpartition().to_host().numpy()
    assert not np.isnan(got).any()
    assert oracle.rel_frobenius(got, ref) <= 1e-5      # f32 output: the products and sums are exact up to fp32 rounding
    # errors the autotuner must see as an invalid trial, not a crash
    with pytest.raises(KernelLaunchError, match="generics"):
        launch.linear_tile(z, x, y, sx, sy, alpha).generics(["64", "64", "64"]).sync_on(_stream())
    with pytest.raises(KernelLaunchError, match="block-scaled format"):
        launch.linear_tile(z, x, y, sx, sy, alpha).generics(["64", "64", "64", "4"]).sync_on(_stream())
    with pytest.raises(KernelLaunchError, match="does not match the inferred partition grid"):
        launch.linear_tile(z, x, y, sx, sy, alpha).grid((1, 1, 1)).sync_on(_stream())
    launch.linear_tile(z, x, y, sx, sy, alpha).compile()
    _status_ok(b200)


def test_full_size_nvfp4_through_the_generic_name(b200, oracle):
    """M = 4096 and the decode shape M = 16 at N = 14336, K = 4096 with a bf16 output; the decode call also with
    registered (prepared) weight scales and from a captured graph."""
    n, k = 14336, 4096
    g = torch.Generator(device="cuda").manual_seed(workloads.SEED_BASE + 4)
    b = torch.randn(n, k, device="cuda", generator=g)
    yp, ys, gb = quant.quant_nvfp4(b)
    y, sy = api.from_torch(yp, "f4e2m1fnx2"), api.from_torch(ys, "f8e4m3fn")
    cols = slice(7100, 7228)
    yref = oracle.dequant_nvfp4(yp[cols].cpu().numpy(), ys[cols].cpu().numpy())
    outs = {}
    for m in (4096, 16):
        a = torch.randn(m, k, device="cuda", generator=g)
        xp, xs, ga = quant.quant_nvfp4(a)
        x, sx = api.from_torch(xp, "f4e2m1fnx2"), api.from_torch(xs, "f8e4m3fn")
        z = api.from_torch(torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)).partition([16, 128])
        launch.linear_tile(z, x, y, sx, sy, ga * gb).sync_on(_stream())
        got = z.unpartition().storage
        rows = slice(0, 8) if m == 16 else slice(2044, 2052)
        ref = oracle.cpu_gemm_nt(oracle.dequant_nvfp4(xp[rows].cpu().numpy(), xs[rows].cpu().numpy()), yref,
                                 alpha=ga * gb, threads=0)
        assert oracle.rel_frobenius(got[rows, cols].float().cpu().numpy(), ref) <= FP4_TOL
        assert not torch.isnan(got.float()).any()
        outs[m] = (got.clone(), x, sx, ga * gb)
    # decode shape again with the weight scales laid out once and registered: one kernel, same bits
    want, x, sx, alpha = outs[16]
    prepared = launch.nvfp4_prepare_weight_scales(sy, n, k, 0)
    launch.nvfp4_register_weight_scales(sy, n, k, prepared, 0)
    try:
        z = api.from_torch(torch.full((16, n), float("nan"), device="cuda", dtype=torch.bfloat16)).partition([16, 128])
        launch.linear_tile(z, x, y, sx, sy, alpha).sync_on(_stream())
        assert torch.equal(z.unpartition().storage, want)
        # ... and from a captured graph (no allocation, no scratch: the prepared form needs none)
        z.unpartition().storage.fill_(float("nan"))
        stream = torch.cuda.Stream()
        torch.cuda.synchronize()
        graph = launch.linear_tile(z, x, y, sx, sy, alpha).graph_on(stream)
        graph.launch().sync()
        torch.cuda.synchronize()
        assert torch.equal(z.unpartition().storage, want)
    finally:
        launch.nvfp4_unregister_weight_scales(sy)
    with pytest.raises(KernelLaunchError, match="not registered"):
        launch.nvfp4_unregister_weight_scales(sy)
    _status_ok(b200)


def test_capture_uses_the_scratch_of_an_earlier_eager_call(b200):
    m, n, k = 256, 448, 512
    a, b = workloads.gemm_normal_inputs(m, n, k, config_index=7)
    xp, xs = quant.quant_mxfp8(a)
    yp, ys = quant.quant_mxfp8(b)
    x, y = api.from_torch(xp.cuda(), "f8e4m3fn"), api.from_torch(yp.cuda(), "f8e4m3fn")
    sx, sy = api.from_torch(xs.cuda(), "f8e8m0fnu"), api.from_torch(ys.cuda(), "f8e8m0fnu")
    z = api.from_torch(torch.full((m, n), float("nan"), device="cuda")).partition([128, 64])
    fresh = torch.cuda.Stream()
    torch.cuda.synchronize()
    # a stream that has never run the kernel has no scratch block, and a capture cannot allocate one
    with pytest.raises(KernelLaunchError, match="stream capture"):
        launch.linear_tile(z, x, y, sx, sy, 1.0).graph_on(fresh)
    torch.cuda.synchronize()
    used = torch.cuda.Stream()
    launch.linear_tile(z, x, y, sx, sy, 1.0).sync_on(used)
    want = z.unpartition().storage.clone()
    z.unpartition().storage.fill_(float("nan"))
    graph = launch.linear_tile(z, x, y, sx, sy, 1.0).graph_on(used)
    for _ in range(2):
        graph.launch().sync()
        torch.cuda.synchronize()
        assert torch.equal(z.unpartition().storage, want)
    _status_ok(b200)
