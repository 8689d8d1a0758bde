"""Block-scaled fp8 GEMM parity on a B200 against the oracle's fp32 dequantised reference."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from cutile_rs_b200 import _lib, api, launch, quant, workloads  # noqa: E402

FP8_TOL = 3e-2   # relative Frobenius error against the fp32 dequantised reference


def _run(lib, aq, bq, sa, sb, m, n, k, out="bf16", alpha=1.0):
    z = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16 if out == "bf16" else torch.float32)
    _lib.check(lib.b200tile_linear_fp8_blk128(aq.data_ptr(), bq.data_ptr(), sa.data_ptr(), sb.data_ptr(),
                                              z.data_ptr(), out.encode(), m, n, k, k, k, n, k // 128, k // 128,
                                              alpha, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return z


@pytest.mark.parametrize("m,n,k,out", [(128, 256, 128, "bf16"), (256, 512, 1024, "f32"), (200, 384, 256, "bf16"),
                                       (1000, 1280, 512, "f32")])
def test_matches_oracle(b200, oracle, m, n, k, out):
    a, b = workloads.gemm_normal_inputs(m, n, k, config_index=3)
    # quantisers: the torch ones must agree with the oracle's bit for bit
    aq, sa = quant.quant_fp8_block(a, 1, 128)
    bq, sb = quant.quant_fp8_block(b, 128, 128)
    aq_o, sa_o = oracle.quant_fp8_block(a.numpy(), 1, 128)
    bq_o, sb_o = oracle.quant_fp8_block(b.numpy(), 128, 128)
    assert np.array_equal(aq.numpy(), aq_o) and np.array_equal(sa.numpy(), sa_o)
    assert np.array_equal(bq.numpy(), bq_o) and np.array_equal(sb.numpy(), sb_o)
    got = _run(b200, aq.cuda(), bq.cuda(), sa.cuda(), sb.cuda(), m, n, k, out, alpha=0.5).float().cpu().numpy()
    ref = oracle.cpu_gemm_nt(oracle.dequant_fp8_block(aq_o, sa_o, 1, 128), oracle.dequant_fp8_block(bq_o, sb_o, 128, 128),
                             alpha=0.5, threads=0)
    assert not np.isnan(got).any()
    assert oracle.rel_frobenius(got, ref) <= (FP8_TOL if out == "bf16" else 1e-5)
    # against the UNquantised product the error is the quantisation error, within the same contract
    full = oracle.cpu_gemm_nt(a.numpy(), b.numpy(), alpha=0.5, threads=0)
    assert oracle.rel_frobenius(got, full) <= 5e-2


def test_known_answer_and_errors(b200):
    # fp8 0x38 = 1.0 with unit scales: every output equals K (the reference's scaled-MMA check,
    # cutile-examples/examples/mxfp8.rs:91-92,129-135, with this kernel's scale granularity)
    m, n, k = 128, 256, 256
    ones = torch.full((max(m, n), k), 0x38, dtype=torch.uint8, device="cuda")
    sa = torch.ones(m, k // 128, device="cuda")
    sb = torch.ones(n // 128, k // 128, device="cuda")
    z = _run(b200, ones[:m], ones[:n], sa, sb, m, n, k, "f32")
    assert torch.all(z == float(k))
    rc = b200.b200tile_linear_fp8_blk128(ones.data_ptr(), ones.data_ptr(), sa.data_ptr(), sb.data_ptr(), z.data_ptr(),
                                         b"f32", m, n, 200, 200, 200, n, 2, 2, 1.0, None)
    assert rc == _lib.ERR_INVALID and b"multiple of the 128-element scale block" in b200.b200tile_last_error()


def test_full_size_slab_and_launcher(b200, oracle):
    # the benchmark's fp8 workload at full size: M=8192, N=28672, K=8192 (device-side generation, oracle slab)
    m, n, k = 8192, 28672, 8192
    g = torch.Generator(device="cuda").manual_seed(workloads.SEED_BASE + 3)
    a = torch.randn(m, k, device="cuda", generator=g)
    b = torch.randn(n, k, device="cuda", generator=g)
    aq, sa = quant.quant_fp8_block(a, 1, 128)
    bq, sb = quant.quant_fp8_block(b, 128, 128)
    del a, b
    x, y = api.from_torch(aq.view(torch.float8_e4m3fn)), api.from_torch(bq.view(torch.float8_e4m3fn))
    z = api.zeros([m, n], "bf16").partition([128, 256])
    res = launch.linear_tile_fp8_blk128(z, x, y, api.from_torch(sa), api.from_torch(sb), 1.0) \
        .sync_on(torch.cuda.current_stream())
    out = res[0].unpartition().storage
    rows, cols = slice(4090, 4098), slice(14300, 14428)
    ad = oracle.dequant_fp8_block(aq[rows].cpu().numpy(), sa[rows].cpu().numpy(), 1, 128)
    c0 = cols.start // 128 * 128
    bd = oracle.dequant_fp8_block(bq[c0:c0 + 256].cpu().numpy(), sb[c0 // 128:c0 // 128 + 2].cpu().numpy(), 128, 128)
    ref = oracle.cpu_gemm_nt(ad, bd, threads=0)[:, cols.start - c0:cols.stop - c0]
    assert oracle.rel_frobenius(out[rows, cols].float().cpu().numpy(), ref) <= FP8_TOL
    # scaling x's scales by 2 doubles the result bit-exactly (power-of-two scaling commutes with rounding)
    res2 = launch.linear_tile_fp8_blk128(api.zeros([m, n], "bf16").partition([128, 256]), x, y, api.from_torch(sa * 2),
                                         api.from_torch(sb), 1.0).sync_on(torch.cuda.current_stream())
    assert torch.equal(res2[0].unpartition().storage, out * 2)


def test_host_row_pipeline_gives_the_bits_of_one_call(b200):
    """`api.HostRowPipeline` over the fp8 linear layer: weights first, then ragged row slabs uploaded / multiplied /
    downloaded on three streams; twice on one plan; bit-identical to one call over device-resident operands."""
    m, n, k = 1100, 640, 512
    a, b = workloads.gemm_normal_inputs(m, n, k, config_index=31)
    aq, sa = quant.quant_fp8_block(a, 1, 128)
    bq, sb = quant.quant_fp8_block(b, 128, 128)
    want = _run(b200, aq.cuda(), bq.cuda(), sa.cuda(), sb.cuda(), m, n, k).cpu()
    host = [t.pin_memory() for t in (aq, sa, bq, sb)]
    dev = [torch.empty_like(t, device="cuda") for t in (aq, sa, bq, sb)]
    z = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    zh = torch.full((m, n), float("nan"), dtype=torch.bfloat16).pin_memory()

    def rows(r0, r1, s):
        _lib.check(b200.b200tile_linear_fp8_blk128(dev[0][r0:].data_ptr(), dev[2].data_ptr(), dev[1][r0:].data_ptr(),
                                                   dev[3].data_ptr(), z[r0:].data_ptr(), b"bf16", r1 - r0, n, k, k, k, n,
                                                   k // 128, k // 128, 1.0, s.cuda_stream))
    pipe = api.HostRowPipeline(m, 256)
    for _ in range(2):
        pipe([(host[2], dev[2]), (host[3], dev[3])], [(host[0], dev[0]), (host[1], dev[1])], [(z, zh)], rows)
        torch.cuda.current_stream().synchronize()
        assert torch.equal(zh, want)
        zh.fill_(float("nan"))
        for d in dev:
            d.zero_()
    with pytest.raises(ValueError, match="one entry per row"):
        pipe([], [(host[2], dev[2])], [(z, zh)], rows)
