"""MXFP8 (e4m3 data, e8m0 scale per 32) block-scaled GEMM parity on a B200."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from cutile_rs_b200 import _lib, quant, workloads  # noqa: E402


def _run(lib, xq, yq, xs, ys, m, n, k, out, alpha=1.0):
    z = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32 if out == "f32" else torch.bfloat16)
    need = lib.b200tile_linear_mxfp8_workspace_bytes(m, n, k)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    _lib.check(lib.b200tile_linear_mxfp8(xq.data_ptr(), yq.data_ptr(), xs.data_ptr(), ys.data_ptr(), z.data_ptr(),
                                         out.encode(), m, n, k, k, k, n, k // 32, k // 32, alpha, ws.data_ptr(), need,
                                         torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return z


def test_reference_known_answer(b200):
    # cutile-examples/examples/mxfp8.rs:84-92,129-135: fp8 0x38 (1.0), E8M0 0x7F (1.0), 16x16x128 -> 128
    m = n = 16
    k = 128
    x = torch.full((m, k), 0x38, dtype=torch.uint8, device="cuda")
    s = torch.full((m, k // 32), 0x7F, dtype=torch.uint8, device="cuda")
    z = _run(b200, x, x, s, s, m, n, k, "f32")
    assert torch.all((z - 128.0).abs() <= 1e-3)


@pytest.mark.parametrize("m,n,k,out", [(128, 224, 128, "f32"), (256, 448, 512, "f32"), (200, 328, 384, "bf16"),
                                       (1024, 1000, 1024, "bf16")])
def test_matches_oracle(b200, oracle, m, n, k, out):
    a, b = workloads.gemm_normal_inputs(m, n, k, config_index=5)
    xq, xs = quant.quant_mxfp8(a)
    yq, ys = quant.quant_mxfp8(b)
    xq_o, xs_o = oracle.quant_mxfp8(a.numpy())
    assert np.array_equal(xq.numpy(), xq_o) and np.array_equal(xs.numpy(), xs_o)
    got = _run(b200, xq.cuda(), yq.cuda(), xs.cuda(), ys.cuda(), m, n, k, out, 0.25).float().cpu().numpy()
    ref = oracle.cpu_gemm_nt(oracle.dequant_mxfp8(xq.numpy(), xs.numpy()), oracle.dequant_mxfp8(yq.numpy(), ys.numpy()),
                             alpha=0.25, threads=0)
    assert not np.isnan(got).any()
    assert oracle.rel_frobenius(got, ref) <= (3e-2 if out == "bf16" else 1e-5)
    full = oracle.cpu_gemm_nt(a.numpy(), b.numpy(), alpha=0.25, threads=0)
    assert oracle.rel_frobenius(got, full) <= 6e-2


@pytest.mark.parametrize("m", [256, 640])     # single-CTA kernel / CTA-pair kernel (from 512 rows)
def test_scale_byte_selection(b200, oracle, m):
    # different power-of-two scales in every 32-block and row: checks the per-MMA scale-byte select
    n, k = 448, 256
    g = torch.Generator().manual_seed(3)
    xq = torch.randint(0, 0x78, (m, k), generator=g, dtype=torch.uint8)
    yq = torch.randint(0, 0x78, (n, k), generator=g, dtype=torch.uint8)
    xs = (120 + torch.randint(0, 12, (m, k // 32), generator=g)).to(torch.uint8)
    ys = (120 + torch.randint(0, 12, (n, k // 32), generator=g)).to(torch.uint8)
    got = _run(b200, xq.cuda(), yq.cuda(), xs.cuda(), ys.cuda(), m, n, k, "f32").cpu().numpy()
    ref = oracle.cpu_gemm_nt(oracle.dequant_mxfp8(xq.numpy(), xs.numpy()), oracle.dequant_mxfp8(yq.numpy(), ys.numpy()),
                             threads=0)
    assert oracle.rel_frobenius(got, ref) <= 1e-5


def test_full_size_slab_and_scale_linearity(b200, oracle):
    """The benchmark's MXFP8 shape at full size (8192 x 28672 x 8192, CTA-pair kernel): device-side generation, an
    oracle slab that straddles tile and CTA boundaries, and a size-independent property: adding 1 to every E8M0 scale
    byte of x doubles the result bit for bit."""
    m, n, k = 8192, 28672, 8192
    g = torch.Generator(device="cuda").manual_seed(workloads.SEED_BASE + 13)
    xq, xs = quant.quant_mxfp8(torch.randn(m, k, device="cuda", generator=g))
    yq, ys = quant.quant_mxfp8(torch.randn(n, k, device="cuda", generator=g))
    out = _run(b200, xq, yq, xs, ys, m, n, k, "bf16", 1.0)
    rows, cols = slice(4090, 4102), slice(14300, 14428)
    ref = oracle.cpu_gemm_nt(oracle.dequant_mxfp8(xq[rows].cpu().numpy(), xs[rows].cpu().numpy()),
                             oracle.dequant_mxfp8(yq[cols].cpu().numpy(), ys[cols].cpu().numpy()), threads=0)
    assert oracle.rel_frobenius(out[rows, cols].float().cpu().numpy(), ref) <= 3e-2
    assert not torch.isnan(out.float()).any()
    out2 = _run(b200, xq, yq, xs + 1, ys, m, n, k, "bf16", 1.0)
    assert torch.equal(out2, out * 2)
    st = _lib.StatusC()
    _lib.check(b200.b200tile_status(torch.cuda.current_stream().cuda_stream, st))
    assert st.code == 0
