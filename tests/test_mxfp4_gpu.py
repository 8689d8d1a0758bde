"""MXFP4 (packed e2m1 data, e8m0 scale per 32) block-scaled GEMM parity on a B200: the operand / scale pairing of
`raw_mmaf_scaled_nvfp4_kernel` (cutile/tests/tensor_and_matrix_ops.rs:224-244) at `linear_tile` scale."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from cutile_rs_b200 import _lib, api, launch, quant, workloads  # noqa: E402


def _run(lib, xq, yq, xs, ys, m, n, k, out, alpha=1.0):
    z = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32 if out == "f32" else torch.bfloat16)
    need = lib.b200tile_linear_mxfp4_workspace_bytes(m, n, k)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    _lib.check(lib.b200tile_linear_mxfp4(xq.data_ptr(), yq.data_ptr(), xs.data_ptr(), ys.data_ptr(), z.data_ptr(),
                                         out.encode(), m, n, k, k // 2, k // 2, n, k // 32, k // 32, alpha, ws.data_ptr(),
                                         need, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    st = _lib.StatusC()
    _lib.check(lib.b200tile_status(torch.cuda.current_stream().cuda_stream, st))
    assert st.code == 0
    return z


def test_known_answer(b200):
    # nibble 0x2 = 1.0 (cutile/tests/tensor_and_matrix_ops.rs:622-682), E8M0 0x7F = 1.0 (mxfp8.rs:91-92): K ones -> K;
    # scale 0x80 = 2.0 on one side doubles it
    m = n = 16
    k = 128
    x = torch.full((m, k // 2), 0x22, dtype=torch.uint8, device="cuda")
    s1 = torch.full((m, k // 32), 0x7F, dtype=torch.uint8, device="cuda")
    s2 = torch.full((m, k // 32), 0x80, dtype=torch.uint8, device="cuda")
    assert torch.all(_run(b200, x, x, s1, s1, m, n, k, "f32") == 128.0)
    assert torch.all(_run(b200, x, x, s2, s1, m, n, k, "f32") == 256.0)


@pytest.mark.parametrize("m,n,k,out", [(128, 192, 128, "f32"), (256, 448, 512, "f32"), (200, 328, 384, "bf16"),
                                       (1024, 1000, 1024, "bf16"), (16, 512, 1024, "f32")])
def test_matches_oracle(b200, oracle, m, n, k, out):
    a, b = workloads.gemm_normal_inputs(m, n, k, config_index=8)
    xq, xs = quant.quant_mxfp4(a)
    yq, ys = quant.quant_mxfp4(b)
    dx, dy = oracle.dequant_mxfp4(xq.numpy(), xs.numpy()), oracle.dequant_mxfp4(yq.numpy(), ys.numpy())
    assert oracle.rel_frobenius(dx, a.numpy()) < 0.2          # the quantiser and the dequantiser agree on the format
    got = _run(b200, xq.cuda(), yq.cuda(), xs.cuda(), ys.cuda(), m, n, k, out, 0.25).float().cpu().numpy()
    ref = oracle.cpu_gemm_nt(dx, dy, alpha=0.25, threads=0)
    assert not np.isnan(got).any()
    assert oracle.rel_frobenius(got, ref) <= (3e-2 if out == "bf16" else 1e-5)


@pytest.mark.parametrize("m", [256, 640])     # single-CTA kernel / CTA-pair kernel (from 512 rows)
def test_scale_byte_pair_selection(b200, oracle, m):
    # different power-of-two scales in every 32-block and row: checks the byte pair each K = 64 instruction picks
    n, k = 448, 512
    g = torch.Generator().manual_seed(4)
    xq = torch.randint(0, 256, (m, k // 2), generator=g, dtype=torch.uint8)
    yq = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8)
    xs = (120 + torch.randint(0, 12, (m, k // 32), generator=g)).to(torch.uint8)
    ys = (120 + torch.randint(0, 12, (n, k // 32), generator=g)).to(torch.uint8)
    got = _run(b200, xq.cuda(), yq.cuda(), xs.cuda(), ys.cuda(), m, n, k, "f32").cpu().numpy()
    ref = oracle.cpu_gemm_nt(oracle.dequant_mxfp4(xq.numpy(), xs.numpy()), oracle.dequant_mxfp4(yq.numpy(), ys.numpy()),
                             threads=0)
    assert oracle.rel_frobenius(got, ref) <= 1e-5


def test_through_the_generic_linear_tile_name(b200, oracle):
    m, n, k = 200, 328, 384
    a, b = workloads.gemm_normal_inputs(m, n, k, config_index=9)
    xq, xs = quant.quant_mxfp4(a)
    yq, ys = quant.quant_mxfp4(b)
    x, y = api.from_torch(xq.cuda(), "f4e2m1fnx2"), api.from_torch(yq.cuda(), "f4e2m1fnx2")
    sx, sy = api.from_torch(xs.cuda(), "f8e8m0fnu"), api.from_torch(ys.cuda(), "f8e8m0fnu")
    z = api.from_torch(torch.full((m, n), float("nan"), device="cuda")).partition([64, 64])
    launch.linear_tile(z, x, y, sx, sy, 0.5).sync_on(torch.cuda.current_stream())
    got = z.unpartition().to_host().numpy()
    ref = oracle.cpu_gemm_nt(oracle.dequant_mxfp4(xq.numpy(), xs.numpy()), oracle.dequant_mxfp4(yq.numpy(), ys.numpy()),
                             alpha=0.5, threads=0)
    assert oracle.rel_frobenius(got, ref) <= 1e-5
    # the same call with explicit generics [BM, BN, BK, BK_PACKED, BK_SCALES = BK / 32]
    z2 = api.from_torch(torch.full((m, n), float("nan"), device="cuda")).partition([64, 64])
    launch.linear_tile(z2, x, y, sx, sy, 0.5).generics(["64", "64", "128", "64", "4"]).sync_on(torch.cuda.current_stream())
    assert torch.equal(z2.unpartition().storage, z.unpartition().storage)
