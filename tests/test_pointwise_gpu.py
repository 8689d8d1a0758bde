"""Element-wise kernels (`b200tile_add_2d`, `b200tile_silu_mul_2d`) against the oracle's restatement of
cutile-kernels/src/pointwise.rs.  The sum is one rounding of an exact value and must match bit for bit; the SwiGLU
product goes through `expf`, which may differ from the oracle's exp in the last place of fp32, so it is compared to
one unit in the last place of the 16-bit type."""
import numpy as np
import pytest
import torch

from cutile_rs_b200 import _lib, api, launch

pytestmark = pytest.mark.gpu


def _stream():
    return torch.cuda.current_stream()


def _pair(rows, cols, dtype, pitch, seed):
    g = torch.Generator().manual_seed(seed)
    pitch = pitch or cols
    a = torch.zeros(rows, pitch, dtype=dtype)
    b = torch.zeros(rows, pitch, dtype=dtype)
    a[:, :cols] = (torch.randn(rows, cols, generator=g) * 3).to(dtype)
    b[:, :cols] = (torch.randn(rows, cols, generator=g) * 2).to(dtype)
    return a, b


CASES = [(64, 4096, torch.float16, None), (33, 1000, torch.float16, None), (7, 1001, torch.float16, None),
         (5, 24, torch.bfloat16, 40), (129, 14336, torch.bfloat16, None), (3, 5, torch.float16, None)]


@pytest.mark.parametrize("rows,cols,dtype,pitch", CASES)
def test_add_is_exact(b200, rows, cols, dtype, pitch):
    a, b = _pair(rows, cols, dtype, pitch, rows + cols)
    ad, bd = a.cuda(), b.cuda()
    out = torch.full_like(ad, 9.0)
    ld = a.stride(0)
    name = b"f16" if dtype == torch.float16 else b"bf16"
    _lib.check(b200.b200tile_add_2d(name, out.data_ptr(), ad.data_ptr(), bd.data_ptr(), rows, cols, ld, ld, ld,
                                    _stream().cuda_stream))
    torch.cuda.synchronize()
    want = (a[:, :cols].float() + b[:, :cols].float()).to(dtype)     # exact fp32 sum, one rounding
    assert torch.equal(out[:, :cols].cpu(), want)
    if ld > cols:
        assert (out[:, cols:] == 9.0).all()


@pytest.mark.parametrize("rows,cols,dtype,pitch", CASES)
def test_silu_mul_matches_oracle(b200, oracle, rows, cols, dtype, pitch):
    a, b = _pair(rows, cols, dtype, pitch, 7 * rows + cols)
    ad, bd = a.cuda(), b.cuda()
    out = torch.full_like(ad, 9.0)
    ld = a.stride(0)
    f16 = dtype == torch.float16
    _lib.check(b200.b200tile_silu_mul_2d(b"f16" if f16 else b"bf16", out.data_ptr(), ad.data_ptr(), bd.data_ptr(), rows,
                                         cols, ld, ld, ld, _stream().cuda_stream))
    torch.cuda.synchronize()
    ref = oracle.silu_mul(a[:, :cols].float().numpy(), b[:, :cols].float().numpy(), is_f16=f16)
    got = out[:, :cols].float().cpu().numpy()
    ulp = 2.0 ** -10 if f16 else 2.0 ** -7
    assert np.all(np.abs(got - ref) <= ulp * np.abs(ref) + 1e-6)
    assert np.mean(got == ref) > 0.99          # differences are rare last-place flips, not a different formula


def test_launchers_in_place_and_errors(b200, oracle):
    rows, cols = 48, 2048
    a, b = _pair(rows, cols, torch.float16, None, 5)
    ad, bd = api.copy_host_to_device(a), api.copy_host_to_device(b)
    out = api.zeros([rows, cols], "f16").partition([1, 512])
    (out, _a, _b) = launch.add_2d_f16(out, ad, bd).sync_on(_stream())
    assert torch.equal(out.unpartition().to_host(), (a.float() + b.float()).half())
    out2 = api.zeros([rows, cols], "f16").partition([1, 1024])
    (out2, _a, _b) = launch.silu_mul_2d_f16(out2, ad, bd).sync_on(_stream())
    ref = oracle.silu_mul(a.float().numpy(), b.float().numpy(), is_f16=True)
    assert np.all(np.abs(out2.unpartition().to_host().float().numpy() - ref) <= 2.0 ** -10 * np.abs(ref) + 1e-6)
    # in place: the residual stream updated with x += y
    x, y = a.cuda(), b.cuda()
    _lib.check(b200.b200tile_add_2d(b"f16", x.data_ptr(), x.data_ptr(), y.data_ptr(), rows, cols, cols, cols, cols,
                                    _stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(x.cpu(), (a.float() + b.float()).half())
    s = _stream().cuda_stream
    assert b200.b200tile_add_2d(b"f32", x.data_ptr(), x.data_ptr(), y.data_ptr(), rows, cols, cols, cols, cols, s) != 0
    assert b200.b200tile_silu_mul_2d(b"f16", x.data_ptr(), x.data_ptr(), y.data_ptr(), rows, cols, 8, cols, cols, s) != 0
    assert b"pitch" in b200.b200tile_last_error()
    with pytest.raises(Exception, match="output partition"):
        launch.add_2d_f16(api.zeros([rows, cols], "f16").partition([2, 512]), ad, bd).sync_on(_stream())
