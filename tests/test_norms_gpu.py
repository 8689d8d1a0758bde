"""RMSNorm / residual-add + RMSNorm (`b200tile_rms_norm`, `b200tile_add_rms_norm`) against the oracle's
restatement of cutile-kernels/src/norms.rs.  The updated residual is a rounded fp32 sum of two 16-bit values
and must match bit for bit; the normalised output depends on the order of the fp32 additions of the squares,
which the reference leaves to its compiler, so it is compared to two units in the last place of the 16-bit type."""
import ctypes
import math

import numpy as np
import pytest
import torch

from cutile_rs_b200 import _lib, api, launch

pytestmark = pytest.mark.gpu

ULP = {torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7}


def _stream():
    return torch.cuda.current_stream()


def _close(got, ref, dtype):
    tol = 2 * ULP[dtype] * np.abs(ref) + 1e-3
    bad = np.abs(got - ref) > tol
    assert not bad.any(), f"{bad.sum()} of {bad.size} beyond 2 ulp; worst {np.abs(got - ref).max()}"


def _inputs(rows, n, dtype, pitch=None, seed=0):
    g = torch.Generator().manual_seed(1234 + seed)
    pitch = pitch or n
    x = torch.zeros(rows, pitch, dtype=dtype)
    r = torch.zeros(rows, pitch, dtype=dtype)
    x[:, :n] = (torch.randn(rows, n, generator=g) * 1.5).to(dtype)
    r[:, :n] = (torch.randn(rows, n, generator=g) * 0.7 + 0.1).to(dtype)
    w = (1.0 + 0.2 * torch.randn(n, generator=g)).to(dtype)
    return r, x, w


@pytest.mark.parametrize("rows,n,dtype,pitch", [
    (64, 4096, torch.float16, None), (333, 4096, torch.float16, None), (17, 128, torch.float16, None),
    (5, 8192, torch.float16, None), (3, 16384, torch.float16, None), (9, 1000, torch.float16, None),
    (7, 1001, torch.float16, None), (6, 2048, torch.float16, 2056), (31, 5120, torch.bfloat16, None),
    (4, 24, torch.bfloat16, 40),
])
def test_add_rms_norm_matches_oracle(b200, oracle, rows, n, dtype, pitch):
    r, x, w = _inputs(rows, n, dtype, pitch, seed=rows + n)
    ld = x.stride(0)
    rd, xd, wd = r.cuda(), x.cuda(), w.cuda()
    out = torch.full_like(xd, 7.0)
    rout = torch.full_like(xd, 7.0)
    name = b"f16" if dtype == torch.float16 else b"bf16"
    _lib.check(b200.b200tile_add_rms_norm(name, rd.data_ptr(), xd.data_ptr(), wd.data_ptr(), out.data_ptr(),
                                          rout.data_ptr(), rows, n, ld, ld, ld, ld, 1e-5, _stream().cuda_stream))
    torch.cuda.synchronize()
    ref_out, ref_res = oracle.add_rms_norm(r[:, :n].float().numpy(), x[:, :n].float().numpy(), w.float().numpy(),
                                           1e-5, is_f16=dtype == torch.float16)
    assert np.array_equal(rout[:, :n].float().cpu().numpy(), ref_res)
    _close(out[:, :n].float().cpu().numpy(), ref_out, dtype)
    if ld > n:   # the padding between rows is not written
        assert (out[:, n:] == 7.0).all() and (rout[:, n:] == 7.0).all()


@pytest.mark.parametrize("rows,n", [(40, 4096), (128, 128), (2, 12288), (3, 77)])
def test_rms_norm_matches_oracle(b200, oracle, rows, n):
    _, x, w = _inputs(rows, n, torch.float16, seed=n)
    xd, wd = x.cuda(), w.cuda()
    out = torch.empty_like(xd)
    _lib.check(b200.b200tile_rms_norm(b"f16", xd.data_ptr(), wd.data_ptr(), out.data_ptr(), rows, n, n, n, 1e-6,
                                      _stream().cuda_stream))
    torch.cuda.synchronize()
    ref, none = oracle.add_rms_norm(None, x.float().numpy(), w.float().numpy(), 1e-6)
    assert none is None
    _close(out.float().cpu().numpy(), ref, torch.float16)


def test_in_place_and_reference_shaped_launchers(b200, oracle):
    """The generated-launcher form (`add_rms_norm_f16(residual, x, w, out, residual_out, eps)` with [1, N]
    output partitions, grid = rows) and the in-place use of the transformer block: the updated residual
    overwrites the residual, the normalised row overwrites x."""
    rows, n = 96, 4096
    r, x, w = _inputs(rows, n, torch.float16, seed=5)
    ref_out, ref_res = oracle.add_rms_norm(r.float().numpy(), x.float().numpy(), w.float().numpy(), 1e-5)
    rd, xd, wd = (api.copy_host_to_device(t) for t in (r, x, w))
    out = api.zeros([rows, n], "f16").partition([1, n])
    rout = api.zeros([rows, n], "f16").partition([1, n])
    (_r, _x, _w, out, rout, _eps) = launch.add_rms_norm_f16(rd, xd, wd, out, rout, 1e-5).sync_on(_stream())
    assert np.array_equal(rout.unpartition().to_host().float().numpy(), ref_res)
    _close(out.unpartition().to_host().float().numpy(), ref_out, torch.float16)
    (_x, _w, o2, _eps) = launch.rms_norm_f16(xd, wd, api.zeros([rows, n], "f16").partition([1, n]), 1e-5) \
        .sync_on(_stream())
    ref2, _ = oracle.add_rms_norm(None, x.float().numpy(), w.float().numpy(), 1e-5)
    _close(o2.unpartition().to_host().float().numpy(), ref2, torch.float16)
    # in place through the typed entry point
    rt, xt, wt = r.cuda(), x.cuda(), w.cuda()
    _lib.check(b200.b200tile_add_rms_norm(b"f16", rt.data_ptr(), xt.data_ptr(), wt.data_ptr(), xt.data_ptr(),
                                          rt.data_ptr(), rows, n, n, n, n, n, 1e-5, _stream().cuda_stream))
    torch.cuda.synchronize()
    assert np.array_equal(rt.float().cpu().numpy(), ref_res)
    _close(xt.float().cpu().numpy(), ref_out, torch.float16)


def test_errors(b200):
    t = torch.zeros(4, 64, dtype=torch.float16, device="cuda")
    w = torch.ones(64, dtype=torch.float16, device="cuda")
    s = _stream().cuda_stream
    assert b200.b200tile_rms_norm(b"f32", t.data_ptr(), w.data_ptr(), t.data_ptr(), 4, 64, 64, 64, 1e-5, s) != 0
    assert b"unsupported element type" in b200.b200tile_last_error()
    assert b200.b200tile_rms_norm(b"f16", t.data_ptr(), w.data_ptr(), t.data_ptr(), 4, 64, 32, 64, 1e-5, s) != 0
    assert b"pitch" in b200.b200tile_last_error()
    assert b200.b200tile_add_rms_norm(b"f16", None, t.data_ptr(), w.data_ptr(), t.data_ptr(), t.data_ptr(), 4, 64,
                                      64, 64, 64, 64, 1e-5, s) != 0
    assert b200.b200tile_rms_norm(b"f16", t.data_ptr(), w.data_ptr(), t.data_ptr(), 0, 64, 64, 64, 1e-5, s) != 0
    with pytest.raises(Exception, match="output partition"):
        launch.rms_norm_f16(api.from_torch(t), api.from_torch(w), api.zeros([4, 64], "f16").partition([2, 64]),
                            1e-5).sync_on(_stream())


def test_full_size_properties(b200):
    """At a transformer's size (32768 tokens x 8192) against size-independent properties: a constant
    row c with unit weights normalises to c / sqrt(c^2 + eps) everywhere, scaling the weights scales the
    output, and the updated residual is the rounded sum."""
    rows, n = 32768, 8192
    x = torch.full((rows, n), 0.5, dtype=torch.float16, device="cuda")
    r = torch.full((rows, n), 1.5, dtype=torch.float16, device="cuda")
    w = torch.ones(n, dtype=torch.float16, device="cuda")
    out, rout = torch.empty_like(x), torch.empty_like(x)
    s = _stream().cuda_stream
    _lib.check(b200.b200tile_add_rms_norm(b"f16", r.data_ptr(), x.data_ptr(), w.data_ptr(), out.data_ptr(),
                                          rout.data_ptr(), rows, n, n, n, n, n, 1e-5, s))
    torch.cuda.synchronize()
    assert (rout == 2.0).all()
    want = torch.tensor(2.0 / math.sqrt(4.0 + 1e-5)).half()
    assert (out == want).all()
    w2 = torch.full_like(w, 0.25)
    out2 = torch.empty_like(x)
    _lib.check(b200.b200tile_add_rms_norm(b"f16", r.data_ptr(), x.data_ptr(), w2.data_ptr(), out2.data_ptr(),
                                          rout.data_ptr(), rows, n, n, n, n, n, 1e-5, s))
    torch.cuda.synchronize()
    assert torch.equal(out2.float(), out.float() * 0.25)
