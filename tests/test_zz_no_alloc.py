"""The allocation-free NVFP4 entry point against the workspace-taking one.

`b200tile_linear_nvfp4_static` exists for callers that cannot hand the library any device memory
(graph-capturing threads that must not touch an allocator, plugins barred from their host's
memory pool, start-up code that runs before an allocator exists); it keeps its scale scratch in a
fixed array inside the library.  The array is shared by every call and keeps the previous call's
contents, so the check runs two different problems back to back through the C ABI and compares
each with the regular entry point and with the oracle's dequantised fp32 reference.  This file sorts
last on purpose: a run that stops at the first failure has then already executed every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from cutile_rs_b200 import _lib, quant  # noqa: E402


def _problem(m, n, k, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn(m, k, device="cuda", generator=g)
    b = torch.randn(n, k, device="cuda", generator=g)
    xp, xs, ga = quant.quant_nvfp4(a)
    yp, ys, gb = quant.quant_nvfp4(b)
    return xp, yp, xs, ys, ga * gb


def _call(lib, static, prob, m, n, k, out):
    xp, yp, xs, ys, alpha = prob
    z = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16 if out == "bf16" else torch.float32)
    stream = torch.cuda.current_stream().cuda_stream
    common = (xp.data_ptr(), yp.data_ptr(), xs.data_ptr(), ys.data_ptr(), z.data_ptr(), out.encode(), m, n, k,
              k // 2, k // 2, n, k // 16, k // 16, alpha)
    if static:
        rc = lib.b200tile_linear_nvfp4_static(*common, -1, stream)
    else:
        need = lib.b200tile_linear_nvfp4_workspace_bytes(m, n, k)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        rc = lib.b200tile_linear_nvfp4(*common, ws.data_ptr(), need, -1, stream)
    _lib.check(rc)
    torch.cuda.synchronize()
    return z


def test_static_scratch_entry_point_matches_workspace_entry_point(b200, oracle):
    lib = b200
    # two calls in a row on different shapes: the second must not be disturbed by what the first
    # left behind in the shared array (the first is larger, so stale scales surround the second's)
    cases = [(384, 1000, 1024, "bf16", 11), (100, 328, 320, "f32", 12)]
    for m, n, k, out, seed in cases:
        prob = _problem(m, n, k, seed)
        want = _call(lib, False, prob, m, n, k, out)
        got = _call(lib, True, prob, m, n, k, out)
        assert not torch.isnan(got.float()).any()
        # same kernels, same operands, same scale values: identical bits (well inside the 3e-2
        # relative-Frobenius contract of the block-scaled GEMM tests)
        assert torch.equal(got, want)
        rel = (got.float() - want.float()).norm() / want.float().norm()
        assert rel <= 3e-2
        # and against the CPU oracle: fp32 GEMM over the dequantised operands
        xp, yp, xs, ys, alpha = prob
        ref = oracle.cpu_gemm_nt(oracle.dequant_nvfp4(xp.cpu().numpy(), xs.cpu().numpy()),
                                 oracle.dequant_nvfp4(yp.cpu().numpy(), ys.cpu().numpy()), alpha=alpha, threads=0)
        assert oracle.rel_frobenius(got.float().cpu().numpy(), ref) <= (3e-2 if out == "bf16" else 1e-5)
        # a further static call takes no device memory: the free-memory figure does not move
        z = torch.empty_like(got)
        stream = torch.cuda.current_stream().cuda_stream
        common = (xp.data_ptr(), yp.data_ptr(), xs.data_ptr(), ys.data_ptr(), z.data_ptr(), out.encode(), m, n, k,
                  k // 2, k // 2, n, k // 16, k // 16, alpha)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        _lib.check(lib.b200tile_linear_nvfp4_static(*common, -1, stream))
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] >= free_before
        assert torch.equal(z, want)
    st = _lib.StatusC()
    _lib.check(lib.b200tile_status(torch.cuda.current_stream().cuda_stream, ctypes.byref(st)))
    assert st.code == 0


def test_static_scratch_entry_point_rejects_oversized_problems(b200):
    lib = b200
    dummy = torch.zeros(64, dtype=torch.uint8, device="cuda")
    # 16384 x 16384 x 8192 needs about 25 MB of scale scratch: beyond the 8 MiB built-in array
    rc = lib.b200tile_linear_nvfp4_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                          dummy.data_ptr(), b"bf16", 16384, 16384, 8192, 4096, 4096, 16384, 512,
                                          512, 1.0, -1, None)
    assert rc == _lib.ERR_INVALID
    msg = lib.b200tile_last_error().decode()
    assert "built-in buffer holds" in msg and "caller workspace" in msg
