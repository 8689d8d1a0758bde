"""A bounded wait that actually runs out.

Every mbarrier wait in the kernels polls with a limit; when the limit is reached the CTA records
{code 1, block, wait site} in the device status record, leaves through its normal exit (Tensor Memory
freed) and the host reads the record with `b200tile_status`.  This test makes one wait run out without
faulting, trapping or hanging anything: it loads `libb200tile_waittest.so`, the same sources built with a
wait limit of 2^20 SM cycles (about half a millisecond) and a producer hook that, when armed, leaves one
k-slab of one tile unloaded, so that the MMA thread's wait for that stage can never be satisfied.  The
product library contains neither the hook nor the short limit.
"""
import ctypes
import os
import time
from ctypes import c_char_p, c_int, c_int64, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

from cutile_rs_b200 import _lib, workloads  # noqa: E402

VARIANT = os.path.join(os.path.dirname(_lib.LIB_PATH), "libb200tile_waittest.so")
SITE_MMA_WAITS_FOR_STAGE = 3   # the wait of the MMA-issuing thread on a stage's `full` barrier


def _load_variant():
    if not os.path.exists(VARIANT):
        raise RuntimeError(f"{VARIANT} is missing: `python -c 'import __graft_entry__ as g; g.build()'` builds it")
    # own symbols first: the product library is loaded in this process too and exports the same names
    lib = ctypes.CDLL(VARIANT, mode=os.RTLD_LOCAL | os.RTLD_DEEPBIND)
    for name in ("b200tile_init", "b200tile_gemm", "b200tile_status", "b200tile_status_reset", "b200tile_last_error"):
        res, args = _lib.SIGNATURES[name]
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    lib.b200tile_test_set_skip_stage.restype = c_int
    lib.b200tile_test_set_skip_stage.argtypes = [c_int]
    return lib


def _gemm(lib, a, b, c, stream):
    m, k = a.shape
    n = b.shape[1]
    return lib.b200tile_gemm(b"bf16", 0, a.data_ptr(), b.data_ptr(), c.data_ptr(), 1, m, n, k, a.stride(0), b.stride(0),
                             c.stride(0), 0, 0, 0, 0, 0, 0, 0, stream)   # config 0: the 128 x 256 single-CTA kernel


def test_wait_runs_out_status_is_recorded_and_the_next_launch_is_clean(b200, oracle):
    var = _load_variant()
    assert var.b200tile_init(0) == 0
    m, n, k = 4096, 2048, 512          # 256 tiles: every SM runs a CTA that takes all of its Tensor Memory
    a, b = workloads.gemm_bf16_inputs(m, n, k, config_index=41)
    ad, bd = a.cuda(), b.cuda()
    s = torch.cuda.current_stream().cuda_stream
    want = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    assert _gemm(b200, ad, bd, want, s) == 0          # the product library's result
    torch.cuda.synchronize()
    ref = oracle.cpu_gemm(a[:32].float().numpy(), b.float().numpy(), threads=0)
    assert oracle.rel_frobenius(want[:32].float().cpu().numpy(), ref) <= 1e-2

    st = _lib.StatusC()
    assert var.b200tile_status_reset(s) == 0
    assert var.b200tile_test_set_skip_stage(1) == 0
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    t0 = time.perf_counter()
    assert _gemm(var, ad, bd, c, s) == 0               # the launch itself succeeds
    rc = var.b200tile_status(s, ctypes.byref(st))      # synchronises the stream
    waited = time.perf_counter() - t0
    assert rc == _lib.ERR_DEVICE and b"device status 1" in var.b200tile_last_error()
    assert (st.code, st.block, st.site) == (1, 0, SITE_MMA_WAITS_FOR_STAGE)
    assert waited < 5.0                                 # gave up after the limit, did not hang
    # the other CTAs finished their tiles; the tile of the CTA that gave up was not stored
    assert torch.isnan(c[:128, :256].float()).all()
    assert torch.equal(c[128:256], want[128:256])

    # disarmed, after a status reset: the same library computes the whole problem, bit for bit, on every SM
    assert var.b200tile_test_set_skip_stage(0) == 0
    assert var.b200tile_status_reset(s) == 0
    for _ in range(2):
        c.fill_(float("nan"))
        assert _gemm(var, ad, bd, c, s) == 0
        assert var.b200tile_status(s, ctypes.byref(st)) == 0 and st.code == 0
        assert torch.equal(c, want)
    # and the product library never saw any of it
    _lib.check(b200.b200tile_status(s, ctypes.byref(st)))
    assert st.code == 0
