"""Grouped (MoE) GEMM over device-side pointer / extent tables against the CPU oracle GEMM."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from cutile_rs_b200 import _lib, api, launch

GEMM_TOL = 1e-2   # relative Frobenius error of a 16-bit GEMM with fp32 accumulation


def _groups(shapes, dtype, seed, pad=0):
    g = torch.Generator().manual_seed(seed)
    a, b, c = [], [], []
    for (m, n, k) in shapes:
        # padded row strides exercise the {rows, cols, stride} extent records
        # (row strides are multiples of 8 elements: the 16-byte rule of the kernel's copies)
        lda, ldn = (k + pad + 7) // 8 * 8, (n + pad + 7) // 8 * 8
        fa = torch.zeros(max(m, 1), lda, dtype=dtype)
        fa[:, :k] = (torch.randn(max(m, 1), k, generator=g) / 4).to(dtype)
        fb = torch.zeros(max(k, 1), ldn, dtype=dtype)
        fb[:, :n] = (torch.randn(max(k, 1), n, generator=g) / 4).to(dtype)
        a.append(fa.cuda()[:m, :k])
        b.append(fb.cuda()[:k, :n])
        c.append(torch.full((max(m, 1), ldn), float("nan"), dtype=dtype, device="cuda")[:m, :n])
    return a, b, c


def _check(oracle, a, b, c):
    for ai, bi, ci in zip(a, b, c):
        if ai.shape[0] == 0:
            continue
        got = ci.float().cpu().numpy()
        assert not np.isnan(got).any()
        if ai.shape[1] == 0:
            assert not got.any()
            continue
        ref = oracle.cpu_gemm(ai.float().cpu().numpy(), bi.float().cpu().numpy(), threads=0)
        assert oracle.rel_frobenius(got, ref) <= GEMM_TOL


@pytest.mark.parametrize("dtype,bn", [(torch.bfloat16, 256), (torch.float16, 128)])
def test_groups_of_many_shapes(b200, oracle, dtype, bn):
    shapes = [(128, 256, 64), (16, 512, 128), (300, 272, 192), (0, 256, 64), (48, 16, 80), (1024, 768, 256),
              (128, 256, 64), (64, 1024, 512)]
    a, b, c = _groups(shapes, dtype, seed=17, pad=8)
    tabs = launch.group_gemm_tables(a, b, c)
    name = "bf16" if dtype == torch.bfloat16 else "f16"
    launch.group_gemm_f16_nt_desc(*tabs, len(shapes), dtype=name, bn=bn).sync()
    _check(oracle, a, b, c)
    st = _lib.StatusC()
    _lib.check(b200.b200tile_status(torch.cuda.current_stream().cuda_stream, st))
    assert st.code == 0


def test_typed_entry_with_caller_workspace_and_graph(b200, oracle):
    """Many small experts (more groups than one prepare pass of 256), a caller workspace, and a
    captured graph replayed after the token counts changed on the device."""
    rng = np.random.default_rng(3)
    shapes = [(int(rng.integers(1, 5)) * 16, 256, 128) for _ in range(300)]
    a, b, c = _groups(shapes, torch.bfloat16, seed=5)
    ap, bp, cp, am, bm, cm = launch.group_gemm_tables(a, b, c)
    need = b200.b200tile_group_gemm_workspace_bytes(len(shapes))
    ws = torch.empty(need + 128, dtype=torch.uint8, device="cuda")
    wp = (ws.data_ptr() + 127) // 128 * 128
    stream = torch.cuda.Stream()

    def run(s):
        _lib.check(b200.b200tile_group_gemm(b"bf16", ap.cu_deviceptr(), bp.cu_deviceptr(), cp.cu_deviceptr(),
                                            am.cu_deviceptr(), bm.cu_deviceptr(), cm.cu_deviceptr(), len(shapes), 256,
                                            wp, need, s.cuda_stream))
    torch.cuda.synchronize()
    run(stream)
    stream.synchronize()
    _check(oracle, a, b, c)
    st = _lib.StatusC()
    _lib.check(b200.b200tile_status(stream.cuda_stream, st))
    assert st.code == 0
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        run(torch.cuda.current_stream())
    # halve every expert's row count on the device only; rows past the new count must stay untouched
    for ci in c:
        ci.fill_(7.0)
    am.storage[:, 0] //= 2
    g.replay()
    torch.cuda.synchronize()
    for (m, n, k), ai, bi, ci in zip(shapes, a, b, c):
        h = m // 2
        if h:
            ref = oracle.cpu_gemm(ai[:h].float().cpu().numpy(), bi.float().cpu().numpy())
            assert oracle.rel_frobenius(ci[:h].float().cpu().numpy(), ref) <= GEMM_TOL
        assert (ci[h:] == 7.0).all()
    with pytest.raises(_lib.B200TileError, match="workspace"):
        _lib.check(b200.b200tile_group_gemm(b"bf16", ap.cu_deviceptr(), bp.cu_deviceptr(), cp.cu_deviceptr(),
                                            am.cu_deviceptr(), bm.cu_deviceptr(), cm.cu_deviceptr(), len(shapes), 256,
                                            wp, need - 1, stream.cuda_stream))


def test_ragged_extents_leave_neighbouring_memory_alone(b200, oracle):
    """Extents that are not multiples of the tile, of 8 elements or of the k slab: rows, columns and k past a
    group's extents are neither read into the product nor written."""
    shapes = [(130, 264, 72), (1, 8, 8), (257, 40, 200), (33, 520, 136), (64, 24, 64), (20, 36, 100), (7, 3, 5)]
    a, b, c = _groups(shapes, torch.float16, seed=23, pad=16)
    # poison what lies behind every operand's extents: it must not reach the result
    for t in a + b:
        base = t._base if t._base is not None else t
        base[:, t.shape[1]:] = float("nan")
    tabs = launch.group_gemm_tables(a, b, c)
    launch.group_gemm_f16_nt_desc(*tabs, len(shapes), dtype="f16", bn=128).sync()
    _check(oracle, a, b, c)
    for ci in c:
        assert torch.isnan(ci._base[:, ci.shape[1]:]).all()      # the padding columns of C keep their NaN fill
    st = _lib.StatusC()
    _lib.check(b200.b200tile_status(torch.cuda.current_stream().cuda_stream, st))
    assert st.code == 0


def test_group_that_breaks_the_16_byte_rule_is_skipped_and_reported(b200, oracle):
    """The tables live on the device, so the call cannot refuse a bad group: the kernel skips it (its C stays
    untouched), reports it through the status record and computes the other groups."""
    shapes = [(64, 128, 64), (32, 128, 64), (48, 256, 128)]
    a, b, c = _groups(shapes, torch.bfloat16, seed=29)
    ap, bp, cp, am, bm, cm = launch.group_gemm_tables(a, b, c)
    ap.storage[1] += 2           # group 1: A no longer 16-byte aligned
    s = torch.cuda.current_stream().cuda_stream
    _lib.check(b200.b200tile_status_reset(s))
    launch.group_gemm_f16_nt_desc(ap, bp, cp, am, bm, cm, len(shapes), dtype="bf16", bn=256).sync()
    st = _lib.StatusC()
    rc = b200.b200tile_status(s, st)
    assert rc == 4 and st.code == 3 and st.site == 1
    _lib.check(b200.b200tile_status_reset(s))
    assert torch.isnan(c[1]).all()
    _check(oracle, [a[0], a[2]], [b[0], b[2]], [c[0], c[2]])
