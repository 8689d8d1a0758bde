"""Rotary position embedding (`b200tile_rope_seq`, generic names `rope_seq_f16` / `rope_seq_dynpos_f16`) against
the oracle's restatement of cutile-kernels/src/positional.rs.  cos and sin come from different libraries
(`sincosf` on the device, correctly rounded values in the oracle), one unit in the last place of f32 apart at
most, so the 16-bit results are compared to one unit in their last place."""
import ctypes

import numpy as np
import pytest
import torch

from cutile_rs_b200 import _lib, api, launch

pytestmark = pytest.mark.gpu
I2 = ctypes.c_int64 * 2


def _stream():
    return torch.cuda.current_stream()


def _inv_freq(d, base=10000.0):
    return (1.0 / base ** (torch.arange(0, d, 2, dtype=torch.float32) / d)).contiguous()


def _close(got, ref, ulp):
    bad = np.abs(got - ref) > ulp * np.abs(ref) + 1e-4
    assert not bad.any(), f"{bad.sum()} of {bad.size}; worst {np.abs(got - ref).max()}"


@pytest.mark.parametrize("seq,heads,d,pos,dtype", [
    (64, 32, 128, 0, torch.float16), (33, 8, 128, 4000, torch.float16), (1, 32, 128, 131071, torch.float16),
    (17, 5, 64, 7, torch.float16), (9, 3, 20, 100, torch.float16), (40, 16, 256, 12345, torch.bfloat16),
])
def test_matches_oracle(b200, oracle, seq, heads, d, pos, dtype):
    g = torch.Generator().manual_seed(seq * 131 + d)
    x = torch.randn(seq, heads, d, generator=g).to(dtype)
    f = _inv_freq(d)
    xd, fd = x.cuda(), f.cuda()
    out = torch.empty_like(xd)
    st = I2(heads * d, d)
    name = b"f16" if dtype == torch.float16 else b"bf16"
    _lib.check(b200.b200tile_rope_seq(name, xd.data_ptr(), fd.data_ptr(), out.data_ptr(), seq, heads, d, st, st, pos,
                                      None, _stream().cuda_stream))
    torch.cuda.synchronize()
    ref = oracle.rope_seq(x.float().numpy(), f.numpy(), pos, is_f16=dtype == torch.float16)
    _close(out.float().cpu().numpy(), ref, 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7)


def test_launchers_device_position_in_place_and_strides(b200, oracle):
    seq, heads, d, pos = 48, 8, 128, 777
    g = torch.Generator().manual_seed(3)
    x = torch.randn(seq, heads, d, generator=g).half()
    f = _inv_freq(d)
    ref = oracle.rope_seq(x.float().numpy(), f.numpy(), pos)
    xd, fd = api.copy_host_to_device(x), api.copy_host_to_device(f)
    out = api.zeros([seq, heads, d], "f16").partition([1, 1, d // 2])
    (_x, _f, out, _p) = launch.rope_seq_f16(xd, fd, out, pos).sync_on(_stream())
    _close(out.unpartition().to_host().float().numpy(), ref, 2.0 ** -10)
    # device-side position: the same launch object gives another result after the scalar is rewritten
    p = api.from_torch(torch.tensor([pos], dtype=torch.int32, device="cuda"))
    out2 = api.zeros([seq, heads, d], "f16").partition([1, 1, d // 2])
    op = launch.rope_seq_dynpos_f16(xd, fd, p, out2)
    (_x, _f, _p, o2) = op.sync_on(_stream())
    _close(o2.unpartition().to_host().float().numpy(), ref, 2.0 ** -10)
    p.storage.fill_(5)
    (_x, _f, _p, o2) = op.sync_on(_stream())
    _close(o2.unpartition().to_host().float().numpy(), oracle.rope_seq(x.float().numpy(), f.numpy(), 5), 2.0 ** -10)
    # in place, on a strided view (q inside a fused qkv buffer): heads*d of 3*heads*d columns per row
    qkv = torch.zeros(seq, 3 * heads * d, dtype=torch.float16, device="cuda")
    qkv[:, :heads * d] = x.cuda().reshape(seq, heads * d)
    st = I2(3 * heads * d, d)
    _lib.check(b200.b200tile_rope_seq(b"f16", qkv.data_ptr(), fd.cu_deviceptr(), qkv.data_ptr(), seq, heads, d, st, st,
                                      pos, None, _stream().cuda_stream))
    torch.cuda.synchronize()
    _close(qkv[:, :heads * d].reshape(seq, heads, d).float().cpu().numpy(), ref, 2.0 ** -10)
    assert (qkv[:, heads * d:] == 0).all()


def test_properties_and_errors(b200):
    """Position 0 is the identity; a rotation keeps the norm of every (lo, hi) pair; odd D is refused."""
    seq, heads, d = 4096, 32, 128
    x = torch.randn(seq, heads, d, device="cuda").half()
    f = _inv_freq(d).cuda()
    out = torch.empty_like(x)
    st = I2(heads * d, d)
    s = _stream().cuda_stream
    _lib.check(b200.b200tile_rope_seq(b"f16", x.data_ptr(), f.data_ptr(), out.data_ptr(), 1, heads, d, st, st, 0, None, s))
    torch.cuda.synchronize()
    assert torch.equal(out[0], x[0])
    _lib.check(b200.b200tile_rope_seq(b"f16", x.data_ptr(), f.data_ptr(), out.data_ptr(), seq, heads, d, st, st, 0, None, s))
    torch.cuda.synchronize()
    n_in = x.float()[..., :64] ** 2 + x.float()[..., 64:] ** 2
    n_out = out.float()[..., :64] ** 2 + out.float()[..., 64:] ** 2
    assert torch.allclose(n_in, n_out, rtol=4e-3, atol=1e-3)
    assert b200.b200tile_rope_seq(b"f16", x.data_ptr(), f.data_ptr(), out.data_ptr(), 4, heads, 127, st, st, 0, None, s) != 0
    assert b"even" in b200.b200tile_last_error()
    assert b200.b200tile_rope_seq(b"f32", x.data_ptr(), f.data_ptr(), out.data_ptr(), 4, heads, d, st, st, 0, None, s) != 0


def _qk_case(seq, qh, kvh, d, max_seq, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(seq, qh, d, generator=g).to(dtype)
    k = (torch.randn(seq, kvh, d, generator=g) * 2.0).to(dtype)
    v = torch.randn(seq, kvh, d, generator=g).to(dtype)
    qw = (1.0 + 0.1 * torch.randn(d, generator=g)).to(dtype)
    kw = (1.0 + 0.1 * torch.randn(d, generator=g)).to(dtype)
    kc = torch.randn(kvh, max_seq, d, generator=g).to(dtype)
    vc = torch.randn(kvh, max_seq, d, generator=g).to(dtype)
    return q, k, v, qw, kw, kc, vc


@pytest.mark.parametrize("seq,qh,kvh,d,max_seq,pos,dtype", [
    (40, 32, 8, 128, 256, 100, torch.float16), (7, 5, 3, 64, 64, 0, torch.float16),
    (3, 4, 4, 256, 16, 13, torch.bfloat16), (9, 2, 1, 16, 32, 5, torch.float16),
    # 512 positions and more take the small-CTA configuration of the kernel
    (600, 8, 2, 128, 640, 17, torch.float16), (512, 3, 1, 64, 512, 0, torch.bfloat16),
])
def test_qk_norm_rope_kv_prefill(b200, oracle, seq, qh, kvh, d, max_seq, pos, dtype):
    q, k, v, qw, kw, kc, vc = _qk_case(seq, qh, kvh, d, max_seq, dtype, seq + d)
    f = _inv_freq(d)
    kc_ref, vc_ref = kc.float().numpy().copy(), vc.float().numpy().copy()
    q_ref = oracle.qk_norm_rope_kv(q.float().numpy(), k.float().numpy(), v.float().numpy(), qw.float().numpy(),
                                   kw.float().numpy(), f.numpy(), kc_ref, vc_ref, 1e-6, pos,
                                   is_f16=dtype == torch.float16)
    dev = [t.cuda() for t in (q, k, v, qw, kw, kc, vc)]
    qd, kd, vd, qwd, kwd, kcd, vcd = dev
    fd = f.cuda()
    qo = torch.empty_like(qd)
    name = b"f16" if dtype == torch.float16 else b"bf16"
    _lib.check(b200.b200tile_qk_norm_rope_kv(name, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), qwd.data_ptr(),
                                             kwd.data_ptr(), fd.data_ptr(), qo.data_ptr(), kcd.data_ptr(),
                                             vcd.data_ptr(), 1e-6, pos, None, seq, qh, kvh, d, max_seq, qh * d,
                                             kvh * d, kvh * d, qh * d, _stream().cuda_stream))
    torch.cuda.synchronize()
    ulp = 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7
    _close(qo.float().cpu().numpy(), q_ref, 2 * ulp)
    _close(kcd.float().cpu().numpy(), kc_ref, 2 * ulp)
    # V rows are copies; rows outside [pos, pos + seq) keep their old contents bit for bit
    assert np.array_equal(vcd.float().cpu().numpy(), vc_ref)
    untouched = np.ones(max_seq, dtype=bool)
    untouched[pos:pos + seq] = False
    assert np.array_equal(kcd.float().cpu().numpy()[:, untouched], kc.float().numpy()[:, untouched])


def test_qk_norm_rope_kv_launchers(b200, oracle):
    """The raw-pointer launchers of the reference: prefill over a token block, then one decode step from a fused
    projection row with the position on the device; both leave the caches as the oracle's."""
    seq, qh, kvh, d, max_seq = 12, 8, 2, 128, 64
    q, k, v, qw, kw, kc, vc = _qk_case(seq, qh, kvh, d, max_seq, torch.float16, 99)
    f = _inv_freq(d)
    kc_ref, vc_ref = kc.float().numpy().copy(), vc.float().numpy().copy()
    q_ref = oracle.qk_norm_rope_kv(q.float().numpy(), k.float().numpy(), v.float().numpy(), qw.float().numpy(),
                                   kw.float().numpy(), f.numpy(), kc_ref, vc_ref, 1e-6, 0)
    t = [api.copy_host_to_device(x) for x in (q, k, v, qw, kw, f, kc, vc)]
    qd, kd, vd, qwd, kwd, fd, kcd, vcd = t
    qo = api.zeros([seq, qh, d], "f16")
    launch.qk_norm_rope_kv_prefill_raw_f16(qd, kd, vd, qwd, kwd, fd, qo, kcd, vcd, 1e-6, 0).sync_on(_stream())
    _close(qo.to_host().float().numpy(), q_ref, 2.0 ** -9)
    # decode: token `seq`, q / k / v taken from one row
    g = torch.Generator().manual_seed(7)
    row = torch.randn((qh + 2 * kvh) * d, generator=g).half()
    q1 = row[:qh * d].reshape(1, qh, d)
    k1 = row[qh * d:(qh + kvh) * d].reshape(1, kvh, d)
    v1 = row[(qh + kvh) * d:].reshape(1, kvh, d)
    q1_ref = oracle.qk_norm_rope_kv(q1.float().numpy(), k1.float().numpy(), v1.float().numpy(), qw.float().numpy(),
                                    kw.float().numpy(), f.numpy(), kc_ref, vc_ref, 1e-6, seq)
    rowd = api.copy_host_to_device(row)
    q1o = api.zeros([qh, d], "f16")
    p = api.from_torch(torch.tensor([seq], dtype=torch.int32, device="cuda"))
    launch.qk_norm_rope_kv_decode_raw_f16(rowd, qwd, kwd, fd, q1o, kcd, vcd, p, 1e-6, qh, kvh).sync_on(_stream())
    _close(q1o.to_host().float().numpy().reshape(1, qh, d), q1_ref, 2.0 ** -9)
    _close(kcd.to_host().float().numpy(), kc_ref, 2.0 ** -9)
    assert np.array_equal(vcd.to_host().float().numpy(), vc_ref)
    # a block that does not fit the cache is refused on the host
    with pytest.raises(Exception, match="do not fit"):
        launch.qk_norm_rope_kv_prefill_raw_f16(qd, kd, vd, qwd, kwd, fd, qo, kcd, vcd, 1e-6, max_seq - 3) \
            .sync_on(_stream())
