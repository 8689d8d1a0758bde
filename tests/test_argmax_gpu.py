"""Token selection kernels (`b200tile_argmax_blocks`, `b200tile_lm_head_argmax_blocks`,
`b200tile_argmax_reduce_blocks`) against the oracle's restatement of cutile-kernels/src/argmax.rs.  The plain block
argmax is exact (maximum and lowest index).  The fused LM head sums its fp32 products in another order than the
tile program, so its block maxima are compared to fp32 rounding of a K-long sum and the chosen indices must name a
logit that is within that rounding of the block's maximum (and are equal wherever the winner is clear)."""
import numpy as np
import pytest
import torch

from cutile_rs_b200 import _lib, api, launch

pytestmark = pytest.mark.gpu


def _stream():
    return torch.cuda.current_stream()


@pytest.mark.parametrize("length,block,dtype", [(32000, 1024, torch.float16), (50257, 4096, torch.float16),
                                                (1000, 64, torch.bfloat16), (5, 8, torch.float16)])
def test_argmax_blocks_exact(b200, oracle, length, block, dtype):
    g = torch.Generator().manual_seed(length)
    x = torch.randn(length, generator=g).to(dtype)
    x[length // 3] = x.max() + 1          # a clear winner ...
    x[(2 * length) // 3] = x[length // 3]   # ... and a tie: the lower index has to win
    blocks = (length + block - 1) // block
    xd = x.cuda()
    bm = torch.empty(blocks, dtype=torch.float32, device="cuda")
    bi = torch.empty(blocks, dtype=torch.int32, device="cuda")
    name = b"f16" if dtype == torch.float16 else b"bf16"
    _lib.check(b200.b200tile_argmax_blocks(name, xd.data_ptr(), bm.data_ptr(), bi.data_ptr(), length, block,
                                           _stream().cuda_stream))
    out = torch.empty(1, dtype=torch.int32, device="cuda")
    _lib.check(b200.b200tile_argmax_reduce_blocks(bm.data_ptr(), bi.data_ptr(), out.data_ptr(), blocks,
                                                  _stream().cuda_stream))
    torch.cuda.synchronize()
    rm, ri = oracle.argmax_blocks(x.float().numpy(), length, block)
    assert np.array_equal(bm.cpu().numpy(), rm)
    assert np.array_equal(bi.cpu().numpy().astype(np.uint32), ri)
    assert int(out.item()) == oracle.argmax_reduce_blocks(rm, ri, blocks) == length // 3


@pytest.mark.parametrize("vocab,k,dtype,pitch", [(32000, 4096, torch.float16, None), (1000, 512, torch.float16, None),
                                                 (777, 96, torch.bfloat16, None), (130, 40, torch.float16, 44),
                                                 (4096, 8192, torch.float16, 8200)])
def test_lm_head_argmax(b200, oracle, vocab, k, dtype, pitch):
    g = torch.Generator().manual_seed(vocab + k)
    pitch = pitch or k
    w = torch.zeros(vocab, pitch, dtype=dtype)
    w[:, :k] = (torch.randn(vocab, k, generator=g) / k ** 0.5).to(dtype)
    h = torch.randn(k, generator=g).to(dtype)
    winner = (vocab * 5) // 7
    w[winner, :k] = (h.float() * (8.0 / k ** 0.5)).to(dtype)   # a logit (~8 sqrt(k)) far above the rest (~N(0, 1))
    wd, hd = w.cuda(), h.cuda()
    blocks = (vocab + 63) // 64
    bm = torch.empty(blocks, dtype=torch.float32, device="cuda")
    bi = torch.empty(blocks, dtype=torch.int32, device="cuda")
    name = b"f16" if dtype == torch.float16 else b"bf16"
    _lib.check(b200.b200tile_lm_head_argmax_blocks(name, wd.data_ptr(), hd.data_ptr(), bm.data_ptr(), bi.data_ptr(),
                                                   vocab, k, pitch, _stream().cuda_stream))
    out = torch.empty(1, dtype=torch.int32, device="cuda")
    _lib.check(b200.b200tile_argmax_reduce_blocks(bm.data_ptr(), bi.data_ptr(), out.data_ptr(), blocks,
                                                  _stream().cuda_stream))
    torch.cuda.synchronize()
    logits = oracle.lm_head_logits(w[:, :k].float().numpy(), h.float().numpy())
    rm, ri = oracle.argmax_blocks(logits, vocab, 64)
    scale = float(np.abs(w[:, :k].float().numpy()).max() * np.abs(h.float().numpy()).max()) * k
    tol = 4 * np.finfo(np.float32).eps * scale
    got_m, got_i = bm.cpu().numpy(), bi.cpu().numpy().astype(np.int64)
    assert np.all(np.abs(got_m - rm) <= tol)
    assert np.all(np.abs(logits[got_i] - rm) <= 2 * tol)      # the index names a maximum, up to rounding
    clear = np.array([np.sort(logits[b * 64:min((b + 1) * 64, vocab)])[-2:] for b in range(blocks) if
                      min((b + 1) * 64, vocab) - b * 64 >= 2])
    sure = [b for b in range(len(clear)) if clear[b][1] - clear[b][0] > 4 * tol]
    assert np.array_equal(got_i[sure], ri.astype(np.int64)[sure])
    assert int(out.item()) == winner


def test_launchers_and_errors(b200, oracle):
    vocab, k = 2048, 1024
    g = torch.Generator().manual_seed(11)
    w = (torch.randn(vocab, k, generator=g) / 32).half()
    h = torch.randn(1, k, generator=g).half()
    w[1234] = (h[0].float() * 0.05).half()
    wd, hd = api.copy_host_to_device(w), api.copy_host_to_device(h)
    blocks = vocab // 64
    bm = api.zeros([blocks], "f32").partition([1])
    bi = api.from_torch(torch.zeros(blocks, dtype=torch.int32, device="cuda")).partition([1])
    (_w, _h, bm, bi, _n) = launch.lm_head_argmax_blocks_f16(wd, hd, bm, bi, vocab).sync_on(_stream())
    out = api.from_torch(torch.zeros(1, dtype=torch.int32, device="cuda")).partition([1])
    (_a, _b, out, _n) = launch.argmax_reduce_blocks_to_u32(bm.unpartition(), bi.unpartition(), out, blocks) \
        .sync_on(_stream())
    assert int(out.unpartition().to_host().item()) == 1234
    # the unfused pair on materialised logits gives the same token
    logits = (w.float() @ h[0].float()).half()
    ld = api.copy_host_to_device(logits)
    bm2 = api.zeros([2], "f32").partition([1])
    bi2 = api.from_torch(torch.zeros(2, dtype=torch.int32, device="cuda")).partition([1])
    (_l, bm2, bi2, _n) = launch.argmax_blocks_f16(ld, bm2, bi2, vocab, 1024).sync_on(_stream())
    rm, ri = oracle.argmax_blocks(logits.float().numpy(), vocab, 1024)
    assert np.array_equal(bm2.unpartition().to_host().numpy(), rm)
    assert np.array_equal(bi2.unpartition().to_host().numpy().astype(np.uint32), ri)
    s = _stream().cuda_stream
    t = torch.zeros(8, device="cuda")
    assert b200.b200tile_lm_head_argmax_blocks(b"f16", t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 64,
                                               32768, 32768, s) != 0
    assert b"exceeds" in b200.b200tile_last_error()
    assert b200.b200tile_argmax_blocks(b"f32", t.data_ptr(), t.data_ptr(), t.data_ptr(), 8, 8, s) != 0
    assert b200.b200tile_argmax_reduce_blocks(t.data_ptr(), t.data_ptr(), t.data_ptr(), 0, s) != 0
