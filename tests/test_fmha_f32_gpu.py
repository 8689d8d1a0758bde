"""fp32 attention on the GPU: the element type and the shapes of the reference's two ASSERTED attention examples
(cutile-examples/examples/flash_attention.rs:199-264 and flash_attention_causal.rs:216-285), checked with the
examples' own tolerances against the committed golden fixture and the CPU oracle."""
import ctypes
import math
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from cutile_rs_b200 import _lib, api, launch  # noqa: E402

I64x2 = ctypes.c_int64 * 2


def _stream():
    return torch.cuda.current_stream()


def _fmha(lib, q, k, v, scale, causal, input_pos=0, pos_tensor=None):
    b, h, s, d = q.shape
    hkv, skv = k.shape[1], k.shape[2]
    o = torch.full((b * h, s, d), float("nan"), dtype=torch.float32, device="cuda")
    args = (b"f32", q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), b, h, hkv, s, skv, d, I64x2(s * d, d),
            I64x2(skv * d, d), I64x2(skv * d, d), I64x2(s * d, d), scale, int(causal))
    if pos_tensor is None:
        _lib.check(lib.b200tile_fmha_fwd(*args, input_pos, _stream().cuda_stream))
    else:
        _lib.check(lib.b200tile_fmha_fwd_dynpos(*args, pos_tensor.data_ptr(), _stream().cuda_stream))
    torch.cuda.synchronize()
    return o


def test_causal_example_against_the_golden_fixture(b200):
    # 2 x 8 x 64 x 32, causal, input_pos = 5; the example accepts |got - exp| <= 2e-3 + 2e-3 |exp|
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "fmha_causal_pos5.npz"))
    q, k, v = (torch.from_numpy(gold[n]).cuda() for n in ("q", "k", "v"))
    got = _fmha(b200, q, k, v, float(gold["scale"]), True, 5).cpu().numpy().reshape(gold["out"].shape)
    exp = gold["out"]
    assert np.all(np.abs(got - exp) <= 2e-3 + 2e-3 * np.abs(exp))
    assert np.max(np.abs(got - exp)) <= 1e-5           # fp32 arithmetic: far inside the example's tolerance
    # the same offset read from device memory at kernel time
    pos = torch.tensor([5], dtype=torch.int32, device="cuda")
    dyn = _fmha(b200, q, k, v, float(gold["scale"]), True, pos_tensor=pos).cpu().numpy().reshape(exp.shape)
    assert np.array_equal(dyn, got)


def test_noncausal_example_shape_against_the_oracle(b200, oracle):
    # flash_attention.rs: f32, heads x 1024 x 64, N(0,1) operands, every |diff| <= 1e-4 (4 of the example's 128
    # (batch, head) pairs, so that the oracle finishes in seconds)
    g = torch.Generator().manual_seed(7)
    b, h, s, d = 1, 4, 1024, 64
    q, k, v = (torch.randn(b, h, s, d, generator=g) for _ in range(3))
    scale = 1.0 / math.sqrt(d)
    got = _fmha(b200, q.cuda(), k.cuda(), v.cuda(), scale, False).cpu().numpy().reshape(b, h, s, d)
    ref = oracle.fmha_ref_cpu(q.numpy(), k.numpy(), v.numpy(), scale, threads=0)
    assert np.max(np.abs(got - ref)) <= 1e-4


@pytest.mark.parametrize("b,h,hkv,s,d,causal,pos", [(2, 4, 2, 300, 128, True, 0), (1, 6, 2, 100, 32, True, 3),
                                                    (1, 2, 2, 129, 64, False, 0), (1, 1, 1, 1, 32, True, 0)])
def test_ragged_gqa_and_head_dims(b200, oracle, b, h, hkv, s, d, causal, pos):
    g = torch.Generator().manual_seed(100 + s)
    q = torch.randn(b, h, s, d, generator=g)
    k, v = torch.randn(b, hkv, s, d, generator=g), torch.randn(b, hkv, s, d, generator=g)
    scale = 1.0 / math.sqrt(d)
    got = _fmha(b200, q.cuda(), k.cuda(), v.cuda(), scale, causal, pos).cpu().numpy().reshape(b, h, s, d)
    ref = oracle.fmha_ref_cpu(q.numpy(), k.numpy(), v.numpy(), scale, input_pos=pos, query_group_size=h // hkv,
                              causal=causal, threads=0)
    assert not np.isnan(got).any()
    assert np.max(np.abs(got - ref)) <= 1e-4


def test_through_the_generated_launcher_with_the_examples_generics(b200):
    # flash_attention_causal.rs:236-258: generics [BM, BN, D, H, CAUSAL, EVEN_K] = [32, 32, 32, 8, 1, 1]
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "fmha_causal_pos5.npz"))
    q, k, v = (api.from_torch(torch.from_numpy(gold[n]).cuda()) for n in ("q", "k", "v"))
    out = api.zeros([16, 64, 32]).partition([1, 32, 32])
    (out, *_r) = launch.fmha(out, q, k, v, float(gold["scale"]), 5, 1, causal=True) \
        .generics(["f32", "32", "32", "32", "8", "1", "1"]).sync_on(_stream())
    got = out.unpartition().to_host().numpy().reshape(gold["out"].shape)
    assert np.max(np.abs(got - gold["out"])) <= 1e-5
    # head_dim 48 has no configuration
    rc = b200.b200tile_fmha_fwd(b"f32", 16, 16, 16, 16, 1, 1, 1, 64, 64, 48, I64x2(3072, 48), I64x2(3072, 48),
                                I64x2(3072, 48), I64x2(3072, 48), 0.1, 0, 0, _stream().cuda_stream)
    assert rc == _lib.ERR_UNSUPPORTED and b"head_dim 48" in b200.b200tile_last_error()
