"""Split-KV GQA decode attention parity on a B200 against the oracle's tile-by-tile restatement."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from cutile_rs_b200 import api, launch  # noqa: E402

ATTN_TOL = 2e-2


def _setup(heads, group, d, cap, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(heads, group, d, generator=g).to(dtype)
    k = torch.randn(heads, cap, d, generator=g).to(dtype)
    v = torch.randn(heads, cap, d, generator=g).to(dtype)
    return q, k, v


def _run(q, k, v, pos, bn, splits, merge=True):
    heads, group, d = q.shape
    name = "bf16" if q.dtype == torch.bfloat16 else "f16"
    att = api.from_torch(torch.full((heads, splits * group, d), float("nan"), dtype=q.dtype, device="cuda"))
    lse = api.from_torch(torch.full((heads, splits * group), float("nan"), dtype=torch.float32, device="cuda"))
    out = api.zeros([heads, group, d], name) if merge else None
    p = api.from_torch(torch.tensor([pos], dtype=torch.int32, device="cuda"))
    launch.decode_attention(api.copy_host_to_device(q), api.copy_host_to_device(k), api.copy_host_to_device(v),
                                 att, lse, p, 1.0 / math.sqrt(d), bn, splits, out=out)
    torch.cuda.synchronize()
    return att.storage, lse.storage, (out.storage if merge else None)


@pytest.mark.parametrize("heads,group,d,cap,pos,bn,splits,dtype", [
    (2, 4, 128, 512, 511, 64, 4, torch.bfloat16),
    (2, 4, 128, 512, 300, 64, 4, torch.bfloat16),     # last tile masked, last split short
    (3, 8, 64, 1000, 700, 128, 8, torch.float16),
    (1, 1, 128, 256, 40, 64, 8, torch.bfloat16),      # most splits empty
    (2, 5, 128, 777, 776, 32, 3, torch.bfloat16),     # odd group, ragged cache
    (8, 4, 128, 4096, 4095, 128, 16, torch.bfloat16),
])
def test_split_and_merge_match_oracle(b200, oracle, heads, group, d, cap, pos, bn, splits, dtype):
    q, k, v = _setup(heads, group, d, cap, dtype, seed=cap + pos)
    att, lse, out = _run(q, k, v, pos, bn, splits)
    is_f16 = dtype == torch.float16
    att_o, lse_o = oracle.fmha_decode_gqa_split(q.float().numpy(), k.float().numpy(), v.float().numpy(), pos + 1, bn,
                                                splits, 1.0 / math.sqrt(d), is_f16)
    out_o = oracle.splitk_reduce_merge(att_o, lse_o, group, is_f16)
    assert not torch.isnan(att.float()).any() and not torch.isnan(lse).any()
    assert oracle.max_abs(att.float().cpu().numpy(), att_o) <= ATTN_TOL
    lse_g = lse.cpu().numpy()
    live = lse_o > -1e29
    assert np.array_equal(lse_g > -1e29, live)                     # same splits are empty
    assert np.max(np.abs(lse_g[live] - lse_o[live])) <= 1e-2        # log2-domain log-sum-exp
    assert oracle.max_abs(out.float().cpu().numpy(), out_o) <= ATTN_TOL
    # and against plain softmax attention over the visible keys
    sc = torch.einsum("hgd,hnd->hgn", q.float(), k.float()[:, :pos + 1]) / math.sqrt(d)
    dense = torch.einsum("hgn,hnd->hgd", torch.softmax(sc, -1), v.float()[:, :pos + 1])
    assert (out.float().cpu() - dense).abs().max().item() <= ATTN_TOL


def test_merge_alone_and_position_is_read_on_device(b200, oracle):
    heads, group, d, cap, bn, splits = 2, 4, 128, 1024, 64, 4
    q, k, v = _setup(heads, group, d, cap, torch.bfloat16, seed=5)
    att, lse, _ = _run(q, k, v, 600, bn, splits, merge=False)
    out = api.zeros([heads, group, d], "bf16")
    launch.decode_merge(api.from_torch(att), api.from_torch(lse), out, splits)
    torch.cuda.synchronize()
    ref = oracle.splitk_reduce_merge(att.float().cpu().numpy(), lse.cpu().numpy(), group, False)
    assert oracle.max_abs(out.storage.float().cpu().numpy(), ref) <= 2.0 ** -7
    # a captured graph follows the device-side position from replay to replay
    qd, kd, vd = (api.copy_host_to_device(t) for t in (q, k, v))
    att_t = api.zeros([heads, splits * group, d], "bf16")
    lse_t = api.from_torch(torch.zeros(heads, splits * group, device="cuda"))
    out_t = api.zeros([heads, group, d], "bf16")
    pos = api.from_torch(torch.tensor([99], dtype=torch.int32, device="cuda"))
    stream = torch.cuda.Stream()
    launch.decode_attention(qd, kd, vd, att_t, lse_t, pos, 1 / math.sqrt(d), bn, splits, out=out_t, stream=stream)
    stream.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        launch.decode_attention(qd, kd, vd, att_t, lse_t, pos, 1 / math.sqrt(d), bn, splits, out=out_t,
                                     stream=torch.cuda.current_stream())
    for p in (99, 600, 1023):
        pos.storage.fill_(p)
        g.replay()
        torch.cuda.synchronize()
        sc = torch.einsum("hgd,hnd->hgn", q.float(), k.float()[:, :p + 1]) / math.sqrt(d)
        dense = torch.einsum("hgn,hnd->hgd", torch.softmax(sc, -1), v.float()[:, :p + 1])
        assert (out_t.storage.float().cpu() - dense).abs().max().item() <= ATTN_TOL


def test_reference_shaped_launchers(b200, oracle):
    """The serving kernels under their reference names, parameter order and inferred grids
    (cutile-kernels/src/attention.rs:398-440, 588-613, 738-757, 921-939)."""
    heads_kv, group, d, cap, pos, bn, splits = 2, 4, 128, 640, 500, 64, 5
    q, k, v = _setup(heads_kv, group, d, cap, torch.float16, seed=3)
    qd, kd, vd = (api.copy_host_to_device(t) for t in (q, k, v))
    att = api.zeros([heads_kv, splits * group, d], "f16")
    lse = api.from_torch(torch.zeros(heads_kv, splits * group, device="cuda"))
    out = api.zeros([heads_kv, group, d], "f16")
    p = api.from_torch(torch.tensor([pos], dtype=torch.int32, device="cuda"))
    scale = 1.0 / math.sqrt(d)
    launch.fmha_decode_gqa_split(qd, kd, vd, att.partition([1, group, d]), lse.partition([1, group]), scale, p,
                                 bn=bn).sync()
    launch.splitk_reduce_merge(att, lse, out.partition([1, group, 32])).sync()
    scale16 = float(np.float16(scale))        # the kernel parameter is an f16 scalar
    att_o, lse_o = oracle.fmha_decode_gqa_split(q.float().numpy(), k.float().numpy(), v.float().numpy(), pos + 1, bn,
                                                splits, scale16, True)
    assert oracle.max_abs(att.storage.float().cpu().numpy(), att_o) <= ATTN_TOL
    assert oracle.max_abs(out.storage.float().cpu().numpy(), oracle.splitk_reduce_merge(att_o, lse_o, group, True)) \
        <= ATTN_TOL
    with pytest.raises(Exception, match="grid"):
        launch.fmha_decode_gqa_split(qd, kd, vd, att.partition([1, group, d]), lse.partition([1, group]), scale, p,
                                     bn=bn).grid((heads_kv, splits + 1, 1)).sync()

    # prefill with GROUP query heads per tile-block, and the dynamic-position kernel, [q_len, heads, D]
    q_len, heads = 200, heads_kv * group
    g = torch.Generator().manual_seed(9)
    qp = torch.randn(q_len, heads, d, generator=g).half()
    kp = torch.randn(heads_kv, q_len, d, generator=g).half()   # equal lengths: the reference CPU attention's shape
    vp = torch.randn(heads_kv, q_len, d, generator=g).half()
    qpd, kpd, vpd = (api.copy_host_to_device(t) for t in (qp, kp, vp))
    ref = oracle.fmha_ref_cpu(qp.permute(1, 0, 2)[None].float().numpy(), kp[None].float().numpy(),
                              vp[None].float().numpy(), scale16, input_pos=40, query_group_size=group, causal=True)
    ref = ref.reshape(heads, q_len, d).transpose(1, 0, 2)
    o1 = api.zeros([q_len, heads, d], "f16")
    launch.fmha_prefill_gqa(qpd, kpd, vpd, o1.partition([32, group, d]), scale16, group, q_len,
                            query_start=40).sync()
    assert oracle.max_abs(o1.storage.float().cpu().numpy(), ref) <= ATTN_TOL
    o2 = api.zeros([q_len, heads, d], "f16")
    p40 = api.from_torch(torch.tensor([40], dtype=torch.int32, device="cuda"))
    launch.fmha_causal(qpd, kpd, vpd, o2.partition([128, 1, d]), scale, group, p40).sync()
    assert oracle.max_abs(o2.storage.float().cpu().numpy(), ref) <= ATTN_TOL
