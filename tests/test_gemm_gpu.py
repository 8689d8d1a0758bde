"""GEMM parity on a B200: the CUDA path, called through the C ABI, against the CPU oracle."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from cutile_rs_b200 import _lib, api, launch, workloads  # noqa: E402
from cutile_rs_b200.tensor import KernelLaunchError  # noqa: E402

BF16_TOL = 1e-2   # relative Frobenius error, bf16 (and f16) against the fp32 oracle


def _stream():
    return torch.cuda.current_stream()


def _status_ok(lib):
    st = _lib.StatusC()
    _lib.check(lib.b200tile_status(_stream().cuda_stream, ctypes.byref(st)))
    assert st.code == 0


def _gemm(lib, dtype, a, b, layout=0, config=-1, accumulate=0, c=None, num_programs=0, group_m=0):
    m, k = a.shape
    n = b.shape[0] if layout else b.shape[1]
    if c is None:
        c = torch.full((m, n), float("nan"), dtype=a.dtype, device="cuda")
    _lib.check(lib.b200tile_gemm(dtype.encode(), layout, a.data_ptr(), b.data_ptr(), c.data_ptr(), 1, m, n, k,
                                 a.stride(0), b.stride(0), c.stride(0), 0, 0, 0, accumulate, config, group_m,
                                 num_programs, _stream().cuda_stream))
    torch.cuda.synchronize()
    return c


def test_f32_config0_is_bit_identical_to_oracle(b200, oracle):
    # the reference's CPU-runnable GEMM: f32 512^3, U[-1,1]
    a, b = workloads.gemm_f32_inputs(512, 512, 512)
    got = _gemm(b200, "f32", a.cuda(), b.cuda()).cpu().numpy()
    ref = oracle.cpu_gemm(a.numpy(), b.numpy(), threads=0)
    assert np.array_equal(got, ref)
    _status_ok(b200)


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (100, 77, 33), (64, 64, 32), (130, 65, 257)])
def test_f32_ragged_shapes_bit_identical(b200, oracle, m, n, k):
    a, b = workloads.gemm_f32_inputs(m, n, k, config_index=10 + m)
    got = _gemm(b200, "f32", a.cuda(), b.cuda()).cpu().numpy()
    assert np.array_equal(got, oracle.cpu_gemm(a.numpy(), b.numpy()))


def test_f32_known_answers(b200, oracle):
    # ones x ones == K (cutile/tests/gpu/book_snippets.rs:165-191)
    ones = torch.ones(64, 64, device="cuda")
    assert torch.all((_gemm(b200, "f32", ones, ones) - 64.0).abs() < 1e-3)
    # patterned persistent example (cutile-examples/examples/persistent_gemm.rs:89-94), through the
    # reference-shaped launcher: 64x64x32, tiles (16,16,8), map [4,1], 4 tile blocks
    x = torch.tensor([[((r % 7) - 3.0) * 0.25 + (c % 5) * 0.125 for c in range(32)] for r in range(64)])
    y = torch.tensor([[((r % 3) + 1.0) * 0.2 - (c % 11) * 0.05 for c in range(64)] for r in range(32)])
    z = api.zeros([64, 64]).partition([16, 16]).map([4, 1], 4)
    (z, _, _) = launch.gemm_persistent(z, api.copy_host_to_device(x), api.copy_host_to_device(y)) \
        .generics(["f32", "16", "16", "8", "4", "1"]).sync_on(_stream())
    got = z.unpartition().to_host().numpy()
    ref = oracle.cpu_gemm(x.numpy(), y.numpy())
    assert np.max(np.abs(got - ref)) < 1e-3 and np.array_equal(got, ref)


def test_f32_accumulate_and_batch(b200, oracle):
    a, b = workloads.gemm_f32_inputs(96, 80, 48, config_index=21)
    c0 = torch.rand(96, 80)
    got = _gemm(b200, "f32", a.cuda(), b.cuda(), accumulate=1, c=c0.clone().cuda()).cpu().numpy()
    # accumulator starts from z (cutile-examples/examples/gemm.rs:28), then ascending-k sums
    ref = c0.numpy().copy()
    for t in range(48):
        ref = (ref + (a.numpy()[:, t:t + 1] * b.numpy()[t:t + 1, :]).astype(np.float32)).astype(np.float32)
    assert np.array_equal(got, ref)
    # batch_matmul: 4 x 128 x 256 x 64, tiles (64,64,32) (cutile-examples/examples/batch_matmul.rs:52-54)
    g = torch.Generator().manual_seed(5)
    xa, yb = torch.rand(4, 128, 64, generator=g), torch.rand(4, 64, 256, generator=g)
    z = api.zeros([4, 128, 256]).partition([1, 64, 64])
    (z, _, _) = launch.batch_matmul(z, api.copy_host_to_device(xa), api.copy_host_to_device(yb)) \
        .generics(["f32", "64", "64", "32"]).sync_on(_stream())
    got = z.unpartition().to_host().numpy()
    for i in range(4):
        assert np.array_equal(got[i], oracle.cpu_gemm(xa[i].numpy(), yb[i].numpy()))


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("config", [0, 1, 2])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 128), (1024, 768, 512), (200, 328, 136)])
def test_bf16_matches_oracle(b200, oracle, layout, config, m, n, k):
    a, b = workloads.gemm_bf16_inputs(m, n, k)
    bd = b.t().contiguous() if layout else b
    got = _gemm(b200, "bf16", a.cuda(), bd.cuda(), layout=layout, config=config).float().cpu().numpy()
    ref = oracle.cpu_gemm(a.float().numpy(), b.float().numpy(), threads=0)
    assert not np.isnan(got).any()
    assert oracle.rel_frobenius(got, ref) <= BF16_TOL
    # stronger than the contract: each output is the bf16 rounding of a near-exact fp32 sum
    assert np.max(np.abs(got - ref)) <= 2.0 ** -7 * np.max(np.abs(ref)) + 1e-6
    _status_ok(b200)


def test_f16_and_known_answer(b200, oracle):
    g = torch.Generator().manual_seed(3)
    a = (torch.randn(256, 192, generator=g) / 14).half()
    b = (torch.randn(192, 384, generator=g) / 14).half()
    got = _gemm(b200, "f16", a.cuda(), b.cuda()).float().cpu().numpy()
    assert oracle.rel_frobenius(got, oracle.cpu_gemm(a.float().numpy(), b.float().numpy(), threads=0)) <= BF16_TOL
    # all-ones f16: every element equals K (sampled +-0.5 in the reference harness, main.rs:977-1024)
    ones_a = torch.ones(256, 1024, dtype=torch.float16, device="cuda")
    ones_b = torch.ones(1024, 256, dtype=torch.float16, device="cuda")
    assert torch.all(_gemm(b200, "f16", ones_a, ones_b) == 1024.0)
    ones = torch.ones(512, 512, dtype=torch.bfloat16, device="cuda")
    assert torch.all(_gemm(b200, "bf16", ones, ones) == 512.0)


def test_bf16_full_size_slab_and_properties(b200, oracle):
    # the headline bf16 workload at full size: 8192^3; the oracle checks a 16-row slab, properties the rest
    m = n = k = 8192
    a, b = workloads.gemm_bf16_inputs(m, n, k)
    ad, bd = a.cuda(), b.cuda()
    c = _gemm(b200, "bf16", ad, bd, config=0)
    rows = slice(4096 - 8, 4096 + 8)
    ref = oracle.cpu_gemm(a[rows].float().numpy(), b.float().numpy(), threads=0)
    assert oracle.rel_frobenius(c[rows].float().cpu().numpy(), ref) <= BF16_TOL
    # scaling A by 2 is exact in bf16 -> C doubles bit-exactly (linearity)
    c2 = _gemm(b200, "bf16", ad * 2, bd, config=0)
    assert torch.equal(c2, c * 2)
    # determinism and independence from the persistent grid size / tile order
    c3 = _gemm(b200, "bf16", ad, bd, config=0, num_programs=37, group_m=3)
    assert torch.equal(c3, c)
    # different tile shapes (and the CTA-pair kernel) add the same k-slabs in the same order
    for cfg in (1, 2, 3):
        assert torch.equal(_gemm(b200, "bf16", ad, bd, config=cfg), c)
    # checksum of checksums against the fp64 column/row sums: sum(C) = (1^T A)(B 1)
    lhs = c.double().sum().item()
    rhs = (ad.double().sum(0) @ bd.double().sum(1)).item()
    assert abs(lhs - rhs) <= 2e-3 * (ad.double().abs().sum(0) @ bd.double().abs().sum(1)).item() ** 0.5 + 1.0
    _status_ok(b200)


def test_reference_shaped_launcher_and_errors(b200, oracle):
    a, b = workloads.gemm_bf16_inputs(512, 512, 256)
    x, y = api.copy_host_to_device(a), api.copy_host_to_device(b)
    z = api.zeros([512, 512], "bf16").partition([128, 256])
    (z, x2, y2, _k) = launch.gemm(z, x, y, k=256).sync_on(_stream())      # generics inferred
    assert x2 is x and y2 is y
    ref = oracle.cpu_gemm(a.float().numpy(), b.float().numpy(), threads=0)
    assert oracle.rel_frobenius(z.unpartition().to_host().float().numpy(), ref) <= BF16_TOL
    # explicit grid that disagrees with the partition is a launch error
    with pytest.raises(KernelLaunchError, match="does not match the inferred partition grid"):
        launch.gemm(api.zeros([512, 512], "bf16").partition([128, 256]), x, y).grid((3, 2, 1)).sync_on(_stream())
    # a tile shape outside the fixed table is reported, not crashed on (TrialState::Invalid path)
    with pytest.raises(KernelLaunchError, match="no precompiled configuration"):
        launch.gemm(api.zeros([512, 512], "bf16").partition([64, 64]), x, y).sync_on(_stream())
    with pytest.raises(KernelLaunchError, match="num_cta_in_cga"):
        launch.gemm(api.zeros([512, 512], "bf16").partition([128, 256]), x, y) \
            .compile_options(launch.CompileOptions(num_cta_in_cga=4)).sync_on(_stream())
    # the reference's published configuration: 256x256x64 tiles on CTA pairs
    zp = api.zeros([512, 512], "bf16").partition([256, 256])
    launch.gemm(zp, x, y).compile_options(launch.CompileOptions(num_cta_in_cga=2)).sync_on(_stream())
    assert oracle.rel_frobenius(zp.unpartition().to_host().float().numpy(), ref) <= BF16_TOL
    # TMA's 16-byte rule: an odd leading dimension is refused with a clear code
    bad = torch.zeros(512, 513, dtype=torch.bfloat16, device="cuda")[:, :512]
    rc = b200.b200tile_gemm(b"bf16", 0, x.cu_deviceptr(), y.cu_deviceptr(), bad.data_ptr(), 1, 512, 512, 256,
                            256, 512, 513, 0, 0, 0, 0, 0, 0, 0, _stream().cuda_stream)
    assert rc == _lib.ERR_ALIGN
    launch.gemm(api.zeros([512, 512], "bf16").partition([128, 256]), x, y).compile()   # warm-up only


def test_streamk_remainder_wave(b200, oracle):
    # 8192 x 1024 (the 8-GPU N-split shard) is 128 tiles on 74 CTA pairs: the 54 tiles of the partial
    # second wave are split along K over all pairs and fixed up through global scratch
    m, n, k = 8192, 1024, 2048
    a, b = workloads.gemm_bf16_inputs(m, n, k, config_index=31)
    ad, bd = a.cuda(), b.cuda()
    c_sk = _gemm(b200, "bf16", ad, bd, config=2)
    c_sk2 = _gemm(b200, "bf16", ad, bd, config=2)
    assert torch.equal(c_sk, c_sk2)                                   # deterministic fix-up order
    c_whole = _gemm(b200, "bf16", ad, bd, config=2, num_programs=148)   # explicit grid: whole tiles only
    ref = oracle.cpu_gemm(a[:64].float().numpy(), b.float().numpy(), threads=0)
    assert oracle.rel_frobenius(c_sk[:64].float().cpu().numpy(), ref) <= BF16_TOL
    # split-K partial sums differ from one long sum only by fp32 rounding: at most one bf16 ulp apart
    diff = (c_sk.float() - c_whole.float()).abs().max().item()
    assert diff <= 2.0 ** -7 * c_whole.float().abs().max().item()
    assert not torch.isnan(c_sk.float()).any()
    _status_ok(b200)


def test_streamk_launch_replays_from_a_graph(b200, oracle):
    """A stream-K launch captured after eager launches on the same stream: every replay must do its own
    hand-off (nothing of the hand-off lives on the host), with inputs that change between replays."""
    m, n, k = 8192, 1024, 2048
    a, b = workloads.gemm_bf16_inputs(m, n, k, config_index=33)
    ad, bd = a.cuda(), b.cuda()
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.Stream()
    rows = slice(4096 - 16, 4096 + 16)
    bf = b.float().numpy()

    def launch_on(s):
        _lib.check(b200.b200tile_gemm(b"bf16", 0, ad.data_ptr(), bd.data_ptr(), c.data_ptr(), 1, m, n, k,
                                      ad.stride(0), bd.stride(0), c.stride(0), 0, 0, 0, 0, 2, 0, 0, s.cuda_stream))
    torch.cuda.synchronize()
    for _ in range(2):                      # eager warm-up: the stream's scratch exists before the capture
        launch_on(stream)
    stream.synchronize()
    eager = c.clone()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        launch_on(torch.cuda.current_stream())
    for rep, scale in enumerate((1.0, 0.5, -2.0, 0.25)):
        ad.copy_((a.float() * scale).to(torch.bfloat16))      # exact scalings: the result scales bit for bit
        c.fill_(float("nan"))
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(c, (eager.float() * scale).to(torch.bfloat16)), f"replay {rep}"
        ref = oracle.cpu_gemm(a[rows].float().numpy() * scale, bf, threads=0)
        assert oracle.rel_frobenius(c[rows].float().cpu().numpy(), ref) <= BF16_TOL
    _status_ok(b200)


@pytest.mark.parametrize("dtype,m,n,k,layout,slab", [("bf16", 1300, 512, 768, 0, 256), ("bf16", 1024, 768, 512, 1, 0),
                                                      ("f32", 300, 256, 128, 0, 256)])
def test_host_operand_pipeline(b200, oracle, dtype, m, n, k, layout, slab):
    """Upload / multiply / download pipeline over host operands: same result as the device-resident
    call (bit for bit: the slabs run the same kernel on the same rows), twice in a row on one stream."""
    td = torch.float32 if dtype == "f32" else torch.bfloat16
    g = torch.Generator().manual_seed(m + n)
    a = (torch.randn(m, k, generator=g) / 8).to(td).pin_memory()
    b = (torch.randn((n, k) if layout else (k, n), generator=g) / 8).to(td).pin_memory()
    c = torch.full((m, n), float("nan"), dtype=td).pin_memory()
    plan = api.HostGemm(m, n, k, dtype, layout, slab)
    stream = torch.cuda.current_stream()
    plan(a, b, c, stream)
    stream.synchronize()
    first = c.clone()
    a2 = (a.float() * 0.5).to(td).pin_memory()
    plan(a2, b, c, stream)         # staging buffers reused while nothing of the first call is pending
    stream.synchronize()
    bm = b.float().t() if layout else b.float()
    if dtype == "f32":
        ref = oracle.cpu_gemm(a.numpy(), b.numpy())
        assert np.array_equal(first.numpy(), ref)
    else:
        ref = oracle.cpu_gemm(a.float().numpy(), bm.contiguous().numpy(), threads=0)
        assert oracle.rel_frobenius(first.float().numpy(), ref) <= 1e-2
        assert oracle.rel_frobenius(c.float().numpy(), 0.5 * ref) <= 1e-2
    assert not torch.isnan(c.float()).any()


@pytest.mark.parametrize("dtype,m,inter,k", [(torch.bfloat16, 300, 384, 320), (torch.float16, 128, 200, 256),
                                             (torch.bfloat16, 1024, 1024, 512)])
def test_linear_with_fused_swiglu(b200, oracle, dtype, m, inter, k):
    """silu(x.Wg^T) * (x.Wu^T) from one kernel against the reference's two-step restatement: GEMM
    outputs rounded to the 16-bit type, then `silu_mul_2d_f16` in fp32 (pointwise.rs:63-75)."""
    g = torch.Generator().manual_seed(inter + k)
    x = (torch.randn(m, k, generator=g) / 4).to(dtype)
    w = (torch.randn(2 * inter, k, generator=g) / 4).to(dtype)
    name = "bf16" if dtype == torch.bfloat16 else "f16"
    out = api.from_torch(torch.full((m, inter), float("nan"), dtype=dtype, device="cuda"))
    launch.linear_swiglu(out, api.copy_host_to_device(x), api.copy_host_to_device(w))
    torch.cuda.synchronize()
    is_f16 = dtype == torch.float16
    rnd = (lambda a: a.astype(np.float16).astype(np.float32)) if is_f16 else oracle.round_bf16
    gate = rnd(oracle.cpu_gemm_nt(x.float().numpy(), w[:inter].float().numpy(), threads=0))
    up = rnd(oracle.cpu_gemm_nt(x.float().numpy(), w[inter:].float().numpy(), threads=0))
    ref = oracle.silu_mul(gate, up, is_f16)
    got = out.storage.float().cpu().numpy()
    assert not np.isnan(got).any()
    assert oracle.rel_frobenius(got, ref) <= 1e-2
    # element-wise: one rounding step of the output type plus the effect of a last-bit difference in gate/up
    assert np.max(np.abs(got - ref) / (np.abs(ref) + 1e-2)) <= 0.05


@pytest.mark.parametrize("dtype,m,n,k", [(torch.bfloat16, 300, 392, 320), (torch.float16, 128, 200, 256),
                                         (torch.bfloat16, 2048, 4096, 512)])
def test_linear_with_bias_and_residual_epilogue(b200, oracle, dtype, m, n, k):
    """x . w^T + bias + residual from one kernel.  Against the oracle (fp32 GEMM, bias added in fp32, rounded to the
    16-bit type, residual added like `add_2d_f16`, pointwise.rs:20-36), and bit for bit against this library's own
    unfused sequence (NT GEMM into memory, then b200tile_add_2d) when there is no bias."""
    g = torch.Generator().manual_seed(n + k)
    x = (torch.randn(m, k, generator=g) / 4).to(dtype)
    w = (torch.randn(n, k, generator=g) / 4).to(dtype)
    bias = torch.randn(n, generator=g).to(dtype)
    res = torch.randn(m, n, generator=g).to(dtype)
    name = "bf16" if dtype == torch.bfloat16 else "f16"
    is_f16 = dtype == torch.float16
    rnd = (lambda a: a.astype(np.float16).astype(np.float32)) if is_f16 else oracle.round_bf16
    xd, wd, bd, rd = (api.copy_host_to_device(t) for t in (x, w, bias, res))
    acc = oracle.cpu_gemm_nt(x.float().numpy(), w.float().numpy(), threads=0)
    for use_bias, use_res in ((True, True), (True, False), (False, True)):
        out = api.from_torch(torch.full((m, n), float("nan"), dtype=dtype, device="cuda"))
        launch.linear_bias_residual(out, xd, wd, bd if use_bias else None, rd if use_res else None)
        torch.cuda.synchronize()
        ref = rnd(acc + (bias.float().numpy()[None, :] if use_bias else 0.0))
        if use_res:
            ref = rnd(ref + res.float().numpy())
        got = out.storage.float().cpu().numpy()
        assert not np.isnan(got).any()
        assert oracle.rel_frobenius(got, ref) <= 1e-2
        # element-wise: the fp32 sums are formed in another order, which can move a 16-bit rounding by one step
        assert np.max(np.abs(got - ref) / (np.abs(ref) + 1.0)) <= (2.0 ** -9 if is_f16 else 2.0 ** -6)
    # no bias: the same bits as GEMM -> memory -> add_2d
    plain = _gemm(b200, name, xd.storage, wd.storage, layout=1, config=0)   # whole tiles: the same k order per output
    unfused = torch.empty_like(plain)
    _lib.check(b200.b200tile_add_2d(name.encode(), unfused.data_ptr(), plain.data_ptr(), rd.storage.data_ptr(), m, n, n, n,
                                    n, _stream().cuda_stream))
    fused = rd.storage.clone()           # in place: out aliases the residual
    ft = api.from_torch(fused)
    launch.linear_bias_residual(ft, xd, wd, None, ft)
    torch.cuda.synchronize()
    assert torch.equal(fused, unfused)
    _status_ok(b200)


@pytest.mark.parametrize("m,n,k,layout", [(300, 520, 192, 0), (256, 512, 64, 1), (1000, 1104, 320, 1), (4096, 4096, 512, 0)])
def test_wide_pair_tile_matches_oracle_and_the_other_configurations(b200, oracle, m, n, k, layout):
    """The 256 x 512 CTA-pair tile (config 3): ragged edges in both layouts, and a shape whose partial last wave is split
    along K (4096 x 4096: 128 tiles on 74 pairs)."""
    a, b = workloads.gemm_bf16_inputs(m, n, k, config_index=50 + m % 7)
    bd = (b.t().contiguous() if layout else b).cuda()
    ad = a.cuda()
    got = _gemm(b200, "bf16", ad, bd, layout=layout, config=3)
    rows = slice(0, min(m, 48))
    ref = oracle.cpu_gemm(a[rows].float().numpy(), b.float().numpy(), threads=0)
    assert oracle.rel_frobenius(got[rows].float().cpu().numpy(), ref) <= BF16_TOL
    assert not torch.isnan(got.float()).any()
    other = _gemm(b200, "bf16", ad, bd, layout=layout, config=0)
    if (m, n) == (4096, 4096):       # split-K partial sums: one bf16 rounding step at most
        assert (got.float() - other.float()).abs().max().item() <= 2.0 ** -7 * other.float().abs().max().item()
        assert torch.equal(got, _gemm(b200, "bf16", ad, bd, layout=layout, config=3))   # deterministic
    else:
        assert torch.equal(got, other)     # whole tiles add the same k slabs in the same order
    _status_ok(b200)


@pytest.mark.parametrize("layout", [0, 1])
def test_f16_accumulators_config4(b200, oracle, layout):
    """Config 4 accumulates in f16 like the reference's benchmark kernel (cutile-benchmarks/benches/gemm.rs:20-41:
    `mma(tile_x, tile_y, tile_z)` with `tile_z: Tile<T>`).  Integer data whose partial sums all fit f16's 11-bit
    significand make the result independent of the order of accumulation: bit-exact against the oracle."""
    m, n, k = 520, 1304, 512
    # (1) position pattern: C[i, j] = (i % 4 + 1) * (j % 512), every row and column of the tile told apart
    a = torch.zeros((m, k), dtype=torch.float16)
    a[:, 0] = (torch.arange(m) % 4 + 1).to(torch.float16)
    b = torch.zeros((k, n), dtype=torch.float16)
    b[0] = (torch.arange(n) % 512).to(torch.float16)
    bd = (b.t().contiguous() if layout else b).cuda()
    got = _gemm(b200, "f16", a.cuda(), bd, layout=layout, config=4).cpu()
    want = ((torch.arange(m) % 4 + 1)[:, None] * (torch.arange(n) % 512)[None, :]).to(torch.float16)
    assert torch.equal(got, want)
    # (2) random small integers over the whole K: |partial sums| <= 4 * 512 = 2048, all exact in f16
    g = torch.Generator().manual_seed(workloads.SEED_BASE + 77)
    a = torch.randint(-2, 3, (m, k), generator=g).to(torch.float16)
    b = torch.randint(-2, 3, (k, n), generator=g).to(torch.float16)
    bd = (b.t().contiguous() if layout else b).cuda()
    got = _gemm(b200, "f16", a.cuda(), bd, layout=layout, config=4).cpu()
    ref = oracle.cpu_gemm(a.float().numpy(), b.float().numpy(), threads=0)
    assert np.array_equal(got.float().numpy(), ref)
    # (3) normal data: f16 rounding of the running sums stays far inside the 16-bit tolerance
    a, bt = workloads.gemm_normal_inputs(m, n, k, config_index=9)
    a, b = a.to(torch.float16), bt.t().contiguous().to(torch.float16)
    bd = (b.t().contiguous() if layout else b).cuda()
    got = _gemm(b200, "f16", a.cuda(), bd, layout=layout, config=4)
    ref = oracle.cpu_gemm(a[:48].float().numpy(), b.float().numpy(), threads=0)
    assert oracle.rel_frobenius(got[:48].float().cpu().numpy(), ref) <= BF16_TOL
    assert not torch.isnan(got.float()).any()
    # only f16 has them
    with pytest.raises(_lib.B200TileError, match="unknown config 4"):
        _gemm(b200, "bf16", a.bfloat16().cuda(), bd.bfloat16(), layout=layout, config=4)
    cfgs = (_lib.ConfigC * 8)()
    assert b200.b200tile_query_configs(b"gemm", b"f16", cfgs, 8) == 5 and cfgs[4].id == 4
    assert b200.b200tile_query_configs(b"gemm", b"bf16", cfgs, 8) == 4
    _status_ok(b200)
