"""NVFP4 block-scaled GEMM parity on a B200 against the oracle's fp32 dequantised reference."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from cutile_rs_b200 import _lib, api, launch, quant, workloads  # noqa: E402

FP4_TOL = 3e-2   # relative Frobenius error against the fp32 dequantised reference


def _run(xp, yp, xs, ys, m, n, k, out, alpha=1.0, config=-1):
    z = api.from_torch(torch.full((m, n), float("nan"), device="cuda",
                                  dtype=torch.float32 if out == "f32" else torch.bfloat16))
    launch.linear_nvfp4(z, api.from_torch(xp, "f4e2m1fnx2"), api.from_torch(yp, "f4e2m1fnx2"),
                        api.from_torch(xs), api.from_torch(ys), alpha, config=config)
    torch.cuda.synchronize()
    return z.storage


@pytest.mark.parametrize("k", [16 * 4, 128])
def test_reference_known_answers(b200, k):
    # nibble 0x2 (= 1.0) with E4M3 scale 0x38 (= 1.0): every output equals K
    # (cutile/tests/tensor_and_matrix_ops.rs:622-682 with K=16; cutile-examples/examples/nvfp4.rs:104-105,
    # 145-151 with 16 x 16 x 128).  K = 64 is this kernel's smallest K.
    m = n = 16
    one = lambda r, c: torch.full((r, c), 0x22, dtype=torch.uint8, device="cuda")
    sc = lambda r, c: torch.full((r, c), 0x38, dtype=torch.uint8, device="cuda")
    z = _run(one(m, k // 2), one(n, k // 2), sc(m, k // 16), sc(n, k // 16), m, n, k, "f32")
    assert torch.all((z - float(k)).abs() <= 1e-3)


@pytest.mark.parametrize("config", [0, 1, 2])
@pytest.mark.parametrize("m,n,k,out", [(128, 256, 64, "f32"), (256, 384, 512, "f32"), (200, 328, 320, "bf16"),
                                       (16, 512, 1024, "bf16")])
def test_matches_oracle(b200, oracle, config, m, n, k, out):
    a, b = workloads.gemm_normal_inputs(m, n, k, config_index=4)
    xp, xs, ga = quant.quant_nvfp4(a)
    yp, ys, gb = quant.quant_nvfp4(b)
    xp_o, xs_o, ga_o = oracle.quant_nvfp4(a.numpy())     # the torch quantiser must agree bit for bit
    assert np.array_equal(xp.numpy(), xp_o) and np.array_equal(xs.numpy(), xs_o) and abs(ga - ga_o) < 1e-12
    got = _run(xp.cuda(), yp.cuda(), xs.cuda(), ys.cuda(), m, n, k, out, ga * gb, config).float().cpu().numpy()
    ref = oracle.cpu_gemm_nt(oracle.dequant_nvfp4(xp.numpy(), xs.numpy()), oracle.dequant_nvfp4(yp.numpy(), ys.numpy()),
                             alpha=ga * gb, threads=0)
    assert not np.isnan(got).any()
    assert oracle.rel_frobenius(got, ref) <= (FP4_TOL if out == "bf16" else 1e-5)


@pytest.mark.parametrize("m,n,k,out", [(256, 256, 256, "f32"), (300, 520, 320, "f32"), (512, 768, 1024, "f32"),
                                       (1000, 1000, 512, "bf16"), (130, 200, 64, "bf16")])
def test_cta_pair_kernel_matches_oracle(b200, oracle, m, n, k, out):
    """Config 3 (CTA pairs, 256 x 256 tiles): scales that differ per row and per 16-block, ragged edges in M and N
    (a pair whose second CTA has no rows at all included); with an f32 output every product and sum is exact."""
    g = torch.Generator().manual_seed(9 + m)
    xp = torch.randint(0, 256, (m, k // 2), generator=g, dtype=torch.uint8)
    yp = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8)
    xs = (0x30 + torch.randint(0, 24, (m, k // 16), generator=g)).to(torch.uint8)   # 0.5 .. 3.5
    ys = (0x30 + torch.randint(0, 24, (n, k // 16), generator=g)).to(torch.uint8)
    got = _run(xp.cuda(), yp.cuda(), xs.cuda(), ys.cuda(), m, n, k, out, 0.5, config=3).float().cpu().numpy()
    ref = oracle.cpu_gemm_nt(oracle.dequant_nvfp4(xp.numpy(), xs.numpy()), oracle.dequant_nvfp4(yp.numpy(), ys.numpy()),
                             alpha=0.5, threads=0)
    assert not np.isnan(got).any()
    assert oracle.rel_frobenius(got, ref) <= (FP4_TOL if out == "bf16" else 1e-6)
    if out == "f32":
        single = _run(xp.cuda(), yp.cuda(), xs.cuda(), ys.cuda(), m, n, k, out, 0.5, config=1).cpu().numpy()
        assert np.array_equal(got, single)      # same products, same order of accumulation along K
    st = _lib.StatusC()
    _lib.check(b200.b200tile_status(torch.cuda.current_stream().cuda_stream, st))
    assert st.code == 0


def test_scale_placement(b200, oracle):
    # scales that differ per row and per 16-block expose any mistake in the Tensor-Memory scale layout
    m, n, k = 256, 384, 256
    g = torch.Generator().manual_seed(9)
    xp = torch.randint(0, 256, (m, k // 2), generator=g, dtype=torch.uint8)
    yp = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8)
    xs = (0x30 + torch.randint(0, 24, (m, k // 16), generator=g)).to(torch.uint8)   # 0.5 .. 3.5
    ys = (0x30 + torch.randint(0, 24, (n, k // 16), generator=g)).to(torch.uint8)
    got = _run(xp.cuda(), yp.cuda(), xs.cuda(), ys.cuda(), m, n, k, "f32").cpu().numpy()
    ref = oracle.cpu_gemm_nt(oracle.dequant_nvfp4(xp.numpy(), xs.numpy()), oracle.dequant_nvfp4(yp.numpy(), ys.numpy()),
                             threads=0)
    assert oracle.rel_frobenius(got, ref) <= 1e-5


def test_full_size_slabs_and_errors(b200, oracle):
    # the benchmark's NVFP4 workload: M=4096 (and the decode shape M=16), N=14336, K=4096
    n, k = 14336, 4096
    g = torch.Generator(device="cuda").manual_seed(workloads.SEED_BASE + 4)
    b = torch.randn(n, k, device="cuda", generator=g)
    yp, ys, gb = quant.quant_nvfp4(b)
    for m in (4096, 16):
        a = torch.randn(m, k, device="cuda", generator=g)
        xp, xs, ga = quant.quant_nvfp4(a)
        z = _run(xp, yp, xs, ys, m, n, k, "bf16", ga * gb)
        rows = slice(0, 8) if m == 16 else slice(2044, 2052)
        cols = slice(7100, 7228)
        ref = oracle.cpu_gemm_nt(oracle.dequant_nvfp4(xp[rows].cpu().numpy(), xs[rows].cpu().numpy()),
                                 oracle.dequant_nvfp4(yp[cols].cpu().numpy(), ys[cols].cpu().numpy()),
                                 alpha=ga * gb, threads=0)
        assert oracle.rel_frobenius(z[rows, cols].float().cpu().numpy(), ref) <= FP4_TOL
        assert not torch.isnan(z.float()).any()
    lib = b200
    rc = lib.b200tile_linear_nvfp4(xp.data_ptr(), yp.data_ptr(), xs.data_ptr(), ys.data_ptr(), z.data_ptr(), b"bf16",
                                   16, n, k, k // 2, k // 2, n, k // 16, k // 16, 1.0, None, 0, -1, None)
    assert rc == _lib.ERR_INVALID and b"workspace" in lib.b200tile_last_error()
    rc = lib.b200tile_linear_nvfp4(xp.data_ptr(), yp.data_ptr(), xs.data_ptr(), ys.data_ptr(), z.data_ptr(), b"bf16",
                                   16, n, 100, 50, 50, n, 8, 8, 1.0, None, 0, -1, None)
    assert rc == _lib.ERR_INVALID and b"multiple of 64" in lib.b200tile_last_error()


@pytest.mark.parametrize("config,m,n,k", [(0, 16, 512, 1024), (1, 200, 328, 320), (2, 256, 384, 512)])
def test_prepared_weight_scales_give_the_same_bits(b200, config, m, n, k):
    """Weight scales laid out once, then a workspace-free call: bit-identical to the call that lays
    them out itself (same kernel, same scale bytes in Tensor Memory)."""
    a, b = workloads.gemm_normal_inputs(m, n, k, config_index=9)
    xp, xs, ga = quant.quant_nvfp4(a)
    yp, ys, gb = quant.quant_nvfp4(b)
    want = _run(xp.cuda(), yp.cuda(), xs.cuda(), ys.cuda(), m, n, k, "f32", ga * gb, config=config)
    xt, yt = api.from_torch(xp.cuda(), "f4e2m1fnx2"), api.from_torch(yp.cuda(), "f4e2m1fnx2")
    prepared = launch.nvfp4_prepare_weight_scales(api.from_torch(ys.cuda()), n, k, config)
    z = api.from_torch(torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32))
    for _ in range(2):   # the prepared buffer is read-only: a second call gives the same result
        launch.linear_nvfp4_prepared(z, xt, yt, api.from_torch(xs.cuda()), prepared, ga * gb, config)
        torch.cuda.synchronize()
        assert torch.equal(z.storage, want)
    with pytest.raises(Exception, match="config"):
        launch.linear_nvfp4_prepared(z, xt, yt, api.from_torch(xs.cuda()), prepared, ga * gb, config=-1)


@pytest.mark.parametrize("m", [1, 31, 32, 33])
def test_decode_sized_m_never_stores_rows_past_m(b200, oracle, m):
    """M <= 32 takes the short A tile (the tensor core still multiplies 128 rows; those past the tile are bytes of the
    weight tile under zero scales): nothing of them may reach memory.  The output lives inside a larger NaN-filled
    buffer whose rows past M must stay NaN."""
    n, k = 384, 512
    a, b = workloads.gemm_normal_inputs(m, n, k, config_index=12)
    xp, xs, ga = quant.quant_nvfp4(a)
    yp, ys, gb = quant.quant_nvfp4(b)
    big = torch.full((m + 130, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    z = api.from_torch(big[:m])
    launch.linear_nvfp4(z, api.from_torch(xp.cuda(), "f4e2m1fnx2"), api.from_torch(yp.cuda(), "f4e2m1fnx2"),
                        api.from_torch(xs.cuda()), api.from_torch(ys.cuda()), ga * gb)
    torch.cuda.synchronize()
    ref = oracle.cpu_gemm_nt(oracle.dequant_nvfp4(xp.numpy(), xs.numpy()), oracle.dequant_nvfp4(yp.numpy(), ys.numpy()),
                             alpha=ga * gb, threads=0)
    got = big[:m].float().cpu().numpy()
    assert not np.isnan(got).any()
    assert oracle.rel_frobenius(got, ref) <= FP4_TOL
    assert torch.isnan(big[m:]).all()


def test_cta_pair_kernel_back_to_back_calls_share_one_workspace(b200):
    """The pair GEMM is launched behind its scale pre-pass with programmatic stream serialisation and starts while the
    pre-pass drains; only its producer warp waits for it.  Twenty calls in a row on one stream and one workspace, the
    scales changed between calls without any host synchronisation: every result must equal the single-CTA kernel's,
    which would not be the case if a GEMM ever read the previous call's scale blocks."""
    m, n, k = 640, 768, 512
    g = torch.Generator(device="cuda").manual_seed(21)
    xp = torch.randint(0, 256, (m, k // 2), generator=g, dtype=torch.uint8, device="cuda")
    yp = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    need = b200.b200tile_linear_nvfp4_workspace_bytes(m, n, k)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    xs_all = (0x30 + torch.randint(0, 24, (20, m, k // 16), generator=g, device="cuda")).to(torch.uint8)
    ys_all = (0x30 + torch.randint(0, 24, (20, n, k // 16), generator=g, device="cuda")).to(torch.uint8)
    outs = torch.full((20, m, n), float("nan"), device="cuda")
    refs = torch.full((20, m, n), float("nan"), device="cuda")

    def call(cfg, xs, ys, z):
        _lib.check(b200.b200tile_linear_nvfp4(xp.data_ptr(), yp.data_ptr(), xs.data_ptr(), ys.data_ptr(), z.data_ptr(), b"f32",
                                              m, n, k, k // 2, k // 2, n, k // 16, k // 16, 1.0, ws.data_ptr(), need, cfg, s))
    for i in range(20):
        call(3, xs_all[i], ys_all[i], outs[i])
    for i in range(20):
        call(1, xs_all[i], ys_all[i], refs[i])
    torch.cuda.synchronize()
    assert not torch.isnan(outs).any()
    assert torch.equal(outs, refs)


def test_decode_calls_chained_back_to_back_see_their_predecessors_output(b200, oracle):
    """Decode-sized calls on prepared weights start under programmatic stream serialisation: a call fetches its weight
    tiles while its predecessor still runs and must wait for it before it touches the activations.  Here every call's
    activations (packed codes AND scales) are rewritten on the same stream right before it, and every output is written
    twice by two calls in a row; twelve steps deep, eagerly and from a captured graph; each output is compared with the
    oracle for the activations and the alpha the last call should have used."""
    m, n, k, calls = 16, 1024, 2048, 12
    g = torch.Generator().manual_seed(404)
    yp = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8)
    ys = (0x30 + torch.randint(0, 24, (n, k // 16), generator=g)).to(torch.uint8)
    xps = [torch.randint(0, 256, (m, k // 2), generator=g, dtype=torch.uint8) for _ in range(calls)]
    xss = [(0x30 + torch.randint(0, 24, (m, k // 16), generator=g)).to(torch.uint8) for _ in range(calls)]
    yd, ysd = api.from_torch(yp.cuda(), "f4e2m1fnx2"), api.from_torch(ys.cuda())
    prepared = launch.nvfp4_prepare_weight_scales(ysd, n, k, 0)
    xp_all, xs_all = torch.stack(xps).cuda(), torch.stack(xss).cuda()
    xp_cur, xs_cur = torch.zeros_like(xp_all[0]), torch.zeros_like(xs_all[0])
    xd, xsd = api.from_torch(xp_cur, "f4e2m1fnx2"), api.from_torch(xs_cur)
    outs = [torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32) for _ in range(calls)]
    yref = oracle.dequant_nvfp4(yp.numpy(), ys.numpy())
    refs = [oracle.cpu_gemm_nt(oracle.dequant_nvfp4(xps[i].numpy(), xss[i].numpy()), yref, alpha=0.5, threads=0)
            for i in range(calls)]

    def step():
        for i in range(calls):
            xp_cur.copy_(xp_all[i])          # device-to-device copies on the same stream: the predecessor of call i
            xs_cur.copy_(xs_all[i])
            launch.linear_nvfp4_prepared(api.from_torch(outs[i]), xd, yd, xsd, prepared, 0.25, config=0)
            # a second call straight behind the first (it overlaps the first one's tail) into the same output with
            # another alpha: its stores must land after the first call's
            launch.linear_nvfp4_prepared(api.from_torch(outs[i]), xd, yd, xsd, prepared, 0.5, config=0)

    def check():
        torch.cuda.synchronize()
        for i in range(calls):
            got = outs[i].cpu().numpy()
            assert not np.isnan(got).any()
            assert oracle.rel_frobenius(got, refs[i]) <= 1e-6, i
            outs[i].fill_(float("nan"))

    step()
    check()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=s, capture_error_mode="relaxed"):
        step()
    for _ in range(3):
        graph.replay()
        check()
    st = _lib.StatusC()
    _lib.check(b200.b200tile_status(torch.cuda.current_stream().cuda_stream, st))
    assert st.code == 0
