"""The N-split GEMM, the (batch x head)-split attention and both NCCL gathers on two GPUs of one box (skipped on a
single-GPU box): every rank runs the real kernels on its shard, the replicated result is compared with the oracle."""
import math
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    import ctypes
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from cutile_rs_b200 import _lib, api, sharding, workloads
        from oracle import oracle
        lib = _lib.load()
        _lib.check(lib.b200tile_init(rank))
        stream = torch.cuda.current_stream()
        m, n, k = 512, 1024, 384
        a, b = workloads.gemm_bf16_inputs(m, n, k, config_index=60)        # identical on every rank (seeded)
        b_r = sharding.shard_columns(b, world, rank, align=256).cuda()
        a_d = a.cuda()
        c_r = torch.full((m, b_r.shape[1]), float("nan"), dtype=torch.bfloat16, device="cuda")
        _lib.check(lib.b200tile_gemm(b"bf16", 0, a_d.data_ptr(), b_r.data_ptr(), c_r.data_ptr(), 1, m, b_r.shape[1], k,
                                     k, b_r.shape[1], b_r.shape[1], 0, 0, 0, 0, -1, 0, 0, stream.cuda_stream))
        c = sharding.all_gather_columns(c_r)
        ref = oracle.cpu_gemm(a.float().numpy(), b.float().numpy(), threads=0)
        ok1 = c.shape == (m, n) and oracle.rel_frobenius(c.float().cpu().numpy(), ref) <= 1e-2

        # host operands: each rank uploads M / world rows of A, NVLink completes A, C columns come back
        op = sharding.ShardedHostGemm(m, b_r.shape[1], k)
        r0, r1 = op.rows
        c_host = torch.full((m, b_r.shape[1]), float("nan"), dtype=torch.bfloat16).pin_memory()
        op(a[r0:r1].contiguous().pin_memory(), b_r.cpu().pin_memory(), c_host)
        torch.cuda.synchronize()
        ok2 = torch.equal(c_host, c_r.cpu())

        # attention: (batch x head) problems split over the ranks, outputs gathered
        bq, h, s, d = 1, 4, 256, 128
        qh, kh, vh = workloads.fmha_inputs(bq, h, s, d, config_index=61)
        sl = lambda t: sharding.shard_problems(t.reshape(bq * h, s, d), world, rank).contiguous().cuda()
        q_r, k_r, v_r = sl(qh), sl(kh), sl(vh)
        o_r = torch.full_like(q_r, float("nan"))
        I2 = ctypes.c_int64 * 2
        _lib.check(lib.b200tile_fmha_fwd(b"bf16", q_r.data_ptr(), k_r.data_ptr(), v_r.data_ptr(), o_r.data_ptr(), 1,
                                         q_r.shape[0], q_r.shape[0], s, s, d, I2(s * d, d), I2(s * d, d), I2(s * d, d),
                                         I2(s * d, d), 1.0 / math.sqrt(d), 1, 0, stream.cuda_stream))
        o = sharding.all_gather_problems(o_r)
        oref = oracle.fmha_ref_cpu(qh.float().numpy(), kh.float().numpy(), vh.float().numpy(), 1.0 / math.sqrt(d),
                                   causal=True, threads=0).reshape(bq * h, s, d)
        ok3 = o.shape == (bq * h, s, d) and float(np.max(np.abs(o.float().cpu().numpy() - oref))) <= 2e-2
        st = _lib.StatusC()
        _lib.check(lib.b200tile_status(stream.cuda_stream, ctypes.byref(st)))
        t = sharding.max_over_ranks(1.0 + rank, torch.device("cuda", rank))
        q.put((rank, bool(ok1), bool(ok2), bool(ok3), st.code, t))
    finally:
        dist.destroy_process_group()


def test_two_ranks_split_run_and_gather(b200):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, ok1, ok2, ok3, code, t in res:
        assert ok1, f"rank {rank}: gathered GEMM differs from the oracle"
        assert ok2, f"rank {rank}: host-operand GEMM differs from the device-operand one"
        assert ok3, f"rank {rank}: gathered attention differs from the oracle"
        assert code == 0 and t == 2.0
