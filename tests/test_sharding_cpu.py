"""N-split / (batch x head)-split sharding and reassembly with two gloo ranks on CPU."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

from cutile_rs_b200 import sharding  # noqa: E402


def test_split_range_alignment_and_cover():
    for total, world, align in [(8192, 8, 256), (28672, 8, 128), (14336, 8, 128), (1000, 3, 8), (256, 7, 1)]:
        spans = [sharding.split_range(total, world, r, align) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(s % align == 0 and e % align == 0 for s, e in spans)
    assert sharding.split_range(28672, 8, 3, 128) == (3 * 3584, 4 * 3584)
    with pytest.raises(ValueError):
        sharding.split_range(100, 4, 4)
    with pytest.raises(ValueError):
        sharding.split_range(100, 4, 0, align=8)


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(7)
        a = torch.randn(32, 24, generator=g)
        b = torch.randn(24, 48, generator=g)
        b_r = sharding.shard_columns(b, world, rank, align=8)
        c_r = a @ b_r                                   # stands in for the per-rank kernel
        c = sharding.all_gather_columns(c_r)
        ok1 = torch.allclose(c, a @ b, atol=1e-5)
        bt_r = sharding.shard_rows(b.t().contiguous(), world, rank, align=8)
        ok2 = torch.equal(bt_r, b_r.t().contiguous())
        o = torch.arange(6 * 4 * 2, dtype=torch.float32).reshape(6, 4, 2)
        o_r = sharding.shard_problems(o, world, rank) * 1.0
        ok3 = torch.equal(sharding.all_gather_problems(o_r), o)
        # row slabs gathered in place into the full activation matrix (the upload path of ShardedHostGemm)
        a_full = torch.full((32, 24), float("nan"))
        r0, r1 = rank * 16, (rank + 1) * 16
        a_full[r0:r1] = a[r0:r1]
        sharding.all_gather_rows(a_full, a_full[r0:r1])
        ok4 = torch.equal(a_full, a)
        # the chunked pipeline of ShardedHostGemm with the kernel and the copies replaced by torch on CPU: chunk j of
        # the rank's rows into its block of the chunk-major matrix, gather in place, multiply, rows back by the map
        chunks, sub = 2, 8
        a_cm = torch.full((chunks, world * sub, 24), float("nan"))
        c_out = torch.full((32, b_r.shape[1]), float("nan"))
        for j in range(chunks):
            a_cm[j, rank * sub:(rank + 1) * sub] = a[r0 + j * sub:r0 + (j + 1) * sub]
            dist.all_gather_into_tensor(a_cm[j], a_cm[j, rank * sub:(rank + 1) * sub].clone())
            c_j = a_cm[j] @ b_r
            for r in range(world):
                g0, g1 = sharding.chunk_block_rows(r, world, 32, chunks, j)
                c_out[g0:g1] = c_j[r * sub:(r + 1) * sub]
        ok5 = torch.allclose(c_out, a @ b_r, atol=1e-5)
        t = sharding.max_over_ranks(1.0 + rank, torch.device("cpu"))
        q.put((rank, bool(ok1 and ok2 and ok3 and ok4 and ok5), t))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_split_and_gather():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in res)
    assert all(t == 2.0 for _, _, t in res)          # MAX over ranks


def test_chunk_block_rows_cover_every_row_once():
    for world, m, chunks in [(1, 256, 2), (2, 512, 2), (4, 8192, 4), (8, 8192, 4)]:
        seen = []
        for j in range(chunks):
            for r in range(world):
                g0, g1 = sharding.chunk_block_rows(r, world, m, chunks, j)
                assert g1 - g0 == m // world // chunks and r * (m // world) <= g0 < g1 <= (r + 1) * (m // world)
                seen.extend(range(g0, g1))
        assert sorted(seen) == list(range(m))
