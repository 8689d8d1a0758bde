"""Execution modes the launch boundary must survive: async streams, CUDA-graph replay, the
autotuner's timed closure."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from cutile_rs_b200 import api, benching, launch, tune, workloads  # noqa: E402


def _ref(oracle, a, b):
    """fp32 CPU oracle GEMM of the 16-bit operands, as a device tensor."""
    return torch.from_numpy(oracle.cpu_gemm(a.float().numpy(), b.float().numpy(), threads=0)).cuda()


def test_async_on_two_streams(b200, oracle):
    a, b = workloads.gemm_bf16_inputs(512, 512, 512)
    x, y = api.copy_host_to_device(a), api.copy_host_to_device(b)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    z1 = api.zeros([512, 512], "bf16").partition([128, 256])
    z2 = api.zeros([512, 512], "bf16").partition([128, 128])
    torch.cuda.synchronize()
    launch.gemm(z1, x, y).async_on(s1)
    launch.gemm(z2, x, y).async_on(s2)
    s1.synchronize()
    s2.synchronize()
    ref = _ref(oracle, a, b)
    for z in (z1, z2):
        assert (z.unpartition().storage.float() - ref).norm() / ref.norm() <= 1e-2


def test_cuda_graph_capture_and_replay(b200, oracle):
    a, b = workloads.gemm_bf16_inputs(512, 512, 512)
    x, y = api.copy_host_to_device(a), api.copy_host_to_device(b)
    z = api.zeros([512, 512], "bf16").partition([128, 256])
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = launch.gemm(z, x, y).graph_on(stream)        # capture: the kernel is recorded, not run
    ref = _ref(oracle, a, b)
    graph.launch().sync()
    torch.cuda.synchronize()
    assert (z.unpartition().storage.float() - ref).norm() / ref.norm() <= 1e-2
    # refresh the input in place (graph.update(memcpy) in the reference) and replay
    x.storage.mul_(2)
    graph.launch().sync()
    torch.cuda.synchronize()
    assert (z.unpartition().storage.float() - 2 * ref).norm() / (2 * ref).norm() <= 1e-2
    out = graph.take_output()
    assert out[0] is z


def test_do_bench_and_autotuner_on_device(b200, oracle, tmp_path):
    a, b = workloads.gemm_bf16_inputs(1024, 1024, 1024)
    x, y = api.copy_host_to_device(a), api.copy_host_to_device(b)
    ref = _ref(oracle, a, b)
    stream = torch.cuda.current_stream()

    def setup(s, config):
        z = api.zeros([1024, 1024], "bf16").partition([config.int("BM"), config.int("BN")])
        op = launch.gemm(z, x, y)
        op.sync_on(s)                                    # correctness gate
        if (z.unpartition().storage.float() - ref).norm() / ref.norm() > 1e-2:
            raise RuntimeError("gate failed")
        return lambda st: launch.gemm(z, x, y).async_on(st)

    configs = tune.library_configs("gemm", "bf16") + [tune.Config({"id": 99, "BM": 64, "BN": 64, "BK": 64})]
    opts = benching.BenchOptions(warmup_ms=5, rep_ms=20, min_reps=3, max_reps=50)
    out = tune.Autotuner("gemm_bf16_1024").configs(configs).bench(opts).log(tmp_path / "t.jsonl").run(stream, setup)
    assert out.best is not None and out.best.int("BM") == 128
    invalid = [t for t in out.trials if "Invalid" in t.state]
    assert len(invalid) == 1 and "no precompiled configuration" in invalid[0].state["Invalid"]["reason"]
    m = benching.do_bench(stream, opts, setup(stream, configs[0]))
    assert m.reps() >= 3 and 0 < m.median_ms() < 50
