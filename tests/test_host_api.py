"""Host-side launcher logic: partition grids, mapped partitions, grid inference, tuner (CPU only)."""
import json
import os

import numpy as np
import pytest
import torch

from cutile_rs_b200 import tune
from cutile_rs_b200.benching import BenchOptions, Measurement
from cutile_rs_b200.tensor import (OWNED, GridBound, KernelLaunchError, Partition, Tensor, TensorError,
                                   infer_launch_grid, partition_grid, persistent_num_programs,
                                   validate_grid_bounds, validate_mapped)


def test_partition_grid_is_ceil_div():
    # cutile/src/tensor.rs:428-440 doc examples
    assert partition_grid([256], [64]) == (4, 1, 1)
    assert partition_grid([128, 256], [32, 64]) == (4, 4, 1)
    assert partition_grid([100, 77, 5], [64, 64, 2]) == (2, 2, 3)
    with pytest.raises(TensorError, match="positive"):
        partition_grid([0, 4], [1, 1])
    with pytest.raises(TensorError, match="rank 3"):
        partition_grid([1, 1, 1, 1], [1, 1, 1, 1])


def test_partition_kernel_args_order():
    # ptr, dims, strides, partition dims, partition strides (cutile/src/tensor.rs:1723-1739)
    t = Tensor(torch.zeros(6, 10))
    p = t.partition([2, 5])
    kinds = [k for k, _ in p.kernel_args()]
    vals = [v for _, v in p.kernel_args()]
    assert kinds == ["u64"] + ["i32"] * 8
    assert vals[1:] == [6, 10, 10, 1, 2, 5, 1, 1]
    assert [v for _, v in t.kernel_args()][1:] == [6, 10, 10, 1]
    assert p.grid() == (3, 2, 1) and p.unpartition() is t
    with pytest.raises(TensorError):
        t.partition([2])


@pytest.mark.parametrize("map_shape,grid,n,expect", [
    ([4, 1], (2, 3, 1), 3, (3, 1, 1)),          # swizzle_accepts_tile_block_count
    ([1, OWNED], (2, 3, 1), 2, (2, 1, 1)),      # owned_axis_excluded_from_streamed_tile_count
    ([OWNED, 1], (2, 3, 1), 3, (3, 1, 1)),      # owned_axis_accepts_leading_owned
    ([1], (8, 1, 1), 4, (4, 1, 1)),             # swizzle_accepts_rank1_map
    ([1, 4, 1], (2, 3, 4), 6, (6, 1, 1)),       # swizzle_accepts_rank3_map
])
def test_mapped_partition_accepts(map_shape, grid, n, expect):
    # cutile/src/tensor.rs:2204-2344
    assert validate_mapped(map_shape, grid, n) == expect


@pytest.mark.parametrize("map_shape,grid,n,msg", [
    ([4, 1], (2, 3, 1), 7, "num_tile_blocks cannot exceed the streamed logical tile count"),
    ([1, OWNED], (2, 3, 1), 3, "num_tile_blocks cannot exceed the streamed logical tile count"),
    ([OWNED, OWNED], (2, 3, 1), 1, "at least one streamed (non-OWNED) map axis"),
    ([4, 1], (2, 3, 1), 0, "num_tile_blocks > 0"),
    ([4, 1], (2, 3, 4), 3, "map rank must match the logical partition grid rank"),
    ([1], (2, 3, 1), 2, "map rank must match the logical partition grid rank"),
    ([1, 1, 1, 1], (2, 3, 4), 2, "rank-1 through rank-3 map shape"),
])
def test_mapped_partition_rejects(map_shape, grid, n, msg):
    with pytest.raises(TensorError) as e:
        validate_mapped(map_shape, grid, n)
    assert msg in str(e.value)


def test_grid_bounds_and_inference():
    # cutile/src/tile_kernel.rs:1509-1594
    E, A = GridBound.Exact, GridBound.AtMost
    validate_grid_bounds((4, 1, 1), [E((4, 1, 1))])
    with pytest.raises(KernelLaunchError):
        validate_grid_bounds((4, 1, 1), [E((2, 1, 1))])
    for g in [(3, 2, 1), (2, 2, 1), (2, 1, 1)]:
        validate_grid_bounds(g, [A((3, 2, 1))])
    for g in [(4, 1, 1), (1, 3, 1), (6, 1, 1)]:
        with pytest.raises(KernelLaunchError):
            validate_grid_bounds(g, [A((3, 2, 1))])
    with pytest.raises(KernelLaunchError):
        validate_grid_bounds((2, 1, 1), [E((3, 1, 1)), A((3, 1, 1))])
    validate_grid_bounds((3, 1, 1), [E((3, 1, 1)), A((4, 1, 1))])
    with pytest.raises(KernelLaunchError, match="partial-coverage"):
        infer_launch_grid((0, 0, 0), [A((3, 1, 1))])
    with pytest.raises(KernelLaunchError, match="Launch grid required"):
        infer_launch_grid((0, 0, 0), [])
    assert infer_launch_grid((0, 0, 0), [E((3, 1, 1)), A((4, 1, 1))]) == (3, 1, 1)
    with pytest.raises(KernelLaunchError):
        infer_launch_grid((0, 0, 0), [E((3, 1, 1)), A((2, 1, 1))])
    assert infer_launch_grid((2, 1, 1), [A((3, 1, 1))]) == (2, 1, 1)
    with pytest.raises(KernelLaunchError):
        infer_launch_grid((4, 1, 1), [A((3, 1, 1))])


def test_prefix_partition_cannot_be_mapped_and_persistent_grid():
    t = Tensor(torch.zeros(128, 256))
    with pytest.raises(TensorError, match="cannot be mapped"):
        t.partition_prefix([32, 64]).map([4, 1], 2)
    mp = t.partition([32, 64]).map([4, 1], 8)
    assert mp.grid() == (8, 1, 1) and mp.grid_bound().kind == "exact"
    assert persistent_num_programs(8192, 8192, 256, 256, 148, 2, 1) == 74
    assert persistent_num_programs(64, 64, 16, 16, 148, 1, 1) == 16


# ------------------------------------ tuner -------------------------------------------------
def test_config_id_and_space_hash():
    c = tune.Config({"BN": 256, "BM": 128, "kind": "a,b"})
    assert c.id == 'BM=128,BN=256,kind="a,b"'
    assert tune.Config({"A": 1}).id != tune.Config({"A": "1"}).id
    assert c.int("BM") == 128 and c.str("kind") == "a,b" and c.int("kind") is None
    a, b = tune.Config({"x": 1}), tune.Config({"x": 2})
    assert tune.space_hash([a, b]) == tune.space_hash([b, a])
    assert tune.space_hash([a]) != tune.space_hash([a, b])
    h = 0xCBF29CE484222325   # FNV-1a of b"x=1\0"
    for byte in b"x=1\x00":
        h = ((h ^ byte) * 0x100000001B3) & (2**64 - 1)
    assert tune.space_hash([a]) == f"{h:016x}"


def _fake_bench(times):
    def bench(stream, opts, f):
        f(stream)
        return Measurement([times[f.tag]] * 5)
    return bench


def _fake_paired(times):
    def paired(stream, opts, a, b):
        return Measurement([times[a.tag] * 1.0] * 5), Measurement([times[b.tag] * 1.0] * 5)
    return paired


def _setup_factory(bad=()):
    def setup(stream, config):
        if config.int("id") in bad:
            raise KernelLaunchError(f"config {config.int('id')} has no precompiled configuration")
        def f(s):
            return None
        f.tag = config.int("id")
        return f
    return setup


def test_autotuner_search_invalid_and_runoff(tmp_path):
    configs = [tune.Config({"id": i}) for i in range(4)]
    times = {0: 3.0, 1: 1.0, 2: 1.1, 3: 9.0}
    t = tune.Autotuner("gemm").configs(configs).prune(lambda c: c.int("id") != 3).log(tmp_path / "log.jsonl")
    t._bench_fn, t._paired_fn = _fake_bench(times), _fake_paired({0: 3.0, 1: 1.2, 2: 1.0})
    out = t.run(None, _setup_factory(bad=(0,)))
    states = {tr.config_id: tr.state for tr in out.trials[:3]}
    assert "Invalid" in states["id=0"] and "no precompiled" in states["id=0"]["Invalid"]["reason"]
    assert states["id=1"]["Measured"]["median_ms"] == 1.0
    assert out.best.id == "id=2"          # the paired runoff, not the sequential medians, decides
    lines = (tmp_path / "log.jsonl").read_text().splitlines()
    assert json.loads(lines[0]) == {"log_schema": 1, "tuner": "gemm", "space": tune.space_hash(configs[:3])}
    assert len(lines) == 1 + 3 + 2        # header, three visits, two runoff records

    # resume: measured candidates are not re-measured, the Invalid one is retried
    calls = []
    def setup2(stream, config):
        calls.append(config.id)
        return _setup_factory()(stream, config)
    t2 = tune.Autotuner("gemm").configs(configs[:3]).log(tmp_path / "log.jsonl")
    t2._bench_fn, t2._paired_fn = _fake_bench({0: 0.5, 1: 1.0, 2: 1.1}), _fake_paired({0: 0.5, 1: 1.0, 2: 1.1})
    out2 = t2.run(None, setup2)
    assert calls[0] == "id=0" and out2.best.id == "id=0"

    # a log that belongs to another tuner or another space is refused
    with pytest.raises(ValueError, match="belongs to tuner"):
        tune.Autotuner("fmha").configs(configs[:3]).log(tmp_path / "log.jsonl").run(None, _setup_factory())
    with pytest.raises(ValueError, match="belongs to tuner"):
        tune.Autotuner("gemm").configs(configs[:2]).log(tmp_path / "log.jsonl").run(None, _setup_factory())
    (tmp_path / "junk.jsonl").write_text("not json\n")
    with pytest.raises(ValueError, match="no valid header"):
        tune.Autotuner("gemm").configs(configs).log(tmp_path / "junk.jsonl").run(None, _setup_factory())


def test_autotuner_budget_and_best_config():
    configs = [tune.Config({"id": i}) for i in range(3)]
    t = tune.Autotuner("k").configs(configs).budget(0.0)
    t._bench_fn = _fake_bench({0: 1.0, 1: 2.0, 2: 3.0})
    out = t.run(None, _setup_factory())
    assert out.trials == [] and out.best is None          # exhausted budget: nothing visited
    trials = [tune.Trial.measured("id=1", Measurement([2.0])), tune.Trial.invalid("id=0", "x"),
              tune.Trial.measured("gone", Measurement([0.1])), tune.Trial.measured("id=2", Measurement([1.5]))]
    assert tune.best_config(configs, trials).id == "id=2"  # a stale record cannot win
    assert tune.best_config(configs, []) is None
    gs = tune.GridSearch().resume(trials)
    class O:
        def configs(self): return configs
        def budget_remaining(self): return None
        def measure(self, i): return tune.Trial.measured(configs[i].id, Measurement([7.0]))
    got = gs.search(O())
    assert [t.config_id for t in got] == ["id=1", "id=2", "id=0"]


def test_measurement_quantiles():
    m = Measurement([4.0, 1.0, 3.0, 2.0])
    assert m.median_ms() == 2.5 and m.min_ms() == 1.0 and m.mean_ms() == 2.5 and m.reps() == 4
    assert m.quantile_ms(0.0) == 1.0 and m.quantile_ms(1.0) == 4.0
    assert BenchOptions().clear_l2 and BenchOptions().min_reps == 5


def test_serving_attention_launchers_infer_reference_generics():
    """Generic strings and grids of the serving kernels as the reference's launchers would produce them
    (cutile-kernels/src/attention.rs:398-440, 588-613, 738-757, 921-939); no device needed."""
    from cutile_rs_b200 import launch
    f16 = torch.float16
    heads_kv, group, d, cap, ns = 2, 4, 128, 640, 5
    q = Tensor(torch.zeros(heads_kv, group, d, dtype=f16))
    k = Tensor(torch.zeros(heads_kv, cap, d, dtype=f16))
    att = Tensor(torch.zeros(heads_kv, ns * group, d, dtype=f16))
    lse = Tensor(torch.zeros(heads_kv, ns * group))
    pos = Tensor(torch.zeros(1, dtype=torch.int32))
    la = launch.fmha_decode_gqa_split(q, k, k, att.partition([1, group, d]), lse.partition([1, group]), 0.088, pos,
                                      bn=64)
    assert la.infer_generics() == ["f16", "4", "64", "128", "5", "2"]
    assert infer_launch_grid((0, 0, 0), la._bounds()) == (heads_kv, ns, 1)
    out = Tensor(torch.zeros(heads_kv, group, d, dtype=f16))
    lm = launch.splitk_reduce_merge(att, lse, out.partition([1, group, 32]))
    assert lm.infer_generics() == ["f16", "4", "128", "32", "5", "20", "2"]
    assert infer_launch_grid((0, 0, 0), lm._bounds()) == (heads_kv, 1, 4)
    qp = Tensor(torch.zeros(200, heads_kv * group, d, dtype=f16))
    op = Tensor(torch.zeros(200, heads_kv * group, d, dtype=f16))
    lg = launch.fmha_prefill_gqa(qp, k, k, op.partition([32, group, d]), 0.088, group, 200)
    assert lg.infer_generics() == ["f16", "32", "128", "128", "4", "128", "1", "0", "2"]
    assert infer_launch_grid((0, 0, 0), lg._bounds()) == (7, heads_kv, 1)
    lc = launch.fmha_causal(qp, k, k, op.partition([128, 1, d]), 0.088, group, pos)
    assert lc.infer_generics() == ["f16", "128", "128", "128", "1", "1"]
    # the f16 scalar parameter is marshalled as two bytes holding the rounded half
    pa = launch._ParamArray()
    pa.push("f16", 0.088)
    assert pa._keep[0].value == int(np.float16(0.088).view(np.uint16))
