"""Host-side tensor metadata: ``Tensor``, ``Partition``, ``MappedLaunchPartition``, ``GridBound``.

Mirrors the launch-facing part of cutile/src/tensor.rs: a tensor is a device pointer plus i32
shape/strides (:649-655), a partition adds a tile shape and yields the launch grid by ceiling
division per axis, rank <= 3 (:252-262, :447-468), and a mapped partition replaces the logical
grid by ``(num_tile_blocks, 1, 1)`` after validation (:346-401).  Device memory itself is owned by
a ``torch.Tensor`` (storage plumbing only); foreign allocations enter the same way as
``Tensor::from_foreign`` (:839-907) through :meth:`Tensor.from_torch`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

OWNED = 0  # map-shape sentinel for an owned axis (cutile/src/tensor.rs:338)

Grid = Tuple[int, int, int]


class TensorError(ValueError):
    """Counterpart of ``Error::Tensor`` (cutile/src/error.rs)."""


class KernelLaunchError(RuntimeError):
    """Counterpart of ``Error::KernelLaunch`` (cutile/src/error.rs:46-47)."""


# dtype vocabulary of the `generics` strings (cuda-core/src/dtype.rs:147-168)
_TORCH_TO_NAME = {
    torch.float32: "f32",
    torch.float16: "f16",
    torch.bfloat16: "bf16",
    torch.uint8: "u8",
    torch.int32: "i32",
    torch.int64: "i64",
}
for _name, _attr in (("f8e4m3fn", "float8_e4m3fn"), ("f8e5m2", "float8_e5m2"),
                     ("f8e8m0fnu", "float8_e8m0fnu")):
    if hasattr(torch, _attr):
        _TORCH_TO_NAME[getattr(torch, _attr)] = _name
_NAME_TO_TORCH = {v: k for k, v in _TORCH_TO_NAME.items()}
# packed FP4 pairs are bytes on the host side (cuda-core/src/dtype.rs:60-110)
_NAME_TO_TORCH["f4e2m1fnx2"] = torch.uint8


def dtype_name(t: torch.dtype) -> str:
    try:
        return _TORCH_TO_NAME[t]
    except KeyError:
        raise TensorError(f"unsupported element type {t}") from None


@dataclass
class GridBound:
    """``GridBound::Exact`` / ``GridBound::AtMost`` (cutile/src/tensor.rs:1677-1685)."""
    kind: str  # "exact" | "at_most"
    grid: Grid

    @staticmethod
    def Exact(grid: Grid) -> "GridBound":
        return GridBound("exact", tuple(grid))

    @staticmethod
    def AtMost(grid: Grid) -> "GridBound":
        return GridBound("at_most", tuple(grid))


class Tensor:
    """Device tensor metadata (pointer, shape, strides in elements, element type name)."""

    def __init__(self, storage: torch.Tensor, dtype: Optional[str] = None):
        if storage.dim() == 0:
            raise TensorError("rank-0 tensors are not supported")
        self.storage = storage
        self.dtype = dtype or dtype_name(storage.dtype)
        self.shape: List[int] = [int(s) for s in storage.shape]
        self.strides: List[int] = [int(s) for s in storage.stride()]
        for v in self.shape + self.strides:
            if v > 2**31 - 1:
                raise TensorError("shape/stride does not fit the i32 kernel ABI")

    # -- construction -------------------------------------------------------------------
    @staticmethod
    def from_torch(t: torch.Tensor, dtype: Optional[str] = None) -> "Tensor":
        return Tensor(t, dtype)

    # -- facts --------------------------------------------------------------------------
    @property
    def rank(self) -> int:
        return len(self.shape)

    def cu_deviceptr(self) -> int:
        return int(self.storage.data_ptr())

    def size(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def num_bytes(self) -> int:
        return self.size() * self.storage.element_size()

    def dtype_str(self) -> str:
        return self.dtype

    # -- partitioning (cutile/src/tensor.rs:1417-1429) ------------------------------------
    def partition(self, partition_shape: Sequence[int]) -> "Partition":
        return Partition(self, list(partition_shape))

    def partition_prefix(self, partition_shape: Sequence[int]) -> "Partition":
        return Partition(self, list(partition_shape)).prefix()

    def reshape(self, shape: Sequence[int]) -> "Tensor":
        return Tensor(self.storage.reshape(*shape), self.dtype)

    # -- transfers (cutile/src/tile_kernel.rs:1446-1457 `to_host_vec`) ----------------------
    def to_host(self, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        """Device -> pinned host copy on ``stream`` (synchronised before returning)."""
        s = stream or torch.cuda.current_stream()
        with torch.cuda.stream(s):
            host = torch.empty(self.storage.shape, dtype=self.storage.dtype, pin_memory=True)
            host.copy_(self.storage, non_blocking=True)
        s.synchronize()
        return host

    def to_host_vec(self, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        return self.to_host(stream).reshape(-1)

    # -- kernel ABI (cutile/src/tensor.rs:2006-2016) -----------------------------------------
    def kernel_args(self) -> List[Tuple[str, int]]:
        """Flattened parameter values: ptr(u64), dims(i32...), strides(i32...)."""
        return ([("u64", self.cu_deviceptr())] + [("i32", d) for d in self.shape] +
                [("i32", s) for s in self.strides])


@dataclass
class Partition:
    """A tensor plus the tile shape each tile-block owns (cutile/src/tensor.rs:252-262)."""
    object: Tensor
    partition_shape: List[int]
    partition_strides: List[int] = field(default_factory=list)
    prefix_coverage: bool = False

    def __post_init__(self):
        if len(self.partition_shape) != self.object.rank:
            raise TensorError(
                f"partition rank {len(self.partition_shape)} != tensor rank {self.object.rank}")
        if any(p <= 0 for p in self.partition_shape):
            raise TensorError("Partition dimensions must be positive.")
        if not self.partition_strides:
            self.partition_strides = [1] * self.object.rank

    def prefix(self) -> "Partition":
        self.prefix_coverage = True
        return self

    def unpartition(self) -> Tensor:
        return self.object

    def dtype_str(self) -> str:
        return self.object.dtype

    def grid(self) -> Grid:
        """ceil(shape / partition_shape) per axis (cutile/src/tensor.rs:447-468)."""
        return partition_grid(self.object.shape, self.partition_shape)

    def grid_bound(self) -> GridBound:
        g = self.grid()
        return GridBound.AtMost(g) if self.prefix_coverage else GridBound.Exact(g)

    def map(self, map_shape: Sequence[int], num_tile_blocks: int) -> "MappedLaunchPartition":
        if self.prefix_coverage:
            raise TensorError("a partial-coverage (prefix) partition cannot be mapped: a mapped "
                              "schedule covers its full index space by construction")
        return MappedLaunchPartition(self, list(map_shape), int(num_tile_blocks))

    def kernel_args(self) -> List[Tuple[str, int]]:
        """Tensor args followed by partition dims and strides (cutile/src/tensor.rs:1723-1739)."""
        return (self.object.kernel_args() + [("i32", d) for d in self.partition_shape] +
                [("i32", s) for s in self.partition_strides])


def partition_grid(shape: Sequence[int], partition_shape: Sequence[int]) -> Grid:
    if not all(x > 0 for x in shape):
        raise TensorError("Shape dimensions must be positive.")
    rank = len(shape)
    if rank < 1 or rank > 3:
        raise TensorError("Mutable tensor must be at most rank 3.")
    g = [-(-int(s) // int(p)) for s, p in zip(shape, partition_shape)]
    while len(g) < 3:
        g.append(1)
    return (g[0], g[1], g[2])


@dataclass
class MappedLaunchPartition:
    """Host-side mapped partition (cutile/src/tensor.rs:346-401)."""
    partition: Partition
    map_shape: List[int]
    num_tile_blocks: int

    def validate(self, partition_grid_: Grid, num_tile_blocks: int) -> Grid:
        return validate_mapped(self.map_shape, partition_grid_, num_tile_blocks)

    def grid(self) -> Grid:
        return self.validate(self.partition.grid(), self.num_tile_blocks)

    def grid_bound(self) -> GridBound:
        return GridBound.Exact(self.grid())

    def unpartition(self) -> Tensor:
        return self.partition.unpartition()

    def dtype_str(self) -> str:
        return self.partition.dtype_str()

    @property
    def partition_shape(self) -> List[int]:
        return self.partition.partition_shape

    @property
    def object(self) -> Tensor:
        return self.partition.object

    def kernel_args(self) -> List[Tuple[str, int]]:
        return self.partition.kernel_args()  # cutile/src/tensor.rs:1890-1892


def validate_mapped(map_shape: Sequence[int], partition_grid_: Grid, num_tile_blocks: int) -> Grid:
    """The checks of ``MappedLaunchPartition::validate`` (cutile/src/tensor.rs:353-400)."""
    map_rank = len(map_shape)
    if map_rank == 0 or map_rank > 3:
        raise TensorError("mapped partitions require a rank-1 through rank-3 map shape.")
    if all(d == OWNED for d in map_shape):
        raise TensorError("mapped partition requires at least one streamed (non-OWNED) map axis.")
    axes = list(partition_grid_)
    if any(a == 0 for a in axes[:map_rank]):
        raise TensorError("mapped partition requires a non-empty logical partition grid.")
    if any(a != 1 for a in axes[map_rank:]):
        raise TensorError("mapped partition map rank must match the logical partition grid rank.")
    streamed = 1
    for axis, md in zip(axes, map_shape):
        if md != OWNED:
            streamed *= axis
            if streamed > 2**32 - 1:
                raise TensorError("mapped partition logical grid is too large")
    if num_tile_blocks == 0:
        raise TensorError("mapped partition requires num_tile_blocks > 0.")
    if num_tile_blocks > streamed:
        raise TensorError(
            "mapped partition num_tile_blocks cannot exceed the streamed logical tile count.")
    return (num_tile_blocks, 1, 1)


def validate_grid_bounds(grid: Grid, bounds: Sequence[GridBound]) -> None:
    """cutile/src/tile_kernel.rs:782-808: exact bindings must equal the grid, partial-coverage
    bindings bound it per axis."""
    for b in bounds:
        if b.kind == "exact" and tuple(b.grid) != tuple(grid):
            raise KernelLaunchError(
                f"launch grid {tuple(grid)} does not match the inferred partition grid "
                f"{tuple(b.grid)}")
    for b in bounds:
        if b.kind != "at_most":
            continue
        for axis in range(3):
            if grid[axis] > b.grid[axis]:
                raise KernelLaunchError(
                    f"launch grid {tuple(grid)} exceeds the partial-coverage partition grid "
                    f"{tuple(b.grid)} on axis {axis}")


def infer_launch_grid(grid: Grid, bounds: Sequence[GridBound]) -> Grid:
    """cutile/src/tile_kernel.rs:934-967."""
    exact = [b.grid for b in bounds if b.kind == "exact"]
    if tuple(grid) != (0, 0, 0):
        validate_grid_bounds(grid, bounds)
        return tuple(grid)
    if not exact:
        if not bounds:
            raise KernelLaunchError("Launch grid required.")
        raise KernelLaunchError(
            "Launch grid required: a partial-coverage (partition_prefix) binding only bounds the "
            "grid; specify the grid explicitly or bind with partition().")
    g = tuple(exact[0])
    validate_grid_bounds(g, bounds)
    return g


def persistent_num_programs(m: int, n: int, bm: int, bn: int, num_sms: int, num_cta_in_cga: int,
                            occupancy: int) -> int:
    """Persistent grid size (cutile-benchmarks/paper/sec5_exp1_safety_overhead/rust/gemm/src/
    main.rs:796-811)."""
    tiles = max(-(-m // bm) * -(-n // bn), 1)
    sm_programs = max(num_sms // max(num_cta_in_cga, 1), 1)
    return max(min(sm_programs, tiles) * max(occupancy, 1), 1)
