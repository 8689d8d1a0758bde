"""b200tile: sm_100a dense-contraction kernels (GEMM, attention forward) behind the cuTile-Rust
launcher contract.  ``api`` creates tensors, ``tensor`` holds the partition/grid logic, ``launch``
the kernel launchers, ``tune``/``benching`` the autotuner and its timing protocol, ``_lib`` the
ctypes binding of the C ABI declared in ``include/b200tile.h``.
"""
from . import api, benching, launch, tensor, tune, workloads  # noqa: F401
from ._lib import B200TileError  # noqa: F401
from .launch import CompileOptions, CudaGraph  # noqa: F401
from .tensor import (OWNED, GridBound, KernelLaunchError, MappedLaunchPartition, Partition,  # noqa: F401
                     Tensor, TensorError)

__all__ = ["api", "benching", "launch", "tensor", "tune", "workloads", "B200TileError",
           "CompileOptions", "CudaGraph", "OWNED", "GridBound", "KernelLaunchError",
           "MappedLaunchPartition", "Partition", "Tensor", "TensorError"]
