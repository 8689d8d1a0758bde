"""Tensor creation and host<->device copies (the subset of cutile/src/api.rs:215-724 the
contraction kernels' callers use).  Storage is a ``torch.Tensor`` on the current CUDA device;
copies are stream-ordered and use pinned host memory, like the reference's
``copy_host_vec_to_device`` / ``to_host_vec`` (cutile/src/tile_kernel.rs:1446-1457).

``randn`` in the reference draws from cuRAND (cutile/src/api.rs:683-698), which cannot be
reproduced off-device; here random tensors come from a seeded host generator so that the kernels
and the CPU oracle see bit-identical inputs.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .tensor import Tensor, _NAME_TO_TORCH


def _device() -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("b200tile needs a CUDA device (sm_100a); there is no CPU fallback")
    return torch.device("cuda", torch.cuda.current_device())


def zeros(shape: Sequence[int], dtype: str = "f32") -> Tensor:
    return Tensor(torch.zeros(*shape, dtype=_NAME_TO_TORCH[dtype], device=_device()), dtype)


def ones(shape: Sequence[int], dtype: str = "f32") -> Tensor:
    return Tensor(torch.ones(*shape, dtype=_NAME_TO_TORCH[dtype], device=_device()), dtype)


def full(shape: Sequence[int], value: float, dtype: str = "f32") -> Tensor:
    return Tensor(torch.full(tuple(shape), value, dtype=_NAME_TO_TORCH[dtype], device=_device()),
                  dtype)


def randn(mean: float, std: float, shape: Sequence[int], seed: Optional[int] = None,
          dtype: str = "f32") -> Tensor:
    g = torch.Generator(device="cpu")
    if seed is not None:
        g.manual_seed(int(seed))
    host = torch.randn(*shape, generator=g, dtype=torch.float32) * std + mean
    return copy_host_to_device(host.to(_NAME_TO_TORCH[dtype]), dtype)


def pin(host: torch.Tensor) -> torch.Tensor:
    """Returns ``host`` in page-locked memory (copying once if needed)."""
    return host if host.is_pinned() else host.contiguous().pin_memory()


def copy_host_to_device(host: torch.Tensor, dtype: Optional[str] = None,
                        stream: Optional[torch.cuda.Stream] = None) -> Tensor:
    """Stream-ordered host -> device copy (``api::copy_host_vec_to_device``)."""
    s = stream or torch.cuda.current_stream()
    with torch.cuda.stream(s):
        dev = torch.empty(host.shape, dtype=host.dtype, device=_device())
        dev.copy_(host, non_blocking=True)
    return Tensor(dev, dtype)


def copy_host_vec_to_device(host: torch.Tensor, dtype: Optional[str] = None) -> Tensor:
    return copy_host_to_device(host.reshape(-1), dtype)


def from_torch(t: torch.Tensor, dtype: Optional[str] = None) -> Tensor:
    """Borrow a foreign allocation (``Tensor::from_foreign``, cutile/src/tensor.rs:839-907)."""
    return Tensor.from_torch(t, dtype)


class HostGemm:
    """C = A.B for operands that live in HOST memory, as one upload / multiply / download pipeline
    (`b200tile_gemm_host`).  The device staging buffers are allocated once here and reused by
    every call; the host operands should be page-locked (:func:`pin`)."""

    def __init__(self, m: int, n: int, k: int, dtype: str = "bf16", b_layout: int = 0, slab_rows: int = 0):
        from . import _lib
        self._lib = _lib.load()
        self._check = _lib.check
        self.m, self.n, self.k, self.dtype, self.b_layout, self.slab_rows = m, n, k, dtype, int(b_layout), slab_rows
        td = _NAME_TO_TORCH[dtype]
        self.a_dev = torch.empty((m, k), dtype=td, device=_device())
        self.b_dev = torch.empty((n, k) if b_layout else (k, n), dtype=td, device=_device())
        self.c_dev = torch.empty((m, n), dtype=td, device=_device())

    def __call__(self, a_host: torch.Tensor, b_host: torch.Tensor, c_host: torch.Tensor,
                 stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        """Queues the pipeline; ``c_host`` is complete once ``stream`` has been synchronised."""
        if tuple(a_host.shape) != (self.m, self.k) or tuple(c_host.shape) != (self.m, self.n) or \
                tuple(b_host.shape) != tuple(self.b_dev.shape):
            raise ValueError("HostGemm: operand shapes do not match the planned problem")
        for t in (a_host, b_host, c_host):
            if t.device.type != "cpu" or not t.is_contiguous() or t.dtype != self.a_dev.dtype:
                raise ValueError("HostGemm: operands must be contiguous host tensors of the planned type")
        s = stream or torch.cuda.current_stream()
        self._check(self._lib.b200tile_gemm_host(self.dtype.encode(), self.b_layout, a_host.data_ptr(),
                                                  b_host.data_ptr(), c_host.data_ptr(), self.a_dev.data_ptr(),
                                                  self.b_dev.data_ptr(), self.c_dev.data_ptr(), self.m, self.n,
                                                  self.k, self.slab_rows, s.cuda_stream))
        return c_host
