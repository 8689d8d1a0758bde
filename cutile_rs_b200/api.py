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
