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


class HostFmha:
    """Attention forward for Q, K, V that live in HOST memory ([problems, seq, head_dim] each, one problem per
    (batch, head)), as one upload / attend / download pipeline over groups of problems: a group's Q, K and V go up
    while the previous group is computed (``b200tile_fmha_fwd``) and the one before that travels back, on three
    streams.  The reference user writes the three phases one after the other (cutile/src/api.rs:371,422 around the
    launch of cutile-benchmarks/benches/fmha.rs:20-146); the elapsed time here approaches bytes up / link bandwidth.
    The device staging buffers are allocated once; the host tensors should be page-locked (:func:`pin`)."""

    def __init__(self, problems: int, seq: int, head_dim: int, dtype: str = "bf16", causal: bool = False,
                 group: int = 32):
        import ctypes
        from . import _lib
        self._lib = _lib.load()
        self._check = _lib.check
        self.problems, self.seq, self.head_dim, self.dtype, self.causal = problems, seq, head_dim, dtype, bool(causal)
        self.group = max(1, min(group, problems))
        td = _NAME_TO_TORCH[dtype]
        shape = (problems, seq, head_dim)
        self.q, self.k, self.v, self.o = (torch.empty(shape, dtype=td, device=_device()) for _ in range(4))
        self._strides = (ctypes.c_int64 * 2)(seq * head_dim, head_dim)
        self._s_in, self._s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def __call__(self, q_host: torch.Tensor, k_host: torch.Tensor, v_host: torch.Tensor, o_host: torch.Tensor,
                 scale: float, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        """Queues the pipeline; ``o_host`` is complete once ``stream`` has been synchronised."""
        for t in (q_host, k_host, v_host, o_host):
            if tuple(t.shape) != tuple(self.q.shape) or t.device.type != "cpu" or not t.is_contiguous() or \
                    t.dtype != self.q.dtype:
                raise ValueError("HostFmha: operands must be contiguous host tensors of the planned shape and type")
        s = stream or torch.cuda.current_stream()
        s_in, s_out, st = self._s_in, self._s_out, self._strides
        s_in.wait_stream(s)       # earlier work on the caller's stream may still use the staging buffers
        s_out.wait_stream(s)
        for p0 in range(0, self.problems, self.group):
            p1 = min(p0 + self.group, self.problems)
            with torch.cuda.stream(s_in):
                self.q[p0:p1].copy_(q_host[p0:p1], non_blocking=True)
                self.k[p0:p1].copy_(k_host[p0:p1], non_blocking=True)
                self.v[p0:p1].copy_(v_host[p0:p1], non_blocking=True)
                up = torch.cuda.Event()
                up.record(s_in)
            s.wait_event(up)
            n = p1 - p0
            self._check(self._lib.b200tile_fmha_fwd(self.dtype.encode(), self.q[p0:p1].data_ptr(), self.k[p0:p1].data_ptr(),
                                                    self.v[p0:p1].data_ptr(), self.o[p0:p1].data_ptr(), 1, n, n, self.seq,
                                                    self.seq, self.head_dim, st, st, st, st, float(scale),
                                                    int(self.causal), 0, s.cuda_stream))
            done = torch.cuda.Event()
            done.record(s)
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                o_host[p0:p1].copy_(self.o[p0:p1], non_blocking=True)
        s.wait_stream(s_in)       # synchronising the caller's stream covers every copy of the call
        s.wait_stream(s_out)
        return o_host


class HostRowPipeline:
    """A linear layer (any kernel that maps row slabs of its activations to the same row slabs of its output) over
    operands in HOST memory, as one upload / compute / download pipeline on three streams: the ``whole`` operands
    (weights and their scales) go up first, then every slab of ``rows_in`` follows, is computed as soon as it has
    arrived (``compute(r0, r1, stream)`` enqueues the kernel for rows [r0, r1) on ``stream``) and its rows of
    ``rows_out`` travel back while the next slab is still coming in.  The block-scaled counterpart of
    :class:`HostGemm`; the reference user writes the three phases in sequence (cutile/src/api.rs:371,422).
    ``whole`` and ``rows_in`` are lists of (host tensor, device tensor), ``rows_out`` of (device tensor, host tensor);
    row-sliced tensors are sliced along their first axis, which holds ``rows`` entries (or a multiple: a scale
    tensor with fewer rows per slab is the caller's to pass as ``whole``)."""

    def __init__(self, rows: int, slab_rows: int):
        if rows <= 0 or slab_rows <= 0:
            raise ValueError("HostRowPipeline: rows and slab_rows must be positive")
        self.rows, self.slab_rows = rows, slab_rows
        _device()
        self._s_in, self._s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def __call__(self, whole, rows_in, rows_out, compute, stream: Optional[torch.cuda.Stream] = None) -> None:
        for h, d in list(whole) + list(rows_in) + [(h_, d_) for d_, h_ in rows_out]:
            if h.device.type != "cpu" or d.device.type != "cuda" or h.shape != d.shape or h.dtype != d.dtype:
                raise ValueError("HostRowPipeline: every pair is (host, device) of one shape and type")
        for h, d in list(rows_in) + [(h_, d_) for d_, h_ in rows_out]:
            if h.shape[0] != self.rows:
                raise ValueError("HostRowPipeline: row-sliced tensors hold one entry per row along their first axis")
        s = stream or torch.cuda.current_stream()
        s_in, s_out = self._s_in, self._s_out
        s_in.wait_stream(s)       # earlier work on the caller's stream may still use the device tensors
        s_out.wait_stream(s)
        with torch.cuda.stream(s_in):
            for h, d in whole:
                d.copy_(h, non_blocking=True)
        for r0 in range(0, self.rows, self.slab_rows):
            r1 = min(r0 + self.slab_rows, self.rows)
            with torch.cuda.stream(s_in):
                for h, d in rows_in:
                    d[r0:r1].copy_(h[r0:r1], non_blocking=True)
                up = torch.cuda.Event()
                up.record(s_in)
            s.wait_event(up)
            compute(r0, r1, s)
            done = torch.cuda.Event()
            done.record(s)
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                for d, h in rows_out:
                    h[r0:r1].copy_(d[r0:r1], non_blocking=True)
        s.wait_stream(s_in)       # synchronising the caller's stream covers every copy of the call
        s.wait_stream(s_out)
