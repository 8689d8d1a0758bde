"""Kernel launchers: the Python mirror of the macro-generated launcher structs.

A launcher is a lazy operation (the ``DeviceOp`` idea, cuda-async/src/device_operation.rs:185-385):
building it validates nothing and touches no device; ``.sync()/.sync_on()/.async_on()`` run the
generated ``execute`` sequence (cutile-macro/src/kernel_launcher_generator.rs:819-987) -- resolve
generics, infer and validate the grid, marshal the flattened parameter array -- and then make ONE
call into the C ABI (``b200tile_launch``) where the reference would JIT-compile and call
``cuLaunchKernel``.  Outputs come back in signature order, the same objects that went in
(:670-687).
"""
from __future__ import annotations

import ctypes
import struct
from ctypes import c_char_p, c_float, c_int32, c_uint, c_uint64, c_void_p
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple, Union

import torch

from . import _lib
from .tensor import (Grid, GridBound, KernelLaunchError, MappedLaunchPartition, Partition, Tensor,
                     infer_launch_grid)


@dataclass
class CompileOptions:
    """``CompileOptions`` (cutile-compiler/src/hints.rs:94-126); ``None`` = not set."""
    occupancy: Optional[int] = None
    num_cta_in_cga: Optional[int] = None
    max_divisibility: Optional[int] = None
    num_worker_warps_per_cta: Optional[int] = None

    def to_c(self) -> _lib.CompileOptionsC:
        f = lambda v: -1 if v is None else int(v)
        return _lib.CompileOptionsC(f(self.occupancy), f(self.num_cta_in_cga),
                                    f(self.max_divisibility), f(self.num_worker_warps_per_cta))


class DevicePtr(int):
    """A raw device address passed as a kernel parameter (`*mut T` in the reference's raw-pointer kernels)."""


class F16(float):
    """A scalar kernel parameter of type f16 (the `qk_scale: f16` of the decode kernels,
    cutile-kernels/src/attention.rs:610,754): two bytes in the parameter array."""


Output = Union[Partition, MappedLaunchPartition]
Arg = Union[Partition, MappedLaunchPartition, Tensor, int, float]


class _ParamArray:
    """Owns the C values behind a ``void*[]`` kernel parameter array."""

    def __init__(self):
        self._keep = []

    def push(self, kind: str, value) -> None:
        if kind == "f16":
            self._keep.append(ctypes.c_uint16(struct.unpack("<H", struct.pack("<e", value))[0]))
            return
        ctype = {"u64": c_uint64, "i32": c_int32, "f32": c_float}[kind]
        self._keep.append(ctype(value))

    def as_c(self):
        arr = (c_void_p * len(self._keep))()
        for i, v in enumerate(self._keep):
            arr[i] = ctypes.cast(ctypes.pointer(v), c_void_p)
        return arr, len(self._keep)


class KernelLauncher:
    """One kernel invocation being built (``TileKernel`` trait, cutile/src/tile_kernel.rs:1036-1106)."""

    kernel_name = ""

    def __init__(self, args: Sequence[Arg]):
        self.args = list(args)
        self._generics: Optional[List[str]] = None
        self._grid: Grid = (0, 0, 0)
        self._opts: Optional[CompileOptions] = None
        self._compile_only = False

    # ---- builder methods (cutile-macro/src/_module.rs:901-923) ----
    def generics(self, generics: Sequence[str]) -> "KernelLauncher":
        self._generics = [str(g) for g in generics]
        return self

    def grid(self, grid: Grid) -> "KernelLauncher":
        self._grid = tuple(int(g) for g in grid)
        return self

    const_grid = grid

    def compile_options(self, opts: CompileOptions) -> "KernelLauncher":
        self._opts = opts
        return self

    # ---- to be provided per kernel ----
    def infer_generics(self) -> List[str]:
        raise KernelLaunchError(f"{self.kernel_name}: generics must be given explicitly")

    # ---- execution ----
    def _resolved_generics(self) -> List[str]:
        return self._generics if self._generics is not None else self.infer_generics()

    def _bounds(self) -> List[GridBound]:
        return [a.grid_bound() for a in self.args if isinstance(a, (Partition, MappedLaunchPartition))]

    def _marshal(self) -> _ParamArray:
        pa = _ParamArray()
        for a in self.args:
            if isinstance(a, (Partition, MappedLaunchPartition, Tensor)):
                for kind, v in a.kernel_args():
                    pa.push(kind, v)
            elif isinstance(a, DevicePtr):
                pa.push("u64", int(a))
            elif isinstance(a, bool):
                pa.push("i32", int(a))
            elif isinstance(a, int):
                pa.push("i32", a)
            elif isinstance(a, F16):
                pa.push("f16", float(a))
            elif isinstance(a, float):
                pa.push("f32", a)
            else:
                raise KernelLaunchError(f"{self.kernel_name}: unsupported argument {type(a)}")
        return pa

    def compile(self) -> "KernelLauncher":
        """Warm-up without launching (the ``.compile()`` path, cutile-macro/src/_module.rs:852-866)."""
        lib = _lib.load()
        gens = self._resolved_generics()
        garr = (c_char_p * len(gens))(*[g.encode() for g in gens])
        opts = self._opts.to_c() if self._opts else None
        rc = lib.b200tile_prepare(self.kernel_name.encode(), garr, len(gens),
                                  ctypes.byref(opts) if opts else None)
        if rc:
            raise KernelLaunchError(lib.b200tile_last_error().decode())
        return self

    def execute(self, stream: torch.cuda.Stream) -> Tuple:
        """Enqueues the kernel on ``stream`` without synchronising."""
        lib = _lib.load()
        gens = self._resolved_generics()
        grid = infer_launch_grid(self._grid, self._bounds())
        pa = self._marshal()
        params, n_params = pa.as_c()
        garr = (c_char_p * len(gens))(*[g.encode() for g in gens])
        cgrid = (c_uint * 3)(*grid)
        opts = self._opts.to_c() if self._opts else None
        rc = lib.b200tile_launch(self.kernel_name.encode(), garr, len(gens),
                                 ctypes.byref(opts) if opts else None, params, n_params, cgrid,
                                 c_void_p(stream.cuda_stream))
        if rc:
            raise KernelLaunchError(lib.b200tile_last_error().decode())
        return self._recover()

    def _recover(self) -> Tuple:
        # a mapped output is returned as its plain partition (cutile/src/tensor.rs:1945-1956)
        return tuple(a.partition if isinstance(a, MappedLaunchPartition) else a for a in self.args)

    def sync_on(self, stream: torch.cuda.Stream) -> Tuple:
        out = self.execute(stream)
        stream.synchronize()
        return out

    def sync(self) -> Tuple:
        return self.sync_on(torch.cuda.current_stream())

    def async_on(self, stream: torch.cuda.Stream) -> Tuple:
        """Enqueue only; the caller orders later work on the same stream (``unsafe async_on``)."""
        return self.execute(stream)

    def graph_on(self, stream: torch.cuda.Stream) -> "CudaGraph":
        return CudaGraph.capture(self, stream)


class CudaGraph:
    """Capture once, replay many times (cuda-async/src/cuda_graph.rs:61-137,179-208)."""

    def __init__(self, graph: torch.cuda.CUDAGraph, output: Tuple, stream: torch.cuda.Stream):
        self._graph = graph
        self._output = output
        self._stream = stream

    @staticmethod
    def capture(op: KernelLauncher, stream: torch.cuda.Stream) -> "CudaGraph":
        _lib.load()
        g = torch.cuda.CUDAGraph()
        stream.synchronize()
        with torch.cuda.graph(g, stream=stream, capture_error_mode="relaxed"):
            out = op.execute(torch.cuda.current_stream())
        return CudaGraph(g, out, stream)

    @staticmethod
    def scope(stream: torch.cuda.Stream, record) -> "CudaGraph":
        """``CudaGraph::scope(&stream, |s| s.record(op))`` (cuda_graph.rs:400-505): ``record`` gets a
        function that enqueues launchers into the capture."""
        _lib.load()
        g = torch.cuda.CUDAGraph()
        outs = []
        stream.synchronize()
        with torch.cuda.graph(g, stream=stream, capture_error_mode="relaxed"):
            cur = torch.cuda.current_stream()
            record(lambda op: outs.append(op.execute(cur)) or outs[-1])
        return CudaGraph(g, tuple(outs), stream)

    def launch(self) -> "CudaGraph":
        self._graph.replay()
        return self

    def sync(self) -> "CudaGraph":
        torch.cuda.current_stream().synchronize()
        return self

    def take_output(self) -> Tuple:
        return self._output


# ---------------------------------------------------------------------------------------------
# Concrete launchers
# ---------------------------------------------------------------------------------------------
class _GemmLauncher(KernelLauncher):
    """z[M,N] = x[M,K] . y[K,N]  (generics [T, BM, BN, BK, ...])."""

    def infer_generics(self) -> List[str]:
        z = self.args[0]
        bm, bn = z.partition_shape[-2], z.partition_shape[-1]
        return [z.dtype_str(), str(bm), str(bn), "64" if z.dtype_str() != "f32" else "16"]


class Gemm(_GemmLauncher):
    kernel_name = "gemm"


class GemmAcc(_GemmLauncher):
    kernel_name = "gemm_acc"


class GemmPersistent(_GemmLauncher):
    kernel_name = "gemm_persistent"

    def infer_generics(self) -> List[str]:
        z = self.args[0]
        base = super().infer_generics()
        ms = z.map_shape if isinstance(z, MappedLaunchPartition) else [8, 1]
        return base + [str(ms[0]), str(ms[1] if len(ms) > 1 else 1)]


class BatchMatmul(_GemmLauncher):
    kernel_name = "batch_matmul"


def gemm(z: Output, x: Tensor, y: Tensor, k: Optional[int] = None) -> Gemm:
    """Non-persistent form: one [BM,BN] tile per tile-block, accumulator starts at zero
    (cutile-benchmarks/paper/sec5_exp1_safety_overhead/rust/gemm/src/main.rs:74-96)."""
    return Gemm([z, x, y] + ([int(k)] if k is not None else []))


def gemm_acc(z: Output, x: Tensor, y: Tensor) -> GemmAcc:
    """z += x . y, z loaded as the initial accumulator (cutile-examples/examples/gemm.rs:20-36)."""
    return GemmAcc([z, x, y])


def gemm_persistent(z: MappedLaunchPartition, x: Tensor, y: Tensor) -> GemmPersistent:
    """Persistent mapped form (main.rs:98-132; cutile-examples/examples/persistent_gemm.rs:26-58)."""
    return GemmPersistent([z, x, y])


def batch_matmul(z: Output, x: Tensor, y: Tensor) -> BatchMatmul:
    """Per-batch GEMM, grid (batch, M/BM, N/BN) (cutile-examples/examples/batch_matmul.rs:17-43)."""
    return BatchMatmul([z, x, y])


class Fmha(KernelLauncher):
    """out (b*h, m, d) partition [1, BM, D]; q (b,h,m,d); k, v (b,hkv,n,d)."""
    kernel_name = "fmha"

    def __init__(self, args, causal: bool):
        super().__init__(args)
        self._causal = bool(causal)

    def infer_generics(self) -> List[str]:
        out, q, k = self.args[0], self.args[1], self.args[2]
        bm, d = out.partition_shape[1], out.partition_shape[2]
        even_k = int(k.shape[2] % 128 == 0)
        return [out.dtype_str(), str(bm), "128", str(d), str(q.shape[1]), str(int(self._causal)),
                str(even_k)]


class FmhaPrefillCausal(KernelLauncher):
    """q [q_len, heads, D]; k, v [kv_heads, kv_len, D]; out partition [BM, 1, D]."""
    kernel_name = "fmha_prefill_causal"

    def __init__(self, args, causal: bool):
        super().__init__(args)
        self._causal = bool(causal)

    def infer_generics(self) -> List[str]:
        out, k = self.args[3], self.args[1]
        bm, d = out.partition_shape[0], out.partition_shape[2]
        kv_len = self.args[6]
        return [out.dtype_str(), str(bm), "128", str(d), str(int(self._causal)),
                str(int(kv_len % 128 == 0)), "2"]


def fmha(out: Output, q: Tensor, k: Tensor, v: Tensor, qk_scale: float, input_pos: int = 0,
         query_group_size: int = 1, causal: bool = False) -> Fmha:
    """Attention forward in the (b,h,m,d) layout of the examples and benchmarks
    (cutile-examples/examples/flash_attention_causal.rs:19-45; cutile-benchmarks/benches/
    fmha.rs:20-37).  ``causal`` only seeds the inferred CAUSAL generic."""
    return Fmha([out, q, k, v, float(qk_scale), int(input_pos), int(query_group_size)], causal)


def fmha_prefill_causal(q: Tensor, k: Tensor, v: Tensor, out: Output, qk_scale: float,
                        query_group_size: int, kv_len: int, query_start: int = 0,
                        causal: bool = True) -> FmhaPrefillCausal:
    """Prefill attention in the serving layout (cutile-kernels/src/attention.rs:242-262)."""
    return FmhaPrefillCausal([q, k, v, out, float(qk_scale), int(query_group_size), int(kv_len),
                              int(query_start)], causal)


class LinearFp8Blk128(KernelLauncher):
    """z [M,N] = alpha * x_q [M,K] . y_q [N,K]^T with fp32 scales per 1x128 (x) / 128x128 (y) block."""
    kernel_name = "linear_tile_fp8_blk128"

    def infer_generics(self) -> List[str]:
        z = self.args[0]
        return [z.dtype_str(), str(z.partition_shape[0]), str(z.partition_shape[1]), "128", "1"]


def linear_tile_fp8_blk128(z: Output, x: Tensor, y: Tensor, x_scales: Tensor, y_scales: Tensor,
                           alpha: float = 1.0) -> LinearFp8Blk128:
    """Block-scaled fp8 linear layer; same parameter list as the reference's scaled `linear_tile`
    (cutile-examples/examples/mxfp8.rs:34-47) with fp32 scales per 128-block."""
    return LinearFp8Blk128([z, x, y, x_scales, y_scales, float(alpha)])


class LinearTile(KernelLauncher):
    """The reference's block-scaled `linear_tile` under its own name: z [M,N] partition [BM,BN] = alpha * x . y^T.
    NVFP4 operands (``f4e2m1fnx2``) infer generics [BM, BN, BK, BK/2, BK/16] (BK/32 when the scales are
    ``f8e8m0fnu``: MXFP4), MXFP8 operands (``f8e4m3fn``) [BM, BN, BK, BK/32]; a bf16 output prepends its type name
    (the reference's output is f32)."""
    kernel_name = "linear_tile"

    def infer_generics(self) -> List[str]:
        z, x = self.args[0], self.args[1]
        bm, bn = z.partition_shape[0], z.partition_shape[1]
        head = [] if z.dtype_str() == "f32" else [z.dtype_str()]
        if x.dtype == "f4e2m1fnx2":
            # UE8M0 scales per 32 elements (MXFP4) or UE4M3 scales per 16 (NVFP4)
            return head + [str(bm), str(bn), "64", "32", "2" if self.args[3].dtype == "f8e8m0fnu" else "4"]
        if x.dtype == "f8e4m3fn":
            return head + [str(bm), str(bn), "64", "2"]
        raise KernelLaunchError(f"linear_tile: operands of type {x.dtype} are not a block-scaled format "
                                "(f4e2m1fnx2 or f8e4m3fn)")


def linear_tile(z: Output, x: Tensor, y: Tensor, x_scales: Tensor, y_scales: Tensor, alpha: float = 1.0) -> LinearTile:
    """`linear_tile` of cutile-examples/examples/nvfp4.rs:37-76 (x, y packed ``f4e2m1fnx2`` [., K/2], scales
    ``f8e4m3fn`` [., K/16]) and of cutile-examples/examples/mxfp8.rs:34-64 (x, y ``f8e4m3fn`` [., K], scales
    ``f8e8m0fnu`` [., K/32]); which of the two runs follows from the generics, as in the reference the operand
    types are part of the kernel's signature.  The scale re-layout scratch belongs to the library (one block per
    stream); weight scales registered with :func:`nvfp4_register_weight_scales` are used in their prepared form."""
    return LinearTile([z, x, y, x_scales, y_scales, float(alpha)])


def nvfp4_register_weight_scales(y_scales: Tensor, n: int, k: int, prepared: torch.Tensor, config: int = 0) -> None:
    """Registers weight scales prepared by :func:`nvfp4_prepare_weight_scales` under the address of their row-major
    original, for decode-sized calls of :func:`linear_tile`.  Keep both tensors alive until unregistered."""
    lib = _lib.load()
    rc = lib.b200tile_nvfp4_register_weight_scales(y_scales.cu_deviceptr(), n, k, y_scales.strides[0], config,
                                                   prepared.data_ptr())
    if rc:
        raise KernelLaunchError(lib.b200tile_last_error().decode())


def nvfp4_unregister_weight_scales(y_scales: Tensor) -> None:
    lib = _lib.load()
    rc = lib.b200tile_nvfp4_unregister_weight_scales(y_scales.cu_deviceptr())
    if rc:
        raise KernelLaunchError(lib.b200tile_last_error().decode())


def linear_nvfp4(z: Tensor, x: Tensor, y: Tensor, x_scales: Tensor, y_scales: Tensor, alpha: float = 1.0,
                 stream: Optional[torch.cuda.Stream] = None, config: int = -1,
                 workspace: Optional[torch.Tensor] = None) -> Tensor:
    """NVFP4 block-scaled linear layer, z = alpha * x . y^T (`linear_tile` of
    cutile-examples/examples/nvfp4.rs:37-76): x [M,K/2], y [N,K/2] packed f4e2m1fnx2 bytes,
    scales [M,K/16], [N,K/16] f8e4m3fn bytes in logical row-major order.  The scale re-layout needs
    device scratch; pass ``workspace`` (uint8, from :func:`nvfp4_workspace`) to keep the call free
    of allocations, otherwise one is taken from the torch caching allocator."""
    lib = _lib.load()
    s = stream or torch.cuda.current_stream()
    m, n = z.shape
    k = x.shape[1] * 2
    need = int(lib.b200tile_linear_nvfp4_workspace_bytes(m, n, k))
    if workspace is None:
        with torch.cuda.stream(s):
            workspace = torch.empty(need, dtype=torch.uint8, device=z.storage.device)
    rc = lib.b200tile_linear_nvfp4(x.cu_deviceptr(), y.cu_deviceptr(), x_scales.cu_deviceptr(),
                                   y_scales.cu_deviceptr(), z.cu_deviceptr(), z.dtype.encode(), m, n, k,
                                   x.strides[0], y.strides[0], z.strides[0], x_scales.strides[0],
                                   y_scales.strides[0], float(alpha), workspace.data_ptr(),
                                   workspace.numel(), config, c_void_p(s.cuda_stream))
    if rc:
        raise KernelLaunchError(lib.b200tile_last_error().decode())
    return z


def nvfp4_workspace(m: int, n: int, k: int) -> torch.Tensor:
    """Scratch buffer large enough for :func:`linear_nvfp4` on an (m, n, k) problem."""
    need = int(_lib.load().b200tile_linear_nvfp4_workspace_bytes(m, n, k))
    return torch.empty(need, dtype=torch.uint8, device="cuda")


def _i64x2(a, b):
    return (ctypes.c_int64 * 2)(int(a), int(b))


def decode_attention(q: Tensor, k: Tensor, v: Tensor, att_partial: Tensor, lse_partial: Tensor,
                     position_start: Tensor, qk_scale: float, bn: int, num_kv_splits: int,
                     out: Optional[Tensor] = None, stream: Optional[torch.cuda.Stream] = None):
    """Typed call: split-KV GQA decode attention (`fmha_decode_gqa_split`, cutile-kernels/src/attention.rs:727-901):
    q [kv_heads, GROUP, D], k/v [kv_heads, kv_capacity, D], scratch att_partial
    [kv_heads, NUM_KV_SPLITS*GROUP, D] and lse_partial [kv_heads, NUM_KV_SPLITS*GROUP] (f32),
    position_start a device u32[1].  With ``out`` [kv_heads, GROUP, D] the merge
    (`splitk_reduce_merge`, :907-1015) runs right behind the split pass on the same stream."""
    lib = _lib.load()
    s = stream or torch.cuda.current_stream()
    heads, group, d = q.shape
    rc = lib.b200tile_fmha_decode_gqa_split(
        q.dtype.encode(), q.cu_deviceptr(), k.cu_deviceptr(), v.cu_deviceptr(), att_partial.cu_deviceptr(),
        lse_partial.cu_deviceptr(), out.cu_deviceptr() if out is not None else None,
        position_start.cu_deviceptr(), heads, group, d, k.shape[1], int(bn), int(num_kv_splits), float(qk_scale),
        _i64x2(q.strides[0], q.strides[1]), _i64x2(k.strides[0], k.strides[1]), _i64x2(v.strides[0], v.strides[1]),
        _i64x2(att_partial.strides[0], att_partial.strides[1]), lse_partial.strides[0],
        _i64x2(out.strides[0], out.strides[1]) if out is not None else None, c_void_p(s.cuda_stream))
    if rc:
        raise KernelLaunchError(lib.b200tile_last_error().decode())
    return (att_partial, lse_partial) if out is None else (att_partial, lse_partial, out)


def decode_merge(att_partial: Tensor, lse_partial: Tensor, out: Tensor, num_kv_splits: int,
                 stream: Optional[torch.cuda.Stream] = None) -> Tensor:
    """Typed call: merge of split-KV partials (`splitk_reduce_merge`, cutile-kernels/src/attention.rs:907-1015)."""
    lib = _lib.load()
    s = stream or torch.cuda.current_stream()
    heads, group, d = out.shape
    rc = lib.b200tile_splitk_reduce_merge(out.dtype.encode(), att_partial.cu_deviceptr(), lse_partial.cu_deviceptr(),
                                          out.cu_deviceptr(), heads, group, d, int(num_kv_splits),
                                          _i64x2(att_partial.strides[0], att_partial.strides[1]),
                                          lse_partial.strides[0], _i64x2(out.strides[0], out.strides[1]),
                                          c_void_p(s.cuda_stream))
    if rc:
        raise KernelLaunchError(lib.b200tile_last_error().decode())
    return out


class FmhaPrefillGqa(KernelLauncher):
    """q [q_len, q_heads, D]; k, v [kv_heads, kv_len, D]; out partition [BM, GROUP, D]."""
    kernel_name = "fmha_prefill_gqa"

    def __init__(self, args, causal: bool):
        super().__init__(args)
        self._causal = bool(causal)

    def infer_generics(self) -> List[str]:
        out = self.args[3]
        bm, group, d = out.partition_shape
        kv_len = self.args[6]
        return [out.dtype_str(), str(bm), "128", str(d), str(group), str(bm * group), str(int(self._causal)),
                str(int(kv_len % 128 == 0)), "2"]


def fmha_prefill_gqa(q: Tensor, k: Tensor, v: Tensor, out: Output, qk_scale: float, query_group_size: int,
                     kv_len: int, query_start: int = 0, causal: bool = True) -> FmhaPrefillGqa:
    """GQA prefill attention with GROUP query heads per tile-block
    (cutile-kernels/src/attention.rs:398-440)."""
    return FmhaPrefillGqa([q, k, v, out, float(qk_scale), int(query_group_size), int(kv_len), int(query_start)],
                          causal)


class FmhaCausal(KernelLauncher):
    """q [m, h, D]; k, v [hkv, n, D]; out partition [BM, 1, D]; the causal offset is a device u32[1]."""
    kernel_name = "fmha_causal"

    def __init__(self, args, causal: bool):
        super().__init__(args)
        self._causal = bool(causal)

    def infer_generics(self) -> List[str]:
        out, k = self.args[3], self.args[1]
        return [out.dtype_str(), str(out.partition_shape[0]), "128", str(out.partition_shape[2]),
                str(int(self._causal)), str(int(k.shape[1] % 128 == 0))]


def fmha_causal(q: Tensor, k: Tensor, v: Tensor, out: Output, qk_scale: float, query_group_size: int,
                position_start: Tensor, causal: bool = True) -> FmhaCausal:
    """Dynamic-position causal attention (cutile-kernels/src/attention.rs:588-613)."""
    return FmhaCausal([q, k, v, out, F16(qk_scale), int(query_group_size), position_start], causal)


class FmhaDecodeGqaSplit(KernelLauncher):
    """Partial pass of split-KV decode; generics [T, GROUP, BN, D, NUM_KV_SPLITS, LATENCY]."""
    kernel_name = "fmha_decode_gqa_split"

    def __init__(self, args, bn: int):
        super().__init__(args)
        self._bn = int(bn)

    def infer_generics(self) -> List[str]:
        q, att = self.args[0], self.args[3]
        group, d = att.partition_shape[1], att.partition_shape[2]
        whole = att.partition.object if isinstance(att, MappedLaunchPartition) else att.object
        return [q.dtype_str(), str(group), str(self._bn), str(d), str(whole.shape[1] // group), "2"]


def fmha_decode_gqa_split(q: Tensor, k: Tensor, v: Tensor, att_out: Output, lse_out: Output, qk_scale: float,
                          position_start: Tensor, bn: int = 128) -> FmhaDecodeGqaSplit:
    """`fmha_decode_gqa_split` (cutile-kernels/src/attention.rs:738-757): att_out is the [1, GROUP, D]
    partition of [kv_heads, NUM_KV_SPLITS*GROUP, D], lse_out the [1, GROUP] partition of
    [kv_heads, NUM_KV_SPLITS*GROUP]; the grid (kv_heads, NUM_KV_SPLITS, 1) follows from them."""
    return FmhaDecodeGqaSplit([q, k, v, att_out, lse_out, F16(qk_scale), position_start], bn)


class SplitkReduceMerge(KernelLauncher):
    """Generics [T, GROUP, D, CHUNK_D, NUM_KV_SPLITS, NS_GROUP, LATENCY]."""
    kernel_name = "splitk_reduce_merge"

    def infer_generics(self) -> List[str]:
        att, out = self.args[0], self.args[2]
        group, chunk = out.partition_shape[1], out.partition_shape[2]
        ns_group = att.shape[1]
        return [att.dtype_str(), str(group), str(att.shape[2]), str(chunk), str(ns_group // group),
                str(ns_group), "2"]


def splitk_reduce_merge(att_partial: Tensor, lse_partial: Tensor, out: Output) -> SplitkReduceMerge:
    """`splitk_reduce_merge` (cutile-kernels/src/attention.rs:921-939); out is the [1, GROUP, CHUNK_D]
    partition of [kv_heads, GROUP, D]."""
    return SplitkReduceMerge([att_partial, lse_partial, out])


class RmsNormF16(KernelLauncher):
    """Generics [T, N, BLOCK_SIZE]; grid (rows, 1, 1) from the [1, N] output partition."""
    kernel_name = "rms_norm_f16"

    def __init__(self, args, block_size: int):
        super().__init__(args)
        self._block = int(block_size)

    def infer_generics(self) -> List[str]:
        x = self.args[0]   # x, or the residual of the same shape and type
        return [x.dtype_str(), str(x.shape[1]), str(self._block)]


class AddRmsNormF16(RmsNormF16):
    kernel_name = "add_rms_norm_f16"


def rms_norm_f16(x: Tensor, w: Tensor, out: Output, eps: float, block_size: int = 512) -> RmsNormF16:
    """`rms_norm_f16` (cutile-kernels/src/norms.rs:22-27): x [rows, N], w [N], out the [1, N] partition of
    [rows, N]."""
    return RmsNormF16([x, w, out, float(eps)], block_size)


def add_rms_norm_f16(residual: Tensor, x: Tensor, w: Tensor, out: Output, residual_out: Output, eps: float,
                     block_size: int = 512) -> AddRmsNormF16:
    """`add_rms_norm_f16` (cutile-kernels/src/norms.rs:77-84): out and residual_out are [1, N] partitions."""
    return AddRmsNormF16([residual, x, w, out, residual_out, float(eps)], block_size)


class RopeSeqF16(KernelLauncher):
    """Generics [T, D, HALF_D]; grid (seq, heads, 2) from the [1, 1, HALF_D] output partition."""
    kernel_name = "rope_seq_f16"

    def infer_generics(self) -> List[str]:
        x = self.args[0]
        return [x.dtype_str(), str(x.shape[2]), str(x.shape[2] // 2)]


class RopeSeqDynposF16(RopeSeqF16):
    kernel_name = "rope_seq_dynpos_f16"


def rope_seq_f16(x: Tensor, inv_freq: Tensor, out: Output, position_start: int) -> RopeSeqF16:
    """`rope_seq_f16` (cutile-kernels/src/positional.rs:20-25): x [seq, heads, D], inv_freq f32 [D/2], out the
    [1, 1, D/2] partition of [seq, heads, D]."""
    return RopeSeqF16([x, inv_freq, out, int(position_start)])


def rope_seq_dynpos_f16(x: Tensor, inv_freq: Tensor, position_start: Tensor, out: Output) -> RopeSeqDynposF16:
    """`rope_seq_dynpos_f16` (cutile-kernels/src/positional.rs:74-79): the position of the first row is a
    device u32[1] (i64 storage is accepted as in the attention launchers)."""
    return RopeSeqDynposF16([x, inv_freq, position_start, out])


class QkNormRopeKvPrefillRawF16(KernelLauncher):
    """Raw-pointer kernel: generics [T, D, HALF_D, MAX_SEQ] and the grid (seq_len, q_heads + kv_heads, 1) are
    given by the caller, as in the reference (no partitioned argument to infer them from)."""
    kernel_name = "qk_norm_rope_kv_prefill_raw_f16"


class QkNormRopeKvDecodeRawF16(KernelLauncher):
    kernel_name = "qk_norm_rope_kv_decode_raw_f16"


def qk_norm_rope_kv_prefill_raw_f16(q: Tensor, k: Tensor, v: Tensor, q_weight: Tensor, k_weight: Tensor,
                                    inv_freq: Tensor, q_out: Tensor, k_cache: Tensor, v_cache: Tensor, eps: float,
                                    position_start: int) -> QkNormRopeKvPrefillRawF16:
    """`qk_norm_rope_kv_prefill_raw_f16` (cutile-kernels/src/experimental/fused_transformer.rs:22-43): contiguous
    q [seq, q_heads, D], k / v [seq, kv_heads, D], caches [kv_heads, MAX_SEQ, D]."""
    seq, qh, d = q.shape
    kvh, max_seq = k_cache.shape[0], k_cache.shape[1]
    ptrs = [DevicePtr(t.cu_deviceptr()) for t in (q, k, v, q_weight, k_weight, inv_freq, q_out, k_cache, v_cache)]
    op = QkNormRopeKvPrefillRawF16(ptrs + [float(eps), int(position_start), int(seq), int(qh), int(kvh)])
    return op.generics([q.dtype_str(), d, d // 2, max_seq]).grid((seq, qh + kvh, 1))


def qk_norm_rope_kv_decode_raw_f16(qkv: Tensor, q_weight: Tensor, k_weight: Tensor, inv_freq: Tensor, q_out: Tensor,
                                   k_cache: Tensor, v_cache: Tensor, position_start: Tensor, eps: float,
                                   num_q_heads: int, num_kv_heads: int) -> QkNormRopeKvDecodeRawF16:
    """`qk_norm_rope_kv_decode_raw_f16` (fused_transformer.rs:356-372): qkv is one fused projection row,
    [(q_heads + 2 kv_heads) * D]; the position is a device u32[1]."""
    d, max_seq = k_cache.shape[2], k_cache.shape[1]
    ptrs = [DevicePtr(t.cu_deviceptr()) for t in (qkv, q_weight, k_weight, inv_freq, q_out, k_cache, v_cache)]
    op = QkNormRopeKvDecodeRawF16(ptrs + [position_start, float(eps), int(num_q_heads), int(num_kv_heads)])
    return op.generics([qkv.dtype_str(), d, d // 2, max_seq]).grid((1, num_q_heads + num_kv_heads, 1))


class ArgmaxBlocksF16(KernelLauncher):
    """Generics [T, BLOCK_SIZE]; grid (blocks, 1, 1) from the [1] output partitions."""
    kernel_name = "argmax_blocks_f16"

    def __init__(self, args, block_size: int):
        super().__init__(args)
        self._block = int(block_size)

    def infer_generics(self) -> List[str]:
        return [self.args[0].dtype_str(), str(self._block)]


class LmHeadArgmaxBlocksF16(KernelLauncher):
    """Generics [T, K]; 64 vocabulary rows per block."""
    kernel_name = "lm_head_argmax_blocks_f16"

    def infer_generics(self) -> List[str]:
        w = self.args[0]
        return [w.dtype_str(), str(w.shape[1])]


class ArgmaxReduceBlocksToU32(KernelLauncher):
    """Generic [BLOCK_SIZE] >= num_blocks; one tile block."""
    kernel_name = "argmax_reduce_blocks_to_u32"

    def __init__(self, args, block_size: int):
        super().__init__(args)
        self._block = int(block_size)

    def infer_generics(self) -> List[str]:
        return [str(self._block)]


def argmax_blocks_f16(logits: Tensor, block_max: Output, block_idx: Output, length: int,
                      block_size: int = 1024) -> ArgmaxBlocksF16:
    """`argmax_blocks_f16` (cutile-kernels/src/argmax.rs:20-25); block_max (f32) and block_idx (u32 / i32 storage)
    are [1] partitions of ceil(len / BLOCK_SIZE) entries."""
    return ArgmaxBlocksF16([logits, block_max, block_idx, int(length)], block_size)


def lm_head_argmax_blocks_f16(weights: Tensor, hidden: Tensor, block_max: Output, block_idx: Output,
                              vocab_size: int) -> LmHeadArgmaxBlocksF16:
    """`lm_head_argmax_blocks_f16` (cutile-kernels/src/argmax.rs:88-94): weights [vocab, K], hidden [1, K]; outputs
    are [1] partitions of ceil(vocab / 64) entries."""
    return LmHeadArgmaxBlocksF16([weights, hidden, block_max, block_idx, int(vocab_size)])


def argmax_reduce_blocks_to_u32(block_max: Tensor, block_idx: Tensor, out: Output, num_blocks: int,
                                block_size: Optional[int] = None) -> ArgmaxReduceBlocksToU32:
    """`argmax_reduce_blocks_to_u32` (cutile-kernels/src/argmax.rs:162-167); out is the [1] partition of a
    one-element tensor.  BLOCK_SIZE defaults to the next power of two >= num_blocks."""
    bs = block_size or max(1, 1 << (int(num_blocks) - 1).bit_length())
    return ArgmaxReduceBlocksToU32([block_max, block_idx, out, int(num_blocks)], bs)


class Add2dF16(KernelLauncher):
    """Generics [T, BLOCK_SIZE]; grid (rows, ceil(cols / BLOCK_SIZE), 1) from the [1, BLOCK_SIZE] output partition."""
    kernel_name = "add_2d_f16"

    def infer_generics(self) -> List[str]:
        out = self.args[0]
        return [out.dtype_str(), str(out.partition_shape[1])]


class SiluMul2dF16(Add2dF16):
    kernel_name = "silu_mul_2d_f16"


def add_2d_f16(out: Output, lhs: Tensor, rhs: Tensor) -> Add2dF16:
    """`add_2d_f16` (cutile-kernels/src/pointwise.rs:20-24): out is the [1, BLOCK_SIZE] partition of [rows, cols]."""
    return Add2dF16([out, lhs, rhs])


def silu_mul_2d_f16(out: Output, gate: Tensor, up: Tensor) -> SiluMul2dF16:
    """`silu_mul_2d_f16` (cutile-kernels/src/pointwise.rs:50-54)."""
    return SiluMul2dF16([out, gate, up])


class GroupGemmF16NtDesc(KernelLauncher):
    """Generics [T, BM, BN, BK, NUM_SM]; the grid is (NUM_SM, 1, 1) as in the reference launcher."""
    kernel_name = "group_gemm_f16_nt_desc"

    def __init__(self, args, dtype: str, bn: int):
        super().__init__(args)
        self._dtype, self._bn = dtype, int(bn)

    def infer_generics(self) -> List[str]:
        return [self._dtype, "128", str(self._bn), "64", str(_lib.load().b200tile_num_sms())]

    def _bounds(self) -> List[GridBound]:
        return []


def group_gemm_f16_nt_desc(a_ptrs: Tensor, b_ptrs: Tensor, c_ptrs: Tensor, a_metas: Tensor, b_metas: Tensor,
                           c_metas: Tensor, num_groups: int, dtype: str = "f16", bn: int = 256) -> GroupGemmF16NtDesc:
    """Persistent grouped GEMM over expert descriptor tables (cutile-kernels/src/experimental/moe.rs:
    66-85): i64 pointer arrays [G] and i32 extent tables [G, 8] = {rows, cols, row stride, ...}, all on
    the device.  The launch grid defaults to one tile-block per SM."""
    la = GroupGemmF16NtDesc([a_ptrs, b_ptrs, c_ptrs, a_metas, b_metas, c_metas, int(num_groups)], dtype, bn)
    return la.grid((_lib.load().b200tile_num_sms(), 1, 1))


def group_gemm_tables(a_list: Sequence[torch.Tensor], b_list: Sequence[torch.Tensor],
                      c_list: Sequence[torch.Tensor]):
    """Builds the six device tables of :func:`group_gemm_f16_nt_desc` from lists of 2-D device tensors
    (the host-side bucketing step of the reference's MoE example)."""
    def tables(ts):
        ptrs = torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64)
        metas = torch.zeros(len(ts), 8, dtype=torch.int32)
        for i, t in enumerate(ts):
            if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
                raise KernelLaunchError("group_gemm: operands must be 2-D with a contiguous last axis")
            metas[i, 0], metas[i, 1], metas[i, 2] = t.shape[0], t.shape[1], t.stride(0)
        dev = ts[0].device
        return Tensor(ptrs.to(dev)), Tensor(metas.to(dev))
    (ap, am), (bp, bm), (cp, cm) = tables(a_list), tables(b_list), tables(c_list)
    return ap, bp, cp, am, bm, cm


def linear_swiglu(out: Tensor, x: Tensor, w_gate_up: Tensor, stream: Optional[torch.cuda.Stream] = None) -> Tensor:
    """out [M, I] = silu(x . w[:I]^T) * (x . w[I:]^T) in one kernel: the NT linear layer and
    `silu_mul_2d_f16` (cutile-kernels/src/pointwise.rs:50-77) fused; x [M, K], w_gate_up [2I, K]."""
    lib = _lib.load()
    s = stream or torch.cuda.current_stream()
    m, inter = out.shape
    k = x.shape[1]
    if tuple(w_gate_up.shape) != (2 * inter, k) or x.shape[0] != m:
        raise KernelLaunchError("linear_swiglu: expected x [M,K], w_gate_up [2I,K], out [M,I]")
    rc = lib.b200tile_linear_swiglu(out.dtype_str().encode(), x.cu_deviceptr(), w_gate_up.cu_deviceptr(),
                                    out.cu_deviceptr(), m, inter, k, x.strides[0], w_gate_up.strides[0],
                                    out.strides[0], c_void_p(s.cuda_stream))
    if rc:
        raise KernelLaunchError(lib.b200tile_last_error().decode())
    return out


def linear_bias_residual(out: Tensor, x: Tensor, w: Tensor, bias: Optional[Tensor] = None,
                         residual: Optional[Tensor] = None, stream: Optional[torch.cuda.Stream] = None) -> Tensor:
    """out [M, N] = x . w^T (+ bias [N]) (+ residual [M, N]) in one kernel (``b200tile_linear_bias_residual``): the NT
    linear layer with the residual add of `add_2d_f16` (cutile-kernels/src/pointwise.rs:20-36) in its epilogue;
    x [M, K], w [N, K]; ``out`` may be ``residual``."""
    lib = _lib.load()
    s = stream or torch.cuda.current_stream()
    m, n = out.shape
    k = x.shape[1]
    if tuple(w.shape) != (n, k) or x.shape[0] != m or (residual is not None and tuple(residual.shape) != (m, n)) or \
            (bias is not None and bias.size() != n):
        raise KernelLaunchError("linear_bias_residual: expected x [M,K], w [N,K], bias [N], residual / out [M,N]")
    rc = lib.b200tile_linear_bias_residual(out.dtype_str().encode(), x.cu_deviceptr(), w.cu_deviceptr(),
                                           bias.cu_deviceptr() if bias is not None else None,
                                           residual.cu_deviceptr() if residual is not None else None, out.cu_deviceptr(),
                                           m, n, k, x.strides[0], w.strides[0],
                                           residual.strides[0] if residual is not None else 0, out.strides[0],
                                           c_void_p(s.cuda_stream))
    if rc:
        raise KernelLaunchError(lib.b200tile_last_error().decode())
    return out


def nvfp4_prepare_weight_scales(y_scales: Tensor, n: int, k: int, config: int = 0,
                                stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """Brings weight scales [N, K/16] into the kernel's tile layout once (``b200tile_nvfp4_prepare_weight_scales``);
    the returned uint8 buffer goes to :func:`linear_nvfp4_prepared` with the same ``config``."""
    lib = _lib.load()
    s = stream or torch.cuda.current_stream()
    need = int(lib.b200tile_nvfp4_weight_scales_bytes(n, k, config))
    with torch.cuda.stream(s):
        buf = torch.empty(need, dtype=torch.uint8, device=y_scales.storage.device)
    rc = lib.b200tile_nvfp4_prepare_weight_scales(y_scales.cu_deviceptr(), n, k, y_scales.strides[0], config,
                                                  buf.data_ptr(), need, c_void_p(s.cuda_stream))
    if rc:
        raise KernelLaunchError(lib.b200tile_last_error().decode())
    return buf


def linear_nvfp4_prepared(z: Tensor, x: Tensor, y: Tensor, x_scales: Tensor, y_scales_prepared: torch.Tensor,
                          alpha: float = 1.0, config: int = 0, stream: Optional[torch.cuda.Stream] = None) -> Tensor:
    """NVFP4 linear layer on weight scales prepared by :func:`nvfp4_prepare_weight_scales`: one kernel, no
    workspace; otherwise the operands of :func:`linear_nvfp4`."""
    lib = _lib.load()
    s = stream or torch.cuda.current_stream()
    m, n = z.shape
    k = x.shape[1] * 2
    rc = lib.b200tile_linear_nvfp4_prepared(x.cu_deviceptr(), y.cu_deviceptr(), x_scales.cu_deviceptr(),
                                            y_scales_prepared.data_ptr(), z.cu_deviceptr(), z.dtype_str().encode(),
                                            m, n, k, x.strides[0], y.strides[0], z.strides[0], x_scales.strides[0],
                                            float(alpha), config, c_void_p(s.cuda_stream))
    if rc:
        raise KernelLaunchError(lib.b200tile_last_error().decode())
    return z
