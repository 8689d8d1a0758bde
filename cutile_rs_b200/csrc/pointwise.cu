// Element-wise kernels over rank-2 16-bit tensors: out = lhs + rhs and out = silu(gate) * up.
//
// Replaces `add_2d_f16` and `silu_mul_2d_f16` (cutile-kernels/src/pointwise.rs:20-36, 50-77).  The sum
// is taken in the 16-bit type (one rounding), as the tile program's `lhs_tile + rhs_tile` is; the SwiGLU
// product follows the program in fp32: sigmoid = 1 / (1 + exp(-gate)), y = (sigmoid * gate) * up, one
// rounding to the 16-bit type.  HBM-bound, two reads and one write per element: 16-byte accesses,
// four of them in flight per thread, grid-stride over the rows' vectors; unaligned tensors or ragged
// row ends take scalar accesses.  (The fused gate/up projection b200tile_linear_swiglu applies the same
// step inside the GEMM epilogue and never writes gate and up.)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "host_common.h"

namespace b200 {
namespace {

constexpr int PW_THREADS = 256;

template <bool F16>
__device__ __forceinline__ float pw_to_f32(uint16_t bits) {
  if (F16) {
    __half_raw r;
    r.x = bits;
    return __half2float(__half(r));
  }
  return __uint_as_float((uint32_t)bits << 16);
}
template <bool F16>
__device__ __forceinline__ uint16_t pw_to_16(float v) {
  if (F16) return __half_as_ushort(__float2half_rn(v));
  return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
// SILU = false: a + b in the 16-bit type; SILU = true: silu(a) * b through fp32.
template <bool F16, bool SILU>
__device__ __forceinline__ uint16_t pw_op(uint16_t a, uint16_t b) {
  const float fa = pw_to_f32<F16>(a), fb = pw_to_f32<F16>(b);
  if (!SILU) return pw_to_16<F16>(__fadd_rn(fa, fb));   // the fp32 sum of two 16-bit values is exact: one rounding
  // fast exp and reciprocal: their error (a few units in the last place of fp32) is far below the
  // rounding of the 16-bit result, and the full-precision forms made the kernel instruction-bound
  const float sig = __fdividef(1.0f, 1.0f + __expf(-fa));
  return pw_to_16<F16>(__fmul_rn(__fmul_rn(sig, fa), fb));
}
template <bool F16, bool SILU>
__device__ __forceinline__ uint4 pw_op8(const uint4& a, const uint4& b) {
  const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
  uint32_t r[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    r[i] = (uint32_t)pw_op<F16, SILU>((uint16_t)(wa[i] & 0xffffu), (uint16_t)(wb[i] & 0xffffu)) |
           ((uint32_t)pw_op<F16, SILU>((uint16_t)(wa[i] >> 16), (uint16_t)(wb[i] >> 16)) << 16);
  return make_uint4(r[0], r[1], r[2], r[3]);
}

struct PwParams {
  uint16_t* out;
  const uint16_t *a, *b;
  int rows, cols;
  long long ld_out, ld_a, ld_b;
  int nv;          // 8-element vectors per row taken by the vector path
};

// Vector index -> (row, vector within the row).  FLAT: the host folded dense tensors into one row, so no
// division at all; otherwise a 32-bit division where the count allows it (a 64-bit one costs about as
// many instructions as the rest of the vector's work).
template <bool FLAT>
__device__ __forceinline__ void pw_split(long long e, int nv, bool small, long long& row, int& v) {
  if (FLAT) {
    row = 0;
    v = (int)e;
  } else if (small) {
    const uint32_t r = (uint32_t)e / (uint32_t)nv;
    row = r;
    v = (int)((uint32_t)e - r * (uint32_t)nv);
  } else {
    row = e / nv;
    v = (int)(e - row * nv);
  }
}

template <bool F16, bool SILU, bool FLAT>
__global__ void __launch_bounds__(PW_THREADS) pointwise_kernel(const PwParams p) {
  const long long total_v = (long long)p.rows * p.nv;
  const bool small = total_v <= 0x7fffffffLL;
  const long long step = (long long)gridDim.x * PW_THREADS;
  long long i = (long long)blockIdx.x * PW_THREADS + threadIdx.x;
  // four vectors per thread and pass, all loads first
  for (; i + 3 * step < total_v; i += 4 * step) {
    uint4 qa[4], qb[4];
    long long off_o[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long e = i + u * step;
      long long row;
      int v;
      pw_split<FLAT>(e, p.nv, small, row, v);
      qa[u] = __ldg(reinterpret_cast<const uint4*>(p.a + row * p.ld_a) + v);
      qb[u] = __ldg(reinterpret_cast<const uint4*>(p.b + row * p.ld_b) + v);
      off_o[u] = row * p.ld_out + (long long)v * 8;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) *reinterpret_cast<uint4*>(p.out + off_o[u]) = pw_op8<F16, SILU>(qa[u], qb[u]);
  }
  for (; i < total_v; i += step) {
    long long row;
    int v;
    pw_split<FLAT>(i, p.nv, small, row, v);
    const uint4 qa = __ldg(reinterpret_cast<const uint4*>(p.a + row * p.ld_a) + v);
    const uint4 qb = __ldg(reinterpret_cast<const uint4*>(p.b + row * p.ld_b) + v);
    *reinterpret_cast<uint4*>(p.out + row * p.ld_out + (long long)v * 8) = pw_op8<F16, SILU>(qa, qb);
  }
  // what the vectors do not cover: ragged row ends, or everything when unaligned
  const int tail = p.cols - p.nv * 8;
  if (tail > 0) {
    const long long total_t = (long long)p.rows * tail;
    for (long long e = (long long)blockIdx.x * PW_THREADS + threadIdx.x; e < total_t; e += step) {
      const long long row = e / tail;
      const int c = p.nv * 8 + (int)(e - row * tail);
      p.out[row * p.ld_out + c] = pw_op<F16, SILU>(p.a[row * p.ld_a + c], p.b[row * p.ld_b + c]);
    }
  }
}

}  // namespace
}  // namespace b200

// dtype: 0 = bf16, 1 = f16; op: 0 = add, 1 = silu(a) * b.  Pitches in elements.  `out` may alias an input.
int b200_pointwise_dispatch(int dtype, int op, void* out, const void* a, const void* b, int rows, int cols,
                            long long ld_out, long long ld_a, long long ld_b, cudaStream_t stream) {
  using namespace b200;
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  PwParams p;
  p.out = static_cast<uint16_t*>(out);
  p.a = static_cast<const uint16_t*>(a);
  p.b = static_cast<const uint16_t*>(b);
  p.rows = rows;
  p.cols = cols;
  p.ld_out = ld_out;
  p.ld_a = ld_a;
  p.ld_b = ld_b;
  const uintptr_t al = reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b);
  const bool vec = (al & 15) == 0 && !(ld_out & 7) && !(ld_a & 7) && !(ld_b & 7);
  p.nv = vec ? cols / 8 : 0;
  // dense tensors whose element count fits the vector index: one long row, no index division in the kernel
  const bool flat = vec && cols % 8 == 0 && ld_out == cols && ld_a == cols && ld_b == cols &&
                    (long long)rows * cols / 8 <= 0x7fffffffLL;
  if (flat) {
    p.nv = (int)((long long)rows * cols / 8);
    p.cols = p.nv * 8;
    p.rows = 1;
  }
  const long long work = (long long)p.rows * (p.nv > 0 ? p.nv : p.cols);
  long long ctas = (work + 4 * PW_THREADS - 1) / (4 * PW_THREADS);
  const long long cap = (long long)di->sm_count * 16;
  ctas = ctas < 1 ? 1 : (ctas > cap ? cap : ctas);
#define B200_PW(F16_, SILU_)                                                               \
  do {                                                                                     \
    if (flat) pointwise_kernel<F16_, SILU_, true><<<(unsigned)ctas, PW_THREADS, 0, stream>>>(p);  \
    else pointwise_kernel<F16_, SILU_, false><<<(unsigned)ctas, PW_THREADS, 0, stream>>>(p);      \
  } while (0)
  if (dtype) {
    if (op) B200_PW(true, true); else B200_PW(true, false);
  } else {
    if (op) B200_PW(false, true); else B200_PW(false, false);
  }
#undef B200_PW
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
