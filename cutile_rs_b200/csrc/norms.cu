// RMSNorm and fused residual-add + RMSNorm over the last dimension of [rows, N] 16-bit tensors.
//
// Replaces `rms_norm_f16` (cutile-kernels/src/norms.rs:22-60) and `add_rms_norm_f16` (:77-137):
//     combined = residual + x          (fp32, from the 16-bit inputs; plain RMSNorm: combined = x)
//     inv      = rsqrt(sum(combined^2) / N + eps)
//     out      = round16((combined * inv) * w)            residual_out = round16(combined)
// The reference reads every row twice (one pass for the sum of squares, one for the output); here a
// row is read once and kept in registers as fp32, so the kernel moves the algorithmic minimum:
// one read of x (and residual) and one write of out (and residual_out).  It is HBM-bound; what
// matters is 16-byte accesses, enough loads in flight, and a grid far larger than the SM count.
//
// Work split: a row is shared by WPR (1, 2, 4 or 8) warps of a 256-thread CTA, each thread owning up
// to four 8-element vectors; 8 / WPR rows per CTA.  Rows longer than 8192 elements, or rows whose
// base / pitch is not 16-byte aligned, take the two-pass route of the reference (re-read instead of
// registers, scalar accesses where needed; the updated residual is then written in the second pass,
// after the last read of the old one, so that the outputs may alias the inputs on every route).
// The order of the fp32 additions differs from the reference's tile reduction, so results agree to
// rounding, not bit for bit.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "host_common.h"

namespace b200 {

namespace {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXV = 4;   // 8-element vectors a thread keeps in registers

template <bool F16>
__device__ __forceinline__ float to_f32(uint16_t bits) {
  if (F16) {
    __half_raw r;
    r.x = bits;
    return __half2float(__half(r));
  }
  return __uint_as_float((uint32_t)bits << 16);
}
template <bool F16>
__device__ __forceinline__ uint16_t to_16(float v) {
  if (F16) return __half_as_ushort(__float2half_rn(v));
  return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
template <bool F16>
__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = to_f32<F16>((uint16_t)(w[i] & 0xffffu));
    f[2 * i + 1] = to_f32<F16>((uint16_t)(w[i] >> 16));
  }
}
template <bool F16>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    w[i] = (uint32_t)to_16<F16>(f[2 * i]) | ((uint32_t)to_16<F16>(f[2 * i + 1]) << 16);
  return make_uint4(w[0], w[1], w[2], w[3]);
}

struct NormParams {
  const uint16_t* residual;   // null for plain RMSNorm
  const uint16_t* x;
  const uint16_t* w;
  uint16_t* out;
  uint16_t* residual_out;     // null for plain RMSNorm
  long long ld_res, ld_x, ld_out, ld_res_out;   // row pitches in elements
  int rows, n;
  int wpr;                    // warps per row
  int nv;                     // 8-element vectors per row taken by the vector path (0: scalar only)
  float eps;
};

// Sum over the WPR warps that share a row.  Every thread of the CTA calls it.
__device__ __forceinline__ float row_sum(float v, int wpr, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (wpr == 1) return v;
  const int warp = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) scratch[warp] = v;
  __syncthreads();
  const int first = warp - warp % wpr;
  float s = 0.0f;
  for (int i = 0; i < wpr; ++i) s += scratch[first + i];
  return s;
}

// CACHE: the row's vectors stay in registers between the two phases (nv <= wpr * 32 * NORM_MAXV).
template <bool F16, bool ADD, bool CACHE>
__global__ void __launch_bounds__(NORM_THREADS) rms_norm_kernel(const NormParams p) {
  __shared__ float scratch[NORM_THREADS / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows_per_cta = (NORM_THREADS / 32) / p.wpr;
  const int row = blockIdx.x * rows_per_cta + warp / p.wpr;
  const bool live = row < p.rows;
  const int idx = (warp % p.wpr) * 32 + lane;      // this thread's place among the row's threads
  const int stride = p.wpr * 32;
  const uint16_t* xr = p.x + (long long)row * p.ld_x;
  const uint16_t* rr = ADD ? p.residual + (long long)row * p.ld_res : nullptr;
  uint16_t* orow = p.out + (long long)row * p.ld_out;
  uint16_t* rorow = ADD ? p.residual_out + (long long)row * p.ld_res_out : nullptr;

  float c[CACHE ? NORM_MAXV : 1][8];
  float ss = 0.0f;
  if (live) {
    // ---- phase 1: combined values, their squares, and (fused form) the updated residual ----
    if (CACHE) {
      uint4 qx[NORM_MAXV], qr[NORM_MAXV];
#pragma unroll
      for (int i = 0; i < NORM_MAXV; ++i) {   // all loads first: up to eight 16-byte loads in flight
        const int vi = idx + i * stride;
        if (vi < p.nv) {
          qx[i] = __ldg(reinterpret_cast<const uint4*>(xr) + vi);
          if (ADD) qr[i] = __ldg(reinterpret_cast<const uint4*>(rr) + vi);
        }
      }
#pragma unroll
      for (int i = 0; i < NORM_MAXV; ++i) {
        const int vi = idx + i * stride;
        if (vi < p.nv) {
          unpack8<F16>(qx[i], c[i]);
          if (ADD) {
            float r8[8];
            unpack8<F16>(qr[i], r8);
#pragma unroll
            for (int e = 0; e < 8; ++e) c[i][e] = r8[e] + c[i][e];
            reinterpret_cast<uint4*>(rorow)[vi] = pack8<F16>(c[i]);
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) ss += c[i][e] * c[i][e];
        }
      }
    } else {
      for (int vi = idx; vi < p.nv; vi += stride) {
        float a[8];
        unpack8<F16>(__ldg(reinterpret_cast<const uint4*>(xr) + vi), a);
        if (ADD) {
          float r8[8];
          unpack8<F16>(__ldg(reinterpret_cast<const uint4*>(rr) + vi), r8);
#pragma unroll
          for (int e = 0; e < 8; ++e) a[e] = r8[e] + a[e];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += a[e] * a[e];
      }
    }
    // elements the vector path does not cover (ragged end, or everything when unaligned)
    for (int e = p.nv * 8 + idx; e < p.n; e += stride) {
      float a = to_f32<F16>(xr[e]);
      if (ADD) a = to_f32<F16>(rr[e]) + a;
      ss += a * a;
    }
  }
  const float total = row_sum(ss, p.wpr, scratch);
  if (!live) return;
  const float inv = rsqrtf(total / (float)p.n + p.eps);

  // ---- phase 2: out = (combined * inv) * w ----
  if (CACHE) {
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int vi = idx + i * stride;
      if (vi < p.nv) {
        float w8[8], o8[8];
        unpack8<F16>(__ldg(reinterpret_cast<const uint4*>(p.w) + vi), w8);
#pragma unroll
        for (int e = 0; e < 8; ++e) o8[e] = (c[i][e] * inv) * w8[e];
        reinterpret_cast<uint4*>(orow)[vi] = pack8<F16>(o8);
      }
    }
  } else {
    for (int vi = idx; vi < p.nv; vi += stride) {
      float a[8], w8[8], o8[8];
      unpack8<F16>(__ldg(reinterpret_cast<const uint4*>(xr) + vi), a);
      if (ADD) {
        float r8[8];
        unpack8<F16>(__ldg(reinterpret_cast<const uint4*>(rr) + vi), r8);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = r8[e] + a[e];
        reinterpret_cast<uint4*>(rorow)[vi] = pack8<F16>(a);
      }
      unpack8<F16>(__ldg(reinterpret_cast<const uint4*>(p.w) + vi), w8);
#pragma unroll
      for (int e = 0; e < 8; ++e) o8[e] = (a[e] * inv) * w8[e];
      reinterpret_cast<uint4*>(orow)[vi] = pack8<F16>(o8);
    }
  }
  for (int e = p.nv * 8 + idx; e < p.n; e += stride) {
    float a = to_f32<F16>(xr[e]);
    if (ADD) {
      a = to_f32<F16>(rr[e]) + a;
      rorow[e] = to_16<F16>(a);
    }
    orow[e] = to_16<F16>((a * inv) * to_f32<F16>(p.w[e]));
  }
}

bool aligned16(const void* ptr, long long ld) {
  return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && (ld & 7) == 0;
}

template <bool F16, bool ADD>
int launch_norm(NormParams p, cudaStream_t stream) {
  const bool vec = aligned16(p.x, p.ld_x) && aligned16(p.out, p.ld_out) && aligned16(p.w, 8) &&
                   (!ADD || (aligned16(p.residual, p.ld_res) && aligned16(p.residual_out, p.ld_res_out)));
  p.nv = vec ? p.n / 8 : 0;
  // as few warps per row as keep the row in registers, so that short rows still fill the CTA
  int wpr = 1;
  while (wpr < 8 && p.nv > wpr * 32 * NORM_MAXV) wpr *= 2;
  if (p.nv == 0) wpr = p.n >= 2048 ? 8 : (p.n >= 256 ? 2 : 1);
  p.wpr = wpr;
  const bool cache = p.nv > 0 && p.nv <= wpr * 32 * NORM_MAXV;
  const int rows_per_cta = (NORM_THREADS / 32) / wpr;
  const long long ctas = ((long long)p.rows + rows_per_cta - 1) / rows_per_cta;
  if (ctas > 0x7fffffffLL) return b200h::set_error(B200_ERR_INVALID, "rms_norm: too many rows");
  if (cache)
    rms_norm_kernel<F16, ADD, true><<<(unsigned)ctas, NORM_THREADS, 0, stream>>>(p);
  else
    rms_norm_kernel<F16, ADD, false><<<(unsigned)ctas, NORM_THREADS, 0, stream>>>(p);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

}  // namespace
}  // namespace b200

// dtype: 0 = bf16, 1 = f16.  residual / residual_out null: plain RMSNorm.  Pitches in elements.
int b200_rms_norm_dispatch(int dtype, const void* residual, const void* x, const void* w, void* out,
                           void* residual_out, int rows, int n, long long ld_res, long long ld_x, long long ld_out,
                           long long ld_res_out, float eps, cudaStream_t stream) {
  using namespace b200;
  if (!b200h::device_info()) return B200_ERR_CUDA;
  NormParams p;
  p.residual = static_cast<const uint16_t*>(residual);
  p.x = static_cast<const uint16_t*>(x);
  p.w = static_cast<const uint16_t*>(w);
  p.out = static_cast<uint16_t*>(out);
  p.residual_out = static_cast<uint16_t*>(residual_out);
  p.ld_res = ld_res;
  p.ld_x = ld_x;
  p.ld_out = ld_out;
  p.ld_res_out = ld_res_out;
  p.rows = rows;
  p.n = n;
  p.wpr = 1;
  p.nv = 0;
  p.eps = eps;
  const bool add = residual != nullptr;
  if (dtype) return add ? launch_norm<true, true>(p, stream) : launch_norm<true, false>(p, stream);
  return add ? launch_norm<false, true>(p, stream) : launch_norm<false, false>(p, stream);
}
