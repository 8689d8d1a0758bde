// Rotary position embedding (chunked / GPT-NeoX layout) over [seq, heads, D] 16-bit tensors.
//
// Replaces `rope_seq_f16` and `rope_seq_dynpos_f16` (cutile-kernels/src/positional.rs:20-62, 74-120):
//     theta = float(position_start + s) * inv_freq[i]               i in [0, D/2)
//     out[s, h, i]       = round16(x[s, h, i] * cos(theta) - x[s, h, i + D/2] * sin(theta))
//     out[s, h, i + D/2] = round16(x[s, h, i + D/2] * cos(theta) + x[s, h, i] * sin(theta))
// The reference launches one tile block per (position, head, half) and evaluates cos and sin in each
// of them; the angles depend on the position only, so here a CTA takes one position, D/2 of its
// threads evaluate the angles once into shared memory, and all threads then stream the heads with
// 16-byte loads and stores.  HBM-bound: one read and one write per element.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "host_common.h"

namespace b200 {

namespace {

constexpr int ROPE_THREADS = 256;
constexpr int ROPE_MAX_HALF = 256;   // head_dim up to 512

template <bool F16>
__device__ __forceinline__ float rope_to_f32(uint16_t bits) {
  if (F16) {
    __half_raw r;
    r.x = bits;
    return __half2float(__half(r));
  }
  return __uint_as_float((uint32_t)bits << 16);
}
template <bool F16>
__device__ __forceinline__ uint16_t rope_to_16(float v) {
  if (F16) return __half_as_ushort(__float2half_rn(v));
  return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}

struct RopeParams {
  const uint16_t* x;
  const float* inv_freq;
  uint16_t* out;
  const uint32_t* pos_ptr;    // device-side position of the first row, or null
  int position_start;
  int seq, heads, half_d;
  long long xs_seq, xs_head, os_seq, os_head;   // strides in elements
  int vec;                    // 1: 16-byte accesses are possible
};

template <bool F16>
__global__ void __launch_bounds__(ROPE_THREADS) rope_seq_kernel(const RopeParams p) {
  __shared__ float s_cos[ROPE_MAX_HALF], s_sin[ROPE_MAX_HALF];
  const int s = blockIdx.x;
  const int base = p.pos_ptr ? (int)__ldg(p.pos_ptr) : p.position_start;
  const float pos = (float)(base + s);
  for (int i = threadIdx.x; i < p.half_d; i += ROPE_THREADS) {
    const float theta = __fmul_rn(pos, __ldg(p.inv_freq + i));
    float sn, cs;
    sincosf(theta, &sn, &cs);
    s_cos[i] = cs;
    s_sin[i] = sn;
  }
  __syncthreads();
  const uint16_t* xrow = p.x + (long long)s * p.xs_seq;
  uint16_t* orow = p.out + (long long)s * p.os_seq;
  if (p.vec) {
    const int vph = p.half_d / 8;                      // 8-element vectors per half head
    for (int vi = threadIdx.x; vi < p.heads * vph; vi += ROPE_THREADS) {
      const int h = vi / vph, v = vi - h * vph;
      const uint16_t* xh = xrow + (long long)h * p.xs_head + v * 8;
      uint16_t* oh = orow + (long long)h * p.os_head + v * 8;
      const uint4 qlo = __ldg(reinterpret_cast<const uint4*>(xh));
      const uint4 qhi = __ldg(reinterpret_cast<const uint4*>(xh + p.half_d));
      const uint32_t lo[4] = {qlo.x, qlo.y, qlo.z, qlo.w}, hi[4] = {qhi.x, qhi.y, qhi.z, qhi.w};
      uint32_t ylo[4], yhi[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        uint16_t a[2], b[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const float xl = rope_to_f32<F16>((uint16_t)(lo[e] >> (16 * k)));
          const float xh2 = rope_to_f32<F16>((uint16_t)(hi[e] >> (16 * k)));
          const float cs = s_cos[v * 8 + 2 * e + k], sn = s_sin[v * 8 + 2 * e + k];
          a[k] = rope_to_16<F16>(__fsub_rn(__fmul_rn(xl, cs), __fmul_rn(xh2, sn)));
          b[k] = rope_to_16<F16>(__fadd_rn(__fmul_rn(xh2, cs), __fmul_rn(xl, sn)));
        }
        ylo[e] = (uint32_t)a[0] | ((uint32_t)a[1] << 16);
        yhi[e] = (uint32_t)b[0] | ((uint32_t)b[1] << 16);
      }
      *reinterpret_cast<uint4*>(oh) = make_uint4(ylo[0], ylo[1], ylo[2], ylo[3]);
      *reinterpret_cast<uint4*>(oh + p.half_d) = make_uint4(yhi[0], yhi[1], yhi[2], yhi[3]);
    }
  } else {
    for (int ei = threadIdx.x; ei < p.heads * p.half_d; ei += ROPE_THREADS) {
      const int h = ei / p.half_d, i = ei - h * p.half_d;
      const uint16_t* xh = xrow + (long long)h * p.xs_head;
      uint16_t* oh = orow + (long long)h * p.os_head;
      const float xl = rope_to_f32<F16>(xh[i]), xh2 = rope_to_f32<F16>(xh[i + p.half_d]);
      const float cs = s_cos[i], sn = s_sin[i];
      oh[i] = rope_to_16<F16>(__fsub_rn(__fmul_rn(xl, cs), __fmul_rn(xh2, sn)));
      oh[i + p.half_d] = rope_to_16<F16>(__fadd_rn(__fmul_rn(xh2, cs), __fmul_rn(xl, sn)));
    }
  }
}

}  // namespace
}  // namespace b200

// dtype: 0 = bf16, 1 = f16.  Strides in elements; the innermost stride is 1.  `out` may alias `x`
// (every thread reads both halves of its elements before it writes them).
int b200_rope_seq_dispatch(int dtype, const void* x, const float* inv_freq, void* out, int seq, int heads,
                           int head_dim, long long xs_seq, long long xs_head, long long os_seq, long long os_head,
                           int position_start, const uint32_t* pos_ptr, cudaStream_t stream) {
  using namespace b200;
  if (!b200h::device_info()) return B200_ERR_CUDA;
  if (head_dim % 2 || head_dim / 2 > ROPE_MAX_HALF)
    return b200h::set_error(B200_ERR_UNSUPPORTED, "rope_seq: D=%d must be even and at most %d", head_dim,
                            2 * ROPE_MAX_HALF);
  RopeParams p;
  p.x = static_cast<const uint16_t*>(x);
  p.inv_freq = inv_freq;
  p.out = static_cast<uint16_t*>(out);
  p.pos_ptr = pos_ptr;
  p.position_start = position_start;
  p.seq = seq;
  p.heads = heads;
  p.half_d = head_dim / 2;
  p.xs_seq = xs_seq;
  p.xs_head = xs_head;
  p.os_seq = os_seq;
  p.os_head = os_head;
  const uintptr_t al = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out);
  p.vec = (al & 15) == 0 && p.half_d % 8 == 0 && !(xs_seq & 7) && !(xs_head & 7) && !(os_seq & 7) && !(os_head & 7);
  if (dtype)
    rope_seq_kernel<true><<<(unsigned)seq, ROPE_THREADS, 0, stream>>>(p);
  else
    rope_seq_kernel<false><<<(unsigned)seq, ROPE_THREADS, 0, stream>>>(p);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
