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

// Two 16-bit values <-> two floats with the packed conversion instructions.
template <bool F16>
__device__ __forceinline__ float2 rope_unpack2(uint32_t w) {
  if (F16) return __half22float2(*reinterpret_cast<const __half2*>(&w));
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <bool F16>
__device__ __forceinline__ uint32_t rope_pack2(float a, float b) {
  if (F16) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
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

// ---------------------------------------------------------------------------
// Per-head RMSNorm of Q and K, rotary embedding, and the KV-cache write, in one pass
// ---------------------------------------------------------------------------
// Replaces `qk_norm_rope_kv_prefill_raw_f16` and `qk_norm_rope_kv_decode_raw_f16`
// (cutile-kernels/src/experimental/fused_transformer.rs:22-344, 356 ff.): for every (position, head)
//     inv  = rsqrt(sum(x^2) / D + eps);   n = (x * inv) * w        (fp32, not rounded in between)
//     y_lo = n_lo cos - n_hi sin;  y_hi = n_hi cos + n_lo sin;     theta = float(position + s) * inv_freq
// Q heads go to q_out [seq, q_heads, D]; K heads to k_cache [kv_heads, MAX_SEQ, D] at row position + s,
// and the V heads are copied to v_cache beside them.  One CTA per position: the angles are
// evaluated once, then groups of D/16 lanes take one head each (a 16-byte vector of the low half and
// one of the high half per lane), reduce the squares with shuffles, and write 16-byte vectors.
namespace b200 {
namespace {

struct QkRopeParams {
  const uint16_t *q, *k, *v, *qw, *kw;
  const float* inv_freq;
  uint16_t *q_out, *k_cache, *v_cache;
  const uint32_t* pos_ptr;
  int position_start, seq, q_heads, kv_heads, half_d, max_seq;
  long long q_ss, k_ss, v_ss, qo_ss;   // row (position) strides in elements; heads are D apart
  float eps;
};

// Kept out of line so that the argument reduction of sincosf does not set the register count of the
// streaming part of the kernel.
__device__ __noinline__ void rope_angles(float pos, const float* __restrict__ inv_freq, int half_d, float* s_cos,
                                         float* s_sin) {
  for (int i = threadIdx.x; i < half_d; i += blockDim.x) {
    float sn, cs;
    sincosf(__fmul_rn(pos, __ldg(inv_freq + i)), &sn, &cs);
    s_cos[i] = cs;
    s_sin[i] = sn;
  }
}

template <bool F16, int THREADS>
__global__ void __launch_bounds__(THREADS, 1024 / THREADS) qk_norm_rope_kv_kernel(const QkRopeParams p) {
  __shared__ __align__(16) float s_cos[ROPE_MAX_HALF], s_sin[ROPE_MAX_HALF];
  const int s = blockIdx.x;
  const int base = p.pos_ptr ? (int)__ldg(p.pos_ptr) : p.position_start;
  const int cache_pos = base + s;
  const int d = 2 * p.half_d;
  const int lanes = p.half_d / 8;                 // lanes per head: a power of two, 1..32
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % lanes;                   // this lane's vector inside each half
  const int heads_per_warp = 32 / lanes;
  const int total = p.q_heads + p.kv_heads;       // heads to normalise and rotate
  const int items = total + p.kv_heads;           // ... and V heads to copy
  const int step = (blockDim.x / 32) * heads_per_warp;
  const bool cache_ok = cache_pos >= 0 && cache_pos < p.max_seq;

  // item i: Q head i, K head i - q_heads, or V head i - total.  Source vectors of the low and high half.
  auto load_item = [&](int i, uint4& qlo, uint4& qhi) {
    if (i >= items) return;
    const uint16_t* x;
    if (i < p.q_heads) x = p.q + (long long)s * p.q_ss + (long long)i * d;
    else if (i < total) x = p.k + (long long)s * p.k_ss + (long long)(i - p.q_heads) * d;
    else x = p.v + (long long)s * p.v_ss + (long long)(i - total) * d;
    qlo = __ldg(reinterpret_cast<const uint4*>(x) + sub);
    qhi = __ldg(reinterpret_cast<const uint4*>(x + p.half_d) + sub);
  };
  // every lane of a warp calls this for every round (the shuffles need all of them)
  auto finish_item = [&](int i, const uint4& qlo, const uint4& qhi) {
    const bool rot = i < total;
    float lo[8], hi[8];
    float ss = 0.0f;
    if (rot) {
      const uint32_t wl[4] = {qlo.x, qlo.y, qlo.z, qlo.w}, wh[4] = {qhi.x, qhi.y, qhi.z, qhi.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 a = rope_unpack2<F16>(wl[e]), b = rope_unpack2<F16>(wh[e]);
        lo[2 * e] = a.x;
        lo[2 * e + 1] = a.y;
        hi[2 * e] = b.x;
        hi[2 * e + 1] = b.y;
        ss += a.x * a.x + b.x * b.x;
        ss += a.y * a.y + b.y * b.y;
      }
    }
    for (int o = lanes >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (i >= items) return;
    if (!rot) {
      if (cache_ok) {
        uint16_t* vc = p.v_cache + ((long long)(i - total) * p.max_seq + cache_pos) * d;
        reinterpret_cast<uint4*>(vc)[sub] = qlo;
        reinterpret_cast<uint4*>(vc + p.half_d)[sub] = qhi;
      }
      return;
    }
    const bool is_q = i < p.q_heads;
    const float inv = rsqrtf(ss / (float)d + p.eps);
    const uint16_t* w = is_q ? p.qw : p.kw;
    const uint4 qwl = __ldg(reinterpret_cast<const uint4*>(w) + sub);
    const uint4 qwh = __ldg(reinterpret_cast<const uint4*>(w + p.half_d) + sub);
    const uint32_t wl[4] = {qwl.x, qwl.y, qwl.z, qwl.w}, wh[4] = {qwh.x, qwh.y, qwh.z, qwh.w};
    const float4 c0 = *reinterpret_cast<const float4*>(s_cos + sub * 8), c1 = *reinterpret_cast<const float4*>(s_cos + sub * 8 + 4);
    const float4 n0 = *reinterpret_cast<const float4*>(s_sin + sub * 8), n1 = *reinterpret_cast<const float4*>(s_sin + sub * 8 + 4);
    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
    uint32_t ylo[4], yhi[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 wa = rope_unpack2<F16>(wl[e]), wb = rope_unpack2<F16>(wh[e]);
      const float nl0 = (lo[2 * e] * inv) * wa.x, nl1 = (lo[2 * e + 1] * inv) * wa.y;
      const float nh0 = (hi[2 * e] * inv) * wb.x, nh1 = (hi[2 * e + 1] * inv) * wb.y;
      // the second product of each line is fused into the sum (one rounding less than the tile program)
      ylo[e] = rope_pack2<F16>(fmaf(nl0, cs[2 * e], -(nh0 * sn[2 * e])), fmaf(nl1, cs[2 * e + 1], -(nh1 * sn[2 * e + 1])));
      yhi[e] = rope_pack2<F16>(fmaf(nh0, cs[2 * e], nl0 * sn[2 * e]), fmaf(nh1, cs[2 * e + 1], nl1 * sn[2 * e + 1]));
    }
    uint16_t* o;
    if (is_q) {
      o = p.q_out + (long long)s * p.qo_ss + (long long)i * d;
    } else {
      if (!cache_ok) return;
      o = p.k_cache + ((long long)(i - p.q_heads) * p.max_seq + cache_pos) * d;
    }
    reinterpret_cast<uint4*>(o)[sub] = make_uint4(ylo[0], ylo[1], ylo[2], ylo[3]);
    reinterpret_cast<uint4*>(o + p.half_d)[sub] = make_uint4(yhi[0], yhi[1], yhi[2], yhi[3]);
  };
  // Two rounds per iteration with all four loads issued first; the first iteration's loads go out
  // before the angles are evaluated, which do not depend on them.  64 bytes in flight per thread
  // and 1024 resident threads per SM are what it takes to keep HBM busy at one position per CTA.
  int i0 = warp * heads_per_warp;
  int ia = i0 + lane / lanes, ib = ia + step;
  uint4 alo = make_uint4(0, 0, 0, 0), ahi = alo, blo = alo, bhi = alo;
  load_item(ia, alo, ahi);
  load_item(ib, blo, bhi);
  rope_angles((float)cache_pos, p.inv_freq, p.half_d, s_cos, s_sin);
  __syncthreads();
  while (i0 < items) {
    finish_item(ia, alo, ahi);
    asm volatile("" ::: "memory");   // finish one head before the next: shorter live ranges
    if (i0 + step < items) finish_item(ib, blo, bhi);   // warp-uniform condition
    i0 += 2 * step;
    if (i0 >= items) break;
    ia = i0 + lane / lanes;
    ib = ia + step;
    load_item(ia, alo, ahi);
    load_item(ib, blo, bhi);
  }
}

}  // namespace
}  // namespace b200

int b200_qk_norm_rope_kv_dispatch(int dtype, const void* q, const void* k, const void* v, const void* q_weight,
                                  const void* k_weight, const float* inv_freq, void* q_out, void* k_cache,
                                  void* v_cache, float eps, int position_start, const uint32_t* pos_ptr, int seq,
                                  int q_heads, int kv_heads, int head_dim, int max_seq, long long q_ss,
                                  long long k_ss, long long v_ss, long long qo_ss, cudaStream_t stream) {
  using namespace b200;
  if (!b200h::device_info()) return B200_ERR_CUDA;
  const int half = head_dim / 2, lanes = half / 8;
  if (head_dim % 16 || lanes < 1 || lanes > 32 || (lanes & (lanes - 1)))
    return b200h::set_error(B200_ERR_UNSUPPORTED, "qk_norm_rope_kv: D=%d has no configuration (16, 32, ..., 512)",
                            head_dim);
  const uintptr_t al = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                       reinterpret_cast<uintptr_t>(q_weight) | reinterpret_cast<uintptr_t>(k_weight) |
                       reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_cache) |
                       reinterpret_cast<uintptr_t>(v_cache);
  if ((al & 15) || (q_ss & 7) || (k_ss & 7) || (v_ss & 7) || (qo_ss & 7))
    return b200h::set_error(B200_ERR_ALIGN, "qk_norm_rope_kv: pointers and row pitches must be multiples of 16 bytes");
  QkRopeParams p;
  p.q = static_cast<const uint16_t*>(q);
  p.k = static_cast<const uint16_t*>(k);
  p.v = static_cast<const uint16_t*>(v);
  p.qw = static_cast<const uint16_t*>(q_weight);
  p.kw = static_cast<const uint16_t*>(k_weight);
  p.inv_freq = inv_freq;
  p.q_out = static_cast<uint16_t*>(q_out);
  p.k_cache = static_cast<uint16_t*>(k_cache);
  p.v_cache = static_cast<uint16_t*>(v_cache);
  p.pos_ptr = pos_ptr;
  p.position_start = position_start;
  p.seq = seq;
  p.q_heads = q_heads;
  p.kv_heads = kv_heads;
  p.half_d = half;
  p.max_seq = max_seq;
  p.q_ss = q_ss;
  p.k_ss = k_ss;
  p.v_ss = v_ss;
  p.qo_ss = qo_ss;
  p.eps = eps;
  // One CTA per position.  Prefill: small CTAs (64 threads, 16 per SM) drift apart, so the loads of some
  // overlap the arithmetic of others; 256-thread CTAs moved in step and reached 0.6 of the HBM rate where
  // these reach 0.77.  Few positions (decode): one wide CTA per position finishes its heads in one pass.
#define B200_QK(T_)                                                                     \
  do {                                                                                  \
    if (dtype) qk_norm_rope_kv_kernel<true, T_><<<(unsigned)seq, T_, 0, stream>>>(p);   \
    else qk_norm_rope_kv_kernel<false, T_><<<(unsigned)seq, T_, 0, stream>>>(p);        \
  } while (0)
  if (seq >= 512) B200_QK(64);
  else B200_QK(256);
#undef B200_QK
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
