// Greedy-decode token selection: block argmax over logits, the LM-head matrix-vector product fused with
// the block argmax (the logits are never written), and the final reduction over the blocks.
//
// Replaces `argmax_blocks_f16`, `lm_head_argmax_blocks_f16` and `argmax_reduce_blocks_to_u32`
// (cutile-kernels/src/argmax.rs:20-69, 81-143, 155-199).  Ties go to the lowest index at every level;
// positions past the end count as -1e30, as in the reference.
//
// The fused kernel is a GEMV over [vocab, K] 16-bit weights: HBM-bound on the weights (one read each).
// A CTA owns 64 vocabulary rows (the block size the reference fixes), its 8 warps take 8 rows each,
// four rows at a time with one 16-byte load per row and lane in flight; the hidden vector sits in
// shared memory in its 16-bit form.  Products and sums are fp32; the order of the additions differs
// from the reference's tile reduction, so a logit agrees to rounding and the chosen token can differ
// only between logits that are equal to within that rounding.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "host_common.h"

namespace b200 {
namespace {

constexpr float ARGMAX_MASKED = -1.0e30f;
constexpr int LMH_ROWS = 64;        // vocabulary rows per block (argmax.rs:97)
constexpr int LMH_THREADS = 256;
constexpr int LMH_MAX_K = 16384;    // hidden vector in shared memory: 32 KB

template <bool F16>
__device__ __forceinline__ float am_to_f32(uint16_t bits) {
  if (F16) {
    __half_raw r;
    r.x = bits;
    return __half2float(__half(r));
  }
  return __uint_as_float((uint32_t)bits << 16);
}
template <bool F16>
__device__ __forceinline__ float2 am_unpack2(uint32_t w) {
  if (F16) return __half22float2(*reinterpret_cast<const __half2*>(&w));
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

// (value, index) with "greater value, then lower index" order
__device__ __forceinline__ void am_take(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) {
    v = ov;
    i = oi;
  }
}
__device__ __forceinline__ void am_warp(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    am_take(v, i, ov, oi);
  }
}
// Block-wide result in thread 0.  `sv`, `si`: one slot per warp.
__device__ __forceinline__ void am_block(float& v, int& i, float* sv, int* si) {
  am_warp(v, i);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sv[warp] = v;
    si[warp] = i;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    v = lane < nw ? sv[lane] : ARGMAX_MASKED;
    i = lane < nw ? si[lane] : 0x7fffffff;
    am_warp(v, i);
  }
}

template <bool F16>
__global__ void __launch_bounds__(256) argmax_blocks_kernel(const uint16_t* __restrict__ logits, float* block_max,
                                                            uint32_t* block_idx, int len, int block_size) {
  __shared__ float sv[8];
  __shared__ int si[8];
  const int base = blockIdx.x * block_size;
  float v = ARGMAX_MASKED;
  int idx = 0x7fffffff;
  for (int e = threadIdx.x; e < block_size; e += blockDim.x) {
    const int g = base + e;
    // past the end: -1e30 at its natural index (argmax.rs:41-46)
    am_take(v, idx, g < len ? am_to_f32<F16>(__ldg(logits + g)) : ARGMAX_MASKED, g);
  }
  am_block(v, idx, sv, si);
  if (threadIdx.x == 0) {
    block_max[blockIdx.x] = v;
    block_idx[blockIdx.x] = (uint32_t)idx;
  }
}

template <bool F16, bool VEC>
__global__ void __launch_bounds__(LMH_THREADS) lm_head_argmax_blocks_kernel(const uint16_t* __restrict__ w,
                                                                            const uint16_t* __restrict__ hidden,
                                                                            float* block_max, uint32_t* block_idx,
                                                                            int vocab, int k, long long ldw) {
  __shared__ __align__(16) uint16_t sh[LMH_MAX_K];
  __shared__ float sv[8];
  __shared__ int si[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (VEC) {
    for (int v8 = threadIdx.x; v8 < k / 8; v8 += LMH_THREADS)
      reinterpret_cast<uint4*>(sh)[v8] = __ldg(reinterpret_cast<const uint4*>(hidden) + v8);
  } else {
    for (int e = threadIdx.x; e < k; e += LMH_THREADS) sh[e] = __ldg(hidden + e);
  }
  __syncthreads();
  const int row0 = blockIdx.x * LMH_ROWS + warp * (LMH_ROWS / 8);
  float best = ARGMAX_MASKED;
  int best_i = 0x7fffffff;
#pragma unroll 1
  for (int r4 = 0; r4 < LMH_ROWS / 8; r4 += 4) {
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const uint16_t* rp[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = row0 + r4 + j;
      rp[j] = w + (long long)(r < vocab ? r : vocab - 1) * ldw;   // rows past the end are masked below
    }
    if (VEC) {
      for (int v8 = lane; v8 < k / 8; v8 += 32) {
        uint4 q[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) q[j] = __ldg(reinterpret_cast<const uint4*>(rp[j]) + v8);
        const uint4 hq = reinterpret_cast<const uint4*>(sh)[v8];
        const uint32_t hw[4] = {hq.x, hq.y, hq.z, hq.w};
        float2 h2[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) h2[e] = am_unpack2<F16>(hw[e]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t ww[4] = {q[j].x, q[j].y, q[j].z, q[j].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 w2 = am_unpack2<F16>(ww[e]);
            acc[j] = fmaf(w2.x, h2[e].x, acc[j]);
            acc[j] = fmaf(w2.y, h2[e].y, acc[j]);
          }
        }
      }
    } else {
      for (int e = lane; e < k; e += 32) {
        const float h = am_to_f32<F16>(sh[e]);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] = fmaf(am_to_f32<F16>(__ldg(rp[j] + e)), h, acc[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
      const int r = row0 + r4 + j;
      am_take(best, best_i, r < vocab ? acc[j] : ARGMAX_MASKED, r);
    }
  }
  am_block(best, best_i, sv, si);
  if (threadIdx.x == 0) {
    block_max[blockIdx.x] = best;
    block_idx[blockIdx.x] = (uint32_t)best_i;
  }
}

__global__ void __launch_bounds__(1024) argmax_reduce_blocks_kernel(const float* __restrict__ block_max,
                                                                    const uint32_t* __restrict__ block_idx,
                                                                    uint32_t* out, int num_blocks) {
  __shared__ float sv[32];
  __shared__ int si[32];
  float v = ARGMAX_MASKED;
  int idx = 0x7fffffff;   // the reference's filler for slots that do not win (argmax.rs:187-190)
  for (int b = threadIdx.x; b < num_blocks; b += blockDim.x) am_take(v, idx, __ldg(block_max + b), (int)__ldg(block_idx + b));
  am_block(v, idx, sv, si);
  if (threadIdx.x == 0) out[0] = (uint32_t)idx;
}

}  // namespace
}  // namespace b200

int b200_argmax_blocks_dispatch(int dtype, const void* logits, float* block_max, uint32_t* block_idx, int len,
                                int block_size, cudaStream_t stream) {
  using namespace b200;
  if (!b200h::device_info()) return B200_ERR_CUDA;
  const int blocks = (len + block_size - 1) / block_size;
  if (dtype)
    argmax_blocks_kernel<true><<<blocks, 256, 0, stream>>>(static_cast<const uint16_t*>(logits), block_max, block_idx,
                                                           len, block_size);
  else
    argmax_blocks_kernel<false><<<blocks, 256, 0, stream>>>(static_cast<const uint16_t*>(logits), block_max,
                                                            block_idx, len, block_size);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_lm_head_argmax_blocks_dispatch(int dtype, const void* weights, const void* hidden, float* block_max,
                                        uint32_t* block_idx, int vocab, int k, long long ldw, cudaStream_t stream) {
  using namespace b200;
  if (!b200h::device_info()) return B200_ERR_CUDA;
  if (k > LMH_MAX_K)
    return b200h::set_error(B200_ERR_UNSUPPORTED, "lm_head_argmax_blocks: K=%d exceeds %d", k, LMH_MAX_K);
  const int blocks = (vocab + LMH_ROWS - 1) / LMH_ROWS;
  const bool vec = k % 8 == 0 && !(ldw & 7) && !((reinterpret_cast<uintptr_t>(weights) | reinterpret_cast<uintptr_t>(hidden)) & 15);
  const uint16_t* w = static_cast<const uint16_t*>(weights);
  const uint16_t* h = static_cast<const uint16_t*>(hidden);
  if (dtype) {
    if (vec) lm_head_argmax_blocks_kernel<true, true><<<blocks, LMH_THREADS, 0, stream>>>(w, h, block_max, block_idx, vocab, k, ldw);
    else lm_head_argmax_blocks_kernel<true, false><<<blocks, LMH_THREADS, 0, stream>>>(w, h, block_max, block_idx, vocab, k, ldw);
  } else {
    if (vec) lm_head_argmax_blocks_kernel<false, true><<<blocks, LMH_THREADS, 0, stream>>>(w, h, block_max, block_idx, vocab, k, ldw);
    else lm_head_argmax_blocks_kernel<false, false><<<blocks, LMH_THREADS, 0, stream>>>(w, h, block_max, block_idx, vocab, k, ldw);
  }
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_argmax_reduce_blocks_dispatch(const float* block_max, const uint32_t* block_idx, uint32_t* out,
                                       int num_blocks, cudaStream_t stream) {
  using namespace b200;
  if (!b200h::device_info()) return B200_ERR_CUDA;
  argmax_reduce_blocks_kernel<<<1, 1024, 0, stream>>>(block_max, block_idx, out, num_blocks);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
