// Pieces shared by the attention-forward kernels: tile constants, register re-balancing, the packed
// fp32x2 / three-input-max helpers of the softmax loops, and the launch parameters.
#pragma once
#include <math_constants.h>

#include "sm100_ptx.cuh"

namespace b200 {

constexpr int FA_BM = 128;       // query rows per tile
constexpr int FA_BN = 128;       // key rows per tile
constexpr int FA_THREADS = 384;  // 12 warps
constexpr float FA_RESCALE_THRESHOLD = 8.0f;
// Register budget per role (setmaxnreg): 128 x 56 + 256 x 208 = 60416 <= 65536.
constexpr int FA_SOFTMAX_REGS = 208;
constexpr int FA_OTHER_REGS = 56;

template <int N>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed fp32x2 arithmetic and the three-input maximum halve the instruction count of the softmax
// inner loops (the softmax warps are issue- and latency-bound, not special-function-bound).
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

struct FmhaParams {
  int q_len, kv_len;
  int num_q_pairs;   // ceil(q_len / 256)
  int bh_total;      // batch * heads
  int heads, heads_kv, group;
  int causal, input_pos;
  const uint32_t* pos_ptr;  // when non-null the causal offset is read from device memory
  int head_group;    // (batch*head) problems scheduled together for L2 reuse of K/V
  float scale_log2;  // qk_scale * log2(e)
};

}  // namespace b200
