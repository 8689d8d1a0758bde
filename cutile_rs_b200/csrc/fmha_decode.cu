// Split-KV grouped-query decode attention and its merge step.
//
// Replaces `fmha_decode_gqa_split` and `splitk_reduce_merge` (cutile-kernels/src/attention.rs:
// 727-901, 907-1015): one query token per head, GROUP query heads share a K/V head, the key range
// [0, position_start + 1) is cut into NUM_KV_SPLITS ranges of whole BN-key tiles; every
// (kv head, split) produces a normalised partial output and a log2-domain log-sum-exp, and the
// merge weights the partials by exp2(lse - max lse).
//
// The path is HBM-bound (every K/V byte is read once, ~GROUP FLOP per byte), so the design goal is
// bytes in flight, not tensor throughput: one CTA per (kv head, split), four warps, each warp
// streaming 16-key steps through its own 4-deep cp.async ring (32 KiB per warp, 128 KiB per CTA)
// and running a register-resident online softmax with warp-level mma.sync m16n8k16 (queries padded
// to 16 rows).  tcgen05 would add latency and nothing else here.
#include <math_constants.h>

#include "host_common.h"

namespace b200 {

constexpr int DEC_WARPS = 4;
constexpr int DEC_STAGES = 4;
constexpr int DEC_STEP = 16;  // keys per warp step

__device__ __forceinline__ uint32_t dec_smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <bool F16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (F16)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <bool F16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  uint32_t r;
  if (F16) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
template <bool F16>
__device__ __forceinline__ float unpack16(uint16_t h) {
  if (F16) {
    float f;
    asm("{.reg .b16 t; mov.b16 t, %1; cvt.f32.f16 %0, t;}" : "=f"(f) : "h"(h));
    return f;
  }
  return __uint_as_float((uint32_t)h << 16);
}
__device__ __forceinline__ float dec_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct DecodeParams {
  const void* q;    // [kv_heads, group, D]
  const void* k;    // [kv_heads, kv_cap, D]
  const void* v;
  void* att;        // [kv_heads, splits*group, D]
  float* lse;       // [kv_heads, splits*group]
  const uint32_t* pos;
  int64_t q_head_stride, q_row_stride, k_head_stride, k_row_stride, v_head_stride, v_row_stride;
  int64_t att_head_stride, att_row_stride, lse_head_stride;
  int group, kv_cap, bn, splits;
  float scale_log2;
};

template <int D, bool F16>
__global__ void __launch_bounds__(DEC_WARPS * 32)
fmha_decode_split_kernel(const DecodeParams p) {
  constexpr int ROW_BYTES = D * 2;
  constexpr int CHUNKS = ROW_BYTES / 16;                 // 16-byte chunks per key row
  constexpr int TILE_BYTES = DEC_STEP * ROW_BYTES;       // one 16-key K (or V) tile
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x, split = blockIdx.y;

  // key range of this split: whole BN-key tiles (attention.rs:767-780)
  const int s_kv_raw = (int)__ldg(p.pos) + 1;
  const int s_kv = s_kv_raw < p.kv_cap ? s_kv_raw : p.kv_cap;
  const int tiles = (s_kv + p.bn - 1) / p.bn;
  const int tps = (tiles + p.splits - 1) / p.splits;
  const int key_begin = split * tps * p.bn;
  int key_end = (split * tps + tps) * p.bn;
  if (key_end > s_kv) key_end = s_kv;
  const int n_keys = key_end - key_begin;
  const int n_steps = n_keys > 0 ? (n_keys + DEC_STEP - 1) / DEC_STEP : 0;

  const uint16_t* qh = static_cast<const uint16_t*>(p.q) + (int64_t)head * p.q_head_stride;
  const uint8_t* kh = static_cast<const uint8_t*>(p.k) + (int64_t)head * p.k_head_stride * 2;
  const uint8_t* vh = static_cast<const uint8_t*>(p.v) + (int64_t)head * p.v_head_stride * 2;

  // ---- Q as the A operand: 16 rows (query heads of the group, zero beyond) x D ----
  const int r0 = lane >> 2, r1 = r0 + 8, kq = (lane & 3) * 2;
  uint32_t qa[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int c0 = ks * 16 + kq, c1 = c0 + 8;
    qa[ks][0] = r0 < p.group ? *reinterpret_cast<const uint32_t*>(qh + (int64_t)r0 * p.q_row_stride + c0) : 0u;
    qa[ks][1] = r1 < p.group ? *reinterpret_cast<const uint32_t*>(qh + (int64_t)r1 * p.q_row_stride + c0) : 0u;
    qa[ks][2] = r0 < p.group ? *reinterpret_cast<const uint32_t*>(qh + (int64_t)r0 * p.q_row_stride + c1) : 0u;
    qa[ks][3] = r1 < p.group ? *reinterpret_cast<const uint32_t*>(qh + (int64_t)r1 * p.q_row_stride + c1) : 0u;
  }

  uint8_t* my_ring = smem + warp * (DEC_STAGES * STAGE_BYTES);
  const uint32_t ring = dec_smem_u32(my_ring);
  auto issue_step = [&](int step, int stage) {
    // 16 keys x CHUNKS chunks for K and for V; lanes take consecutive 16-byte chunks
    const int key0 = key_begin + step * DEC_STEP;
#pragma unroll
    for (int i = lane; i < DEC_STEP * CHUNKS; i += 32) {
      const int row = i / CHUNKS, ch = i % CHUNKS;
      int key = key0 + row;
      if (key >= p.kv_cap) key = p.kv_cap - 1;  // stay inside the cache; such keys are masked
      const uint32_t dst = ring + stage * STAGE_BYTES + row * ROW_BYTES + ((ch ^ (row & 7)) << 4);
      cp_async16(dst, kh + (int64_t)key * p.k_row_stride * 2 + ch * 16);
      cp_async16(dst + TILE_BYTES, vh + (int64_t)key * p.v_row_stride * 2 + ch * 16);
    }
  };

  float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.0f, 0.0f};
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

  // steps warp, warp + 4, ... ; prologue fills STAGES-1 slots
  const int my_steps = n_steps > warp ? (n_steps - warp + DEC_WARPS - 1) / DEC_WARPS : 0;
#pragma unroll
  for (int s = 0; s < DEC_STAGES - 1; ++s) {
    if (s < my_steps) issue_step(warp + s * DEC_WARPS, s);
    cp_async_commit();
  }
  for (int it = 0; it < my_steps; ++it) {
    const int stage = it % DEC_STAGES;
    const int pre = it + DEC_STAGES - 1;
    if (pre < my_steps) issue_step(warp + pre * DEC_WARPS, pre % DEC_STAGES);
    cp_async_commit();
    cp_async_wait<DEC_STAGES - 1>();
    __syncwarp();
    const uint32_t sK = ring + stage * STAGE_BYTES, sV = sK + TILE_BYTES;
    const int key0 = key_begin + (warp + it * DEC_WARPS) * DEC_STEP;

    // S[16 q x 16 keys] = Q K^T
    float s[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
    {
      const int mid = lane >> 3, row = lane & 7;
      const int key = (mid >> 1) * 8 + row;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int ch = ks * 2 + (mid & 1);
        uint32_t kb[4];
        ldsm_x4(sK + key * ROW_BYTES + ((ch ^ (key & 7)) << 4), kb);
        mma16816<F16>(s[0], qa[ks], kb[0], kb[1]);
        mma16816<F16>(s[1], qa[ks], kb[2], kb[3]);
      }
    }
    // scale, mask keys past the end of the range, online softmax per query row
    float tmax[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + nt * 8 + kq + (e & 1);
        float x = s[nt][e] * p.scale_log2;
        if (key >= key_end) x = -CUDART_INF_F;
        s[nt][e] = x;
        tmax[e >> 1] = fmaxf(tmax[e >> 1], x);
      }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
      tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
      const float m_new = fmaxf(m_run[h], tmax[h]);
      const float m_use = m_new == -CUDART_INF_F ? 0.0f : m_new;
      alpha[h] = dec_ex2(m_run[h] - m_use);   // exp2(-inf) = 0 on the first step
      m_run[h] = m_new;
      float sum = 0.0f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const float a = dec_ex2(s[nt][2 * h] - m_use), b = dec_ex2(s[nt][2 * h + 1] - m_use);
        s[nt][2 * h] = a;
        s[nt][2 * h + 1] = b;
        sum += a + b;
      }
      l_run[h] = l_run[h] * alpha[h] + sum;
    }
    // P (16 q x 16 keys, rounded to the 16-bit type: attention.rs:866-868) as the A operand
    uint32_t pa[4];
    pa[0] = pack16<F16>(s[0][0], s[0][1]);
    pa[1] = pack16<F16>(s[0][2], s[0][3]);
    pa[2] = pack16<F16>(s[1][0], s[1][1]);
    pa[3] = pack16<F16>(s[1][2], s[1][3]);
    // O = O * alpha + P V
    {
      const int mid = lane >> 3, row = lane & 7;
      const int key = (mid & 1) * 8 + row;
#pragma unroll
      for (int c = 0; c < D / 16; ++c) {
        const int ch = c * 2 + (mid >> 1);
        uint32_t vb[4];
        ldsm_x4_trans(sV + key * ROW_BYTES + ((ch ^ (key & 7)) << 4), vb);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float (&acc)[4] = o[c * 2 + half];
          acc[0] *= alpha[0];
          acc[1] *= alpha[0];
          acc[2] *= alpha[1];
          acc[3] *= alpha[1];
          mma16816<F16>(acc, pa, vb[half * 2], vb[half * 2 + 1]);
        }
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  __syncthreads();  // every warp is done with its ring: reuse shared memory for the merge

  // ---- combine the four warps' (m, l, O) ----
  float* sm_m = reinterpret_cast<float*>(smem);                 // [warps][16]
  float* sm_l = sm_m + DEC_WARPS * 16;                          // [warps][16]
  float* sm_o = sm_l + DEC_WARPS * 16;                          // [warps][16][D]
  if ((lane & 3) == 0) {
    sm_m[warp * 16 + r0] = m_run[0];
    sm_m[warp * 16 + r1] = m_run[1];
    sm_l[warp * 16 + r0] = l_run[0];
    sm_l[warp * 16 + r1] = l_run[1];
  }
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    float* base = sm_o + (warp * 16) * D + nt * 8 + kq;
    base[r0 * D] = o[nt][0];
    base[r0 * D + 1] = o[nt][1];
    base[r1 * D] = o[nt][2];
    base[r1 * D + 1] = o[nt][3];
  }
  __syncthreads();
  uint16_t* att = static_cast<uint16_t*>(p.att) + (int64_t)head * p.att_head_stride +
                  (int64_t)(split * p.group) * p.att_row_stride;
  float* lse = p.lse + (int64_t)head * p.lse_head_stride + split * p.group;
  for (int idx = threadIdx.x; idx < p.group * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    float m_all = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) m_all = fmaxf(m_all, sm_m[w * 16 + g]);
    float l_all = 0.0f, acc = 0.0f;
    if (m_all != -CUDART_INF_F) {
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) {
        const float wgt = dec_ex2(sm_m[w * 16 + g] - m_all);
        l_all += sm_l[w * 16 + g] * wgt;
        acc += sm_o[(w * 16 + g) * D + d] * wgt;
      }
    }
    // an empty split contributes nothing: att = 0, lse = -1e30 (attention.rs:790-795 start values)
    const float l_safe = fmaxf(l_all, 1e-8f);
    const float val = m_all == -CUDART_INF_F ? 0.0f : acc / l_safe;
    att[(int64_t)g * p.att_row_stride + d] = (uint16_t)(pack16<F16>(val, 0.0f) & 0xFFFF);
    if (d == 0) lse[g] = m_all == -CUDART_INF_F ? -1.0e30f : m_all + log2f(l_safe);
  }
}

// out[head][g][d] = sum_s w_s att[head][s*group+g][d],  w_s = exp2(lse_s - max) / max(sum, 1e-8)
template <bool F16>
__global__ void splitk_reduce_merge_kernel(const void* att, const float* lse, void* out, int group, int D,
                                           int splits, int64_t att_head_stride, int64_t att_row_stride,
                                           int64_t lse_head_stride, int64_t out_head_stride,
                                           int64_t out_row_stride) {
  const int head = blockIdx.x;
  const uint16_t* a = static_cast<const uint16_t*>(att) + (int64_t)head * att_head_stride;
  const float* l = lse + (int64_t)head * lse_head_stride;
  uint16_t* o = static_cast<uint16_t*>(out) + (int64_t)head * out_head_stride;
  for (int idx = threadIdx.x; idx < group * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    float mx = -CUDART_INF_F;
    for (int s = 0; s < splits; ++s) mx = fmaxf(mx, l[s * group + g]);
    float sum = 0.0f, acc = 0.0f;
    for (int s = 0; s < splits; ++s) {
      const float w = exp2f(l[s * group + g] - mx);
      sum += w;
      acc += w * unpack16<F16>(a[(int64_t)(s * group + g) * att_row_stride + d]);
    }
    const float val = acc / fmaxf(sum, 1e-8f);
    o[(int64_t)g * out_row_stride + d] = (uint16_t)(pack16<F16>(val, 0.0f) & 0xFFFF);
  }
}

template <int D, bool F16>
static int launch_decode(const DecodeParams& p, int kv_heads, void* out, int64_t out_head_stride,
                         int64_t out_row_stride, cudaStream_t stream) {
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  constexpr int SMEM = DEC_WARPS * DEC_STAGES * 2 * DEC_STEP * D * 2;
  static_assert(SMEM >= (int)((DEC_WARPS * 32 + DEC_WARPS * 16 * D) * sizeof(float)), "merge area must fit");
  auto kern = fmha_decode_split_kernel<D, F16>;
  static bool attr_done[64] = {};
  if (!attr_done[di->ordinal]) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    attr_done[di->ordinal] = true;
  }
  kern<<<dim3(kv_heads, p.splits), DEC_WARPS * 32, SMEM, stream>>>(p);
  B200_CUDA_CHECK(cudaGetLastError());
  if (out) {
    splitk_reduce_merge_kernel<F16><<<kv_heads, 128, 0, stream>>>(p.att, p.lse, out, p.group, D, p.splits,
                                                                 p.att_head_stride, p.att_row_stride,
                                                                 p.lse_head_stride, out_head_stride,
                                                                 out_row_stride);
    B200_CUDA_CHECK(cudaGetLastError());
  }
  return B200_OK;
}

}  // namespace b200

// dtype 0 = bf16, 1 = f16.  Runs the split pass and, when `out` is non-null, the merge.
int b200_fmha_decode_dispatch(int dtype, int head_dim, const void* q, const void* k, const void* v, void* att,
                              float* lse, void* out, const uint32_t* pos, int kv_heads, int group, int kv_cap,
                              int bn, int splits, float qk_scale, const int64_t* strides, cudaStream_t stream) {
  using namespace b200;
  DecodeParams p;
  p.q = q; p.k = k; p.v = v; p.att = att; p.lse = lse; p.pos = pos;
  p.q_head_stride = strides[0]; p.q_row_stride = strides[1];
  p.k_head_stride = strides[2]; p.k_row_stride = strides[3];
  p.v_head_stride = strides[4]; p.v_row_stride = strides[5];
  p.att_head_stride = strides[6]; p.att_row_stride = strides[7];
  p.lse_head_stride = strides[8];
  p.group = group; p.kv_cap = kv_cap; p.bn = bn; p.splits = splits;
  p.scale_log2 = qk_scale * 1.4426950408889634f;
#define B200_DEC_CASE(D_, F16_) return launch_decode<D_, F16_>(p, kv_heads, out, strides[9], strides[10], stream)
  if (head_dim == 128 && dtype == 0) B200_DEC_CASE(128, false);
  if (head_dim == 128 && dtype == 1) B200_DEC_CASE(128, true);
  if (head_dim == 64 && dtype == 0) B200_DEC_CASE(64, false);
  if (head_dim == 64 && dtype == 1) B200_DEC_CASE(64, true);
#undef B200_DEC_CASE
  return b200h::set_error(B200_ERR_UNSUPPORTED, "fmha_decode: no kernel for head_dim %d (64 and 128 are provided)",
                          head_dim);
}

int b200_splitk_merge_dispatch(int dtype, int head_dim, const void* att, const float* lse, void* out, int kv_heads,
                               int group, int splits, const int64_t* strides, cudaStream_t stream) {
  using namespace b200;
  if (!b200h::device_info()) return B200_ERR_CUDA;
  if (dtype)
    splitk_reduce_merge_kernel<true><<<kv_heads, 128, 0, stream>>>(att, lse, out, group, head_dim, splits, strides[0],
                                                                  strides[1], strides[2], strides[3], strides[4]);
  else
    splitk_reduce_merge_kernel<false><<<kv_heads, 128, 0, stream>>>(att, lse, out, group, head_dim, splits, strides[0],
                                                                   strides[1], strides[2], strides[3], strides[4]);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
