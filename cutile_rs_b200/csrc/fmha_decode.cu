// Split-KV grouped-query decode attention and its merge step.
//
// Replaces `fmha_decode_gqa_split` and `splitk_reduce_merge` (cutile-kernels/src/attention.rs:
// 727-901, 907-1015): one query token per head, GROUP query heads share a K/V head, the key range
// [0, position_start + 1) is cut into NUM_KV_SPLITS ranges of whole BN-key tiles; every
// (kv head, split) produces a normalised partial output and a log2-domain log-sum-exp, and the
// merge weights the partials by exp2(lse - max lse).
//
// The path is HBM-bound (every K/V byte is read once, ~GROUP FLOP per byte), so the design goal is
// bytes in flight per SM at the lowest instruction cost, not tensor throughput: one CTA per
// (kv head, split); every warp owns a private ring of K/V stages filled by TMA (tiled loads with
// the 128-byte swizzle, one elected lane issues them, completion on a per-stage mbarrier) and runs a
// register-resident online softmax with warp-level mma.sync m16n8k16 (queries padded to 16 rows)
// fed by conflict-free ldmatrix reads.  tcgen05 would add latency and nothing else here.
#include <math_constants.h>

#include "host_common.h"
#include "sm100_ptx.cuh"

namespace b200 {

__device__ __forceinline__ uint32_t dec_smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
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
  void* att;        // [kv_heads, splits*group, D]
  float* lse;       // [kv_heads, splits*group]
  const uint32_t* pos;
  int64_t q_head_stride, q_row_stride;
  int64_t att_head_stride, att_row_stride, lse_head_stride;
  int group, kv_cap, bn, splits;
  float scale_log2;
};

// WARPS warps per CTA, STEP keys per warp step, STAGES ring slots per warp.
template <int D, int WARPS, int STEP, int STAGES>
struct DecodeCfg {
  static constexpr int HALVES = D / 64;               // 128-byte (64-element) column blocks per row
  static constexpr int SUB = STEP * 128;               // one TMA box: STEP keys x 128 bytes
  static constexpr int TILE = HALVES * SUB;            // K (or V) tile of one step
  static constexpr int STAGE = 2 * TILE;
  static constexpr int RING = STAGES * STAGE;          // per warp
  static constexpr int BAR_OFF = WARPS * RING;         // mbarriers behind the rings
  static constexpr int SMEM = BAR_OFF + WARPS * STAGES * 8 + 16 + 1024;  // + abort flag + alignment slack
  static_assert(SUB % 1024 == 0, "TMA boxes must start on swizzle-atom boundaries");
  static_assert(WARPS * 16 * D * 4 + WARPS * 32 * 4 <= BAR_OFF, "the cross-warp merge reuses the rings");
};

template <int D, bool F16, int WARPS, int STEP, int STAGES>
__global__ void __launch_bounds__(WARPS * 32)
fmha_decode_split_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                         const DecodeParams p, uint32_t* status) {
  using C = DecodeCfg<D, WARPS, STEP, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x, split = blockIdx.y;
  // the merge kernel may be scheduled now; it waits for this grid to finish before it reads
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (lane == 0) {
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }

  const uint32_t ring = dec_smem_u32(smem) + warp * C::RING;
  const uint32_t bars = dec_smem_u32(smem) + C::BAR_OFF + warp * STAGES * 8;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + C::BAR_OFF + WARPS * STAGES * 8);
  WaitCtx wctx{abort_flag, status};
  if (threadIdx.x == 0) *abort_flag = 0;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(bars + s * 8, 1);
    fence_mbar_init();
  }
  __syncthreads();

  // key range of this split: whole BN-key tiles (attention.rs:767-780)
  const int s_kv_raw = (int)__ldg(p.pos) + 1;
  const int s_kv = s_kv_raw < p.kv_cap ? s_kv_raw : p.kv_cap;
  const int tiles = (s_kv + p.bn - 1) / p.bn;
  const int tps = (tiles + p.splits - 1) / p.splits;
  const int key_begin = split * tps * p.bn;
  int key_end = (split * tps + tps) * p.bn;
  if (key_end > s_kv) key_end = s_kv;
  const int n_keys = key_end - key_begin;
  const int n_steps = n_keys > 0 ? (n_keys + STEP - 1) / STEP : 0;
  // this warp takes steps warp, warp + WARPS, ...
  const int my_steps = n_steps > warp ? (n_steps - warp + WARPS - 1) / WARPS : 0;

  // keys past the cache end read as zero (TMA fill) and are masked; nothing is clamped
  auto issue_step = [&](int it) {
    const int stage = it % STAGES;
    const int key0 = key_begin + (warp + it * WARPS) * STEP;
    const uint32_t dst = ring + stage * C::STAGE, bar = bars + stage * 8;
    mbar_expect_tx(bar, C::STAGE);
#pragma unroll
    for (int h = 0; h < C::HALVES; ++h) {
      tma_load_3d(dst + h * C::SUB, &tmK, bar, h * 64, key0, head);
      tma_load_3d(dst + C::TILE + h * C::SUB, &tmV, bar, h * 64, key0, head);
    }
  };
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s)
      if (s < my_steps) issue_step(s);
  }

  // ---- Q as the A operand: 16 rows (query heads of the group, zero beyond) x D ----
  const uint16_t* qh = static_cast<const uint16_t*>(p.q) + (int64_t)head * p.q_head_stride;
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

  // per-lane ldmatrix offsets inside a box: row*128 + ((chunk ^ row) << 4), chunk = j*2 + bit
  const int mid = lane >> 3, row = lane & 7;
  uint32_t offk[4], offv[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    offk[j] = ((mid >> 1) * 8 + row) * 128 + (((j * 2 + (mid & 1)) ^ row) << 4);   // keys by mid>>1, chunk by mid&1
    offv[j] = ((mid & 1) * 8 + row) * 128 + (((j * 2 + (mid >> 1)) ^ row) << 4);   // keys by mid&1, chunk by mid>>1
  }

  float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.0f, 0.0f};
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

  bool alive = true;
  for (int it = 0; it < my_steps; ++it) {
    const int stage = it % STAGES;
    if (!mbar_wait(wctx, bars + stage * 8, (uint32_t)(it / STAGES) & 1u, 70u + (uint32_t)stage)) {
      alive = false;
      break;
    }
    const uint32_t sK = ring + stage * C::STAGE, sV = sK + C::TILE;
    const int key0 = key_begin + (warp + it * WARPS) * STEP;

    // S[16 q x STEP keys] = Q K^T
    float s[STEP / 8][4];
#pragma unroll
    for (int nt = 0; nt < STEP / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
    for (int kb = 0; kb < STEP / 16; ++kb)
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t kf[4];
        ldsm_x4(sK + (ks >> 2) * C::SUB + kb * 2048 + offk[ks & 3], kf);
        mma16816<F16>(s[kb * 2], qa[ks], kf[0], kf[1]);
        mma16816<F16>(s[kb * 2 + 1], qa[ks], kf[2], kf[3]);
      }
    // scale, mask keys past the end of the range (last step only), online softmax per query row
    const bool ragged = key0 + STEP > key_end;
    float tmax[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
    for (int nt = 0; nt < STEP / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float x = s[nt][e] * p.scale_log2;
        if (ragged && key0 + nt * 8 + kq + (e & 1) >= key_end) x = -CUDART_INF_F;
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
      for (int nt = 0; nt < STEP / 8; ++nt) {
        const float a = dec_ex2(s[nt][2 * h] - m_use), b = dec_ex2(s[nt][2 * h + 1] - m_use);
        s[nt][2 * h] = a;
        s[nt][2 * h + 1] = b;
        sum += a + b;
      }
      l_run[h] = l_run[h] * alpha[h] + sum;
    }
    // O *= alpha, skipped while no row of the warp raised its running maximum
    if (!__all_sync(0xffffffffu, alpha[0] == 1.0f && alpha[1] == 1.0f)) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= alpha[0];
        o[i][1] *= alpha[0];
        o[i][2] *= alpha[1];
        o[i][3] *= alpha[1];
      }
    }
    // O += P V, P (16 q x 16 keys per k-step) rounded to the 16-bit type (attention.rs:866-868)
#pragma unroll
    for (int kb = 0; kb < STEP / 16; ++kb) {
      uint32_t pa[4];
      pa[0] = pack16<F16>(s[kb * 2][0], s[kb * 2][1]);
      pa[1] = pack16<F16>(s[kb * 2][2], s[kb * 2][3]);
      pa[2] = pack16<F16>(s[kb * 2 + 1][0], s[kb * 2 + 1][1]);
      pa[3] = pack16<F16>(s[kb * 2 + 1][2], s[kb * 2 + 1][3]);
#pragma unroll
      for (int c = 0; c < D / 16; ++c) {
        uint32_t vf[4];
        ldsm_x4_trans(sV + (c >> 2) * C::SUB + kb * 2048 + offv[c & 3], vf);
        mma16816<F16>(o[c * 2], pa, vf[0], vf[1]);
        mma16816<F16>(o[c * 2 + 1], pa, vf[2], vf[3]);
      }
    }
    __syncwarp();  // every lane is done reading the slot before it is refilled
    if (lane == 0 && it + STAGES < my_steps) issue_step(it + STAGES);
  }
  (void)alive;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  __syncthreads();  // every warp is done with its ring: reuse shared memory for the merge

  // ---- combine the warps' (m, l, O) ----
  float* sm_m = reinterpret_cast<float*>(smem);                 // [warps][16]
  float* sm_l = sm_m + WARPS * 16;                              // [warps][16]
  float* sm_o = sm_l + WARPS * 16;                              // [warps][16][D]
  if ((lane & 3) == 0) {
    sm_m[warp * 16 + r0] = m_run[0];
    sm_m[warp * 16 + r1] = m_run[1];
    sm_l[warp * 16 + r0] = l_run[0];
    sm_l[warp * 16 + r1] = l_run[1];
  }
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    float* base = sm_o + (warp * 16) * D + nt * 8 + kq;
    if (r0 < p.group) *reinterpret_cast<float2*>(base + r0 * D) = make_float2(o[nt][0], o[nt][1]);
    if (r1 < p.group) *reinterpret_cast<float2*>(base + r1 * D) = make_float2(o[nt][2], o[nt][3]);
  }
  __syncthreads();
  uint16_t* att = static_cast<uint16_t*>(p.att) + (int64_t)head * p.att_head_stride +
                  (int64_t)(split * p.group) * p.att_row_stride;
  float* lse = p.lse + (int64_t)head * p.lse_head_stride + split * p.group;
  for (int idx = threadIdx.x; idx < p.group * (D / 2); idx += blockDim.x) {
    const int g = idx / (D / 2), d = (idx % (D / 2)) * 2;
    float m_all = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) m_all = fmaxf(m_all, sm_m[w * 16 + g]);
    float l_all = 0.0f, acc0 = 0.0f, acc1 = 0.0f;
    if (m_all != -CUDART_INF_F) {
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float wgt = dec_ex2(sm_m[w * 16 + g] - m_all);
        const float2 ov = *reinterpret_cast<const float2*>(sm_o + (w * 16 + g) * D + d);
        l_all += sm_l[w * 16 + g] * wgt;
        acc0 += ov.x * wgt;
        acc1 += ov.y * wgt;
      }
    }
    // an empty split contributes nothing: att = 0, lse = -1e30 (attention.rs:790-795 start values)
    const float l_safe = fmaxf(l_all, 1e-8f);
    const bool empty = m_all == -CUDART_INF_F;
    *reinterpret_cast<uint32_t*>(att + (int64_t)g * p.att_row_stride + d) =
        empty ? 0u : pack16<F16>(acc0 / l_safe, acc1 / l_safe);
    if (d == 0) lse[g] = empty ? -1.0e30f : m_all + log2f(l_safe);
  }
}

// out[head][g][d] = sum_s w_s att[head][s*group+g][d],  w_s = exp2(lse_s - max) / max(sum, 1e-8).
// One CTA per (kv head, query head of the group): 128 threads = (D/VEC column lanes) x (split lanes);
// every split lane walks its share of the splits with VEC-element loads, shared memory adds the lanes.
template <bool F16, int VEC>
__global__ void __launch_bounds__(128)
splitk_reduce_merge_kernel(const void* att, const float* lse, void* out, int group, int D, int splits,
                           int64_t att_head_stride, int64_t att_row_stride, int64_t lse_head_stride,
                           int64_t out_head_stride, int64_t out_row_stride) {
  __shared__ float s_red[4];
  __shared__ float s_acc[128 * VEC];   // [split lanes][D]
  __shared__ float s_w[128];
  // when launched as a programmatic dependent of the split pass: wait until its results are visible
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int head = blockIdx.x, g = blockIdx.y, tid = threadIdx.x;
  const uint16_t* a = static_cast<const uint16_t*>(att) + (int64_t)head * att_head_stride;
  const float* l = lse + (int64_t)head * lse_head_stride + g;
  float mx = -CUDART_INF_F;
  for (int s = tid; s < splits; s += 128) mx = fmaxf(mx, l[s * group]);
#pragma unroll
  for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  if ((tid & 31) == 0) s_red[tid >> 5] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));

  const int col_lanes = D / VEC, split_lanes = 128 / col_lanes;
  const int cl = tid % col_lanes, sl = tid / col_lanes;
  float acc[VEC], wsum = 0.0f;
#pragma unroll
  for (int j = 0; j < VEC; ++j) acc[j] = 0.0f;
  for (int s = sl; s < splits; s += split_lanes) {
    const float w = exp2f(l[s * group] - mx);
    const uint16_t* src = a + (int64_t)(s * group + g) * att_row_stride + cl * VEC;
    uint32_t raw[VEC / 2];
    if (VEC == 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(src);
      raw[0] = v.x; raw[1] = v.y; raw[VEC / 2 - 2] = v.z; raw[VEC / 2 - 1] = v.w;
    } else {
      raw[0] = *reinterpret_cast<const uint32_t*>(src);
    }
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) {
      acc[2 * j] += w * unpack16<F16>((uint16_t)(raw[j] & 0xFFFF));
      acc[2 * j + 1] += w * unpack16<F16>((uint16_t)(raw[j] >> 16));
    }
    wsum += w;
  }
#pragma unroll
  for (int j = 0; j < VEC; ++j) s_acc[sl * D + cl * VEC + j] = acc[j];
  if (cl == 0) s_w[sl] = wsum;
  __syncthreads();
  if (tid < D / 2) {
    float v0 = 0.0f, v1 = 0.0f, wt = 0.0f;
    for (int i = 0; i < split_lanes; ++i) {
      v0 += s_acc[i * D + 2 * tid];
      v1 += s_acc[i * D + 2 * tid + 1];
      wt += s_w[i];
    }
    const float inv = 1.0f / fmaxf(wt, 1e-8f);
    uint16_t* o = static_cast<uint16_t*>(out) + (int64_t)head * out_head_stride + (int64_t)g * out_row_stride;
    *reinterpret_cast<uint32_t*>(o + 2 * tid) = pack16<F16>(v0 * inv, v1 * inv);
  }
}

template <bool F16>
static int launch_merge(const void* att, const float* lse, void* out, int kv_heads, int group, int D, int splits,
                        int64_t att_head_stride, int64_t att_row_stride, int64_t lse_head_stride,
                        int64_t out_head_stride, int64_t out_row_stride, bool dependent, cudaStream_t stream) {
  const bool vec8 = (reinterpret_cast<uintptr_t>(att) % 16 == 0) && att_head_stride % 8 == 0 && att_row_stride % 8 == 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kv_heads, group);
  cfg.blockDim = dim3(128);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent ? 1 : 0;
  if (vec8)
    B200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, splitk_reduce_merge_kernel<F16, 8>, att, lse, out, group, D, splits,
                                       att_head_stride, att_row_stride, lse_head_stride, out_head_stride,
                                       out_row_stride));
  else
    B200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, splitk_reduce_merge_kernel<F16, 2>, att, lse, out, group, D, splits,
                                       att_head_stride, att_row_stride, lse_head_stride, out_head_stride,
                                       out_row_stride));
  return B200_OK;
}

struct DecodeHostArgs {
  const void* k;
  const void* v;
  int64_t k_head_stride, k_row_stride, v_head_stride, v_row_stride;
  int kv_heads;
  void* out;
  int64_t out_head_stride, out_row_stride;
};

template <int D, bool F16, int WARPS, int STEP, int STAGES>
static int launch_decode_variant(const DecodeParams& p, const DecodeHostArgs& h, cudaStream_t stream) {
  using C = DecodeCfg<D, WARPS, STEP, STAGES>;
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  const CUtensorMapDataType dt = F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmK, tmV;
  int rc;
  if ((rc = b200h::encode_tmap_3d(&tmK, dt, 2, h.k, D, p.kv_cap, h.kv_heads, h.k_row_stride * 2, h.k_head_stride * 2,
                                  64, STEP, 1, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  if ((rc = b200h::encode_tmap_3d(&tmV, dt, 2, h.v, D, p.kv_cap, h.kv_heads, h.v_row_stride * 2, h.v_head_stride * 2,
                                  64, STEP, 1, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  auto kern = fmha_decode_split_kernel<D, F16, WARPS, STEP, STAGES>;
  static b200h::DeviceOnce attr_done;
  if (!attr_done.test(di->ordinal)) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    attr_done.set(di->ordinal);
  }
  kern<<<dim3(h.kv_heads, p.splits), WARPS * 32, C::SMEM, stream>>>(tmK, tmV, p, di->status);
  B200_CUDA_CHECK(cudaGetLastError());
  if (h.out)
    return launch_merge<F16>(p.att, p.lse, h.out, h.kv_heads, p.group, D, p.splits, p.att_head_stride,
                             p.att_row_stride, p.lse_head_stride, h.out_head_stride, h.out_row_stride, true, stream);
  return B200_OK;
}

// Eight warps of 16-key steps with three ring slots each (192 KiB of K/V in flight per SM for
// D = 128) measured best among {4 warps x 32 keys x 3, 8 x 16 x 3, 4 x 16 x 6}.
template <int D, bool F16>
static int launch_decode(const DecodeParams& p, const DecodeHostArgs& h, cudaStream_t stream) {
  return launch_decode_variant<D, F16, 8, 16, 3>(p, h, stream);
}

}  // namespace b200

// dtype 0 = bf16, 1 = f16.  Runs the split pass and, when `out` is non-null, the merge.
int b200_fmha_decode_dispatch(int dtype, int head_dim, const void* q, const void* k, const void* v, void* att,
                              float* lse, void* out, const uint32_t* pos, int kv_heads, int group, int kv_cap,
                              int bn, int splits, float qk_scale, const int64_t* strides, cudaStream_t stream) {
  using namespace b200;
  DecodeParams p;
  p.q = q; p.att = att; p.lse = lse; p.pos = pos;
  p.q_head_stride = strides[0]; p.q_row_stride = strides[1];
  p.att_head_stride = strides[6]; p.att_row_stride = strides[7];
  p.lse_head_stride = strides[8];
  p.group = group; p.kv_cap = kv_cap; p.bn = bn; p.splits = splits;
  p.scale_log2 = qk_scale * 1.4426950408889634f;
  DecodeHostArgs h;
  h.k = k; h.v = v;
  h.k_head_stride = strides[2]; h.k_row_stride = strides[3];
  h.v_head_stride = strides[4]; h.v_row_stride = strides[5];
  h.kv_heads = kv_heads; h.out = out;
  h.out_head_stride = strides[9]; h.out_row_stride = strides[10];
#define B200_DEC_CASE(D_, F16_) return launch_decode<D_, F16_>(p, h, stream)
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
  if (head_dim != 64 && head_dim != 128)
    return b200h::set_error(B200_ERR_UNSUPPORTED, "splitk_reduce_merge: head_dim %d (64 and 128 are provided)",
                            head_dim);
  return dtype ? launch_merge<true>(att, lse, out, kv_heads, group, head_dim, splits, strides[0], strides[1],
                                    strides[2], strides[3], strides[4], false, stream)
               : launch_merge<false>(att, lse, out, kv_heads, group, head_dim, splits, strides[0], strides[1],
                                     strides[2], strides[3], strides[4], false, stream);
}
