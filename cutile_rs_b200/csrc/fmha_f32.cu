// Attention forward in fp32 on the CUDA cores: out = softmax(scale * Q K^T + mask) V with every product and sum
// in IEEE fp32 (no tensor-core path rounds an fp32 operand), online softmax, head_dim 32 / 64 / 128.
//
// This is the element type of the reference's two asserted attention examples
// (cutile-examples/examples/flash_attention.rs:199-264: f32, 4 x 32 x 1024 x 64, |diff| <= 1e-4 against the CPU
// reference; flash_attention_causal.rs:216-285: f32, 2 x 8 x 64 x 32, causal with input_pos = 5), the attention
// counterpart of the exact fp32 GEMM: a correctness configuration, not a roofline claim.
//
// One CTA of 256 threads per 64 query rows of one (batch, head); key tiles of 64.  Thread (ty, tx) = (tid / 16,
// tid % 16) owns score rows 4 ty .. 4 ty + 3 and score columns 4 tx .. 4 tx + 3, so a score row lives in the 16
// consecutive lanes of a half-warp (max and sum by shuffles), and output rows 4 ty .. with D / 16 columns.
// Q and K sit transposed in shared memory ([d][row]: the inner products read float4 along the rows), P is handed
// over transposed ([key][row]) and V row-major.
#include <math_constants.h>

#include "../../include/b200tile.h"
#include "host_common.h"

namespace b200 {

constexpr int FF_BM = 64, FF_BN = 64, FF_LD = 68;   // 68: float4-aligned rows that do not all start in one bank

template <int D>
struct FmhaF32Smem {
  static constexpr int QT = 0;                       // [D][FF_LD]
  static constexpr int KT = QT + D * FF_LD;          // [D][FF_LD]
  static constexpr int VS = KT + D * FF_LD;          // [FF_BN][D]
  static constexpr int PT = VS + FF_BN * D;          // [FF_BN][FF_LD]
  static constexpr int FLOATS = PT + FF_BN * FF_LD;
};

struct FmhaF32Params {
  const float* q;
  const float* k;
  const float* v;
  float* out;
  int heads, heads_kv, q_len, kv_len;
  int64_t qs0, qs1, ks0, ks1, vs0, vs1, os0, os1;   // element strides: (batch * heads + head), row
  float scale_log2;
  int causal, input_pos;
  const uint32_t* pos_ptr;
};

template <int D>
__global__ void __launch_bounds__(256) fmha_f32_kernel(const FmhaF32Params p) {
  extern __shared__ float4 smem_f4[];
  float* smem = reinterpret_cast<float*>(smem_f4);
  float* Qt = smem + FmhaF32Smem<D>::QT;
  float* Kt = smem + FmhaF32Smem<D>::KT;
  float* Vs = smem + FmhaF32Smem<D>::VS;
  float* Pt = smem + FmhaF32Smem<D>::PT;
  constexpr int DC = D / 16;   // output columns per thread
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int bh = blockIdx.y, b = bh / p.heads, h = bh % p.heads;
  const int hkv = h / (p.heads / p.heads_kv);
  const int q0 = blockIdx.x * FF_BM;
  const int input_pos = p.pos_ptr ? (int)*p.pos_ptr : p.input_pos;
  const float* qb = p.q + (int64_t)bh * p.qs0;
  const float* kb = p.k + ((int64_t)b * p.heads_kv + hkv) * p.ks0;
  const float* vb = p.v + ((int64_t)b * p.heads_kv + hkv) * p.vs0;
  float* ob = p.out + (int64_t)bh * p.os0;

  // Q tile, transposed; rows past q_len read as zero
  for (int i = tid; i < FF_BM * D; i += 256) {
    const int r = i / D, d = i % D;
    Qt[d * FF_LD + r] = (q0 + r < p.q_len) ? qb[(int64_t)(q0 + r) * p.qs1 + d] : 0.0f;
  }
  float m_run[4], l_run[4], o[4][DC];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m_run[i] = -CUDART_INF_F;
    l_run[i] = 0.0f;
#pragma unroll
    for (int c = 0; c < DC; ++c) o[i][c] = 0.0f;
  }
  // last key any row of this tile may see
  int kv_end = p.kv_len;
  if (p.causal) {
    const int last = q0 + FF_BM - 1 + input_pos + 1;
    kv_end = last < kv_end ? last : kv_end;
  }
  for (int k0 = 0; k0 < kv_end; k0 += FF_BN) {
    __syncthreads();   // the previous tile's K, V and P are no longer read
    for (int i = tid; i < FF_BN * D; i += 256) {
      const int r = i / D, d = i % D;
      const bool in = k0 + r < p.kv_len;
      Kt[d * FF_LD + r] = in ? kb[(int64_t)(k0 + r) * p.ks1 + d] : 0.0f;
      Vs[r * D + d] = in ? vb[(int64_t)(k0 + r) * p.vs1 + d] : 0.0f;
    }
    __syncthreads();
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.0f;
#pragma unroll 8
    for (int d = 0; d < D; ++d) {
      const float4 qv = *reinterpret_cast<const float4*>(Qt + d * FF_LD + ty * 4);
      const float4 kv = *reinterpret_cast<const float4*>(Kt + d * FF_LD + tx * 4);
      const float qa[4] = {qv.x, qv.y, qv.z, qv.w}, ka[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = fmaf(qa[i], ka[j], s[i][j]);
    }
    float pr[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = q0 + ty * 4 + i;
      int lim = p.kv_len - 1;                       // last visible key of this row
      if (p.causal && row + input_pos < lim) lim = row + input_pos;
      float mx = -CUDART_INF_F;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = k0 + tx * 4 + j;
        s[i][j] = col <= lim ? s[i][j] * p.scale_log2 : -CUDART_INF_F;
        mx = fmaxf(mx, s[i][j]);
      }
#pragma unroll
      for (int off = 8; off >= 1; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float m_new = fmaxf(m_run[i], mx);
      const float m_use = m_new == -CUDART_INF_F ? 0.0f : m_new;   // nothing visible yet: keep the exponents finite
      const float alpha = exp2f(m_run[i] - m_use);                 // exp2(-inf) = 0 on the first visible tile
      float sum = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        pr[i][j] = exp2f(s[i][j] - m_use);
        sum += pr[i][j];
      }
#pragma unroll
      for (int off = 8; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      l_run[i] = l_run[i] * alpha + sum;
      m_run[i] = m_new;
#pragma unroll
      for (int c = 0; c < DC; ++c) o[i][c] *= alpha;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      *reinterpret_cast<float4*>(Pt + (tx * 4 + j) * FF_LD + ty * 4) = make_float4(pr[0][j], pr[1][j], pr[2][j], pr[3][j]);
    __syncthreads();
#pragma unroll 4
    for (int n = 0; n < FF_BN; ++n) {
      const float4 pv = *reinterpret_cast<const float4*>(Pt + n * FF_LD + ty * 4);
      const float pa[4] = {pv.x, pv.y, pv.z, pv.w};
      float va[DC];
      if constexpr (DC == 2) {
        const float2 v2 = *reinterpret_cast<const float2*>(Vs + n * D + tx * 2);
        va[0] = v2.x; va[1] = v2.y;
      } else {
#pragma unroll
        for (int c4 = 0; c4 < DC / 4; ++c4) {
          const float4 v4 = *reinterpret_cast<const float4*>(Vs + n * D + c4 * 64 + tx * 4);
          va[c4 * 4] = v4.x; va[c4 * 4 + 1] = v4.y; va[c4 * 4 + 2] = v4.z; va[c4 * 4 + 3] = v4.w;
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < DC; ++c) o[i][c] = fmaf(pa[i], va[c], o[i][c]);
    }
  }
  // normalise and store: thread columns are tx * 2 + c (D = 32) or 64 (c / 4) + 4 tx + c % 4
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = q0 + ty * 4 + i;
    if (row >= p.q_len) continue;
    const float inv = 1.0f / fmaxf(l_run[i], 1e-8f);   // cutile-kernels/src/attention.rs:385-390
    float* orow = ob + (int64_t)row * p.os1;
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      const int col = DC == 2 ? tx * 2 + c : (c >> 2) * 64 + tx * 4 + (c & 3);
      orow[col] = o[i][c] * inv;
    }
  }
}

template <int D>
static int launch_fmha_f32(const FmhaF32Params& p, int batch, cudaStream_t stream) {
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  constexpr int bytes = FmhaF32Smem<D>::FLOATS * (int)sizeof(float);
  auto kern = fmha_f32_kernel<D>;
  static b200h::DeviceOnce attr_done;
  if (!attr_done.test(di->ordinal)) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    attr_done.set(di->ordinal);
  }
  const dim3 grid((p.q_len + FF_BM - 1) / FF_BM, batch * p.heads, 1);
  kern<<<grid, 256, bytes, stream>>>(p);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

}  // namespace b200

int b200_fmha_f32_dispatch(int head_dim, const void* q, const void* k, const void* v, void* out, int batch, int heads,
                           int heads_kv, int q_len, int kv_len, const int64_t* qs, const int64_t* ks,
                           const int64_t* vs, const int64_t* os, float qk_scale, int causal, int input_pos,
                           const uint32_t* pos_ptr, cudaStream_t stream) {
  using namespace b200;
  if ((long long)batch * heads > 65535)
    return b200h::set_error(B200_ERR_UNSUPPORTED, "fmha(f32): batch * heads (%lld) exceeds 65535", (long long)batch * heads);
  FmhaF32Params p;
  p.q = static_cast<const float*>(q);
  p.k = static_cast<const float*>(k);
  p.v = static_cast<const float*>(v);
  p.out = static_cast<float*>(out);
  p.heads = heads; p.heads_kv = heads_kv; p.q_len = q_len; p.kv_len = kv_len;
  p.qs0 = qs[0]; p.qs1 = qs[1]; p.ks0 = ks[0]; p.ks1 = ks[1];
  p.vs0 = vs[0]; p.vs1 = vs[1]; p.os0 = os[0]; p.os1 = os[1];
  p.scale_log2 = qk_scale * 1.4426950408889634f;   // exp(x) = exp2(x log2 e), as the reference folds it into the scale
  p.causal = causal; p.input_pos = input_pos; p.pos_ptr = pos_ptr;
  if (head_dim == 32) return launch_fmha_f32<32>(p, batch, stream);
  if (head_dim == 64) return launch_fmha_f32<64>(p, batch, stream);
  if (head_dim == 128) return launch_fmha_f32<128>(p, batch, stream);
  return b200h::set_error(B200_ERR_UNSUPPORTED, "fmha(f32): head_dim %d has no precompiled configuration (32, 64, 128)",
                          head_dim);
}
