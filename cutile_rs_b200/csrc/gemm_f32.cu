// Exact-fp32 GEMM:  C[b] (+)= A[b] * B[b]  with every product and sum rounded separately and the
// K loop walked in ascending order per output element.  That is the arithmetic of the
// reference's host check `cpu_gemm` (cutile-examples/examples/persistent_gemm.rs:140-152:
// `acc += x[row*k+inner] * y[inner*n+col]`, no fused multiply-add), so results are bit-identical
// to it.  This is the correctness configuration (f32, 512^3) and the f32 path of `gemm`,
// `gemm_persistent` and `batch_matmul`; it is CUDA-core work by design (TF32 tensor cores would
// not reproduce fp32 results).
#include "host_common.h"

namespace b200 {

constexpr int F32_BN = 64, F32_BK = 32;

// BM x 64 output tile, 4 x 4 outputs per thread (BM / 4 x 16 threads).  The next k-slab travels from global memory into
// registers while the current one is multiplied out of shared memory, and the 64-row tile gives way to a 32-row one
// when it would leave most SMs without a CTA (512^3: 64 tiles of 64 x 64 on 148 SMs took 58 us, a chain of 32
// unhidden global-memory round trips; 128 tiles of 32 x 64 with the prefetch take a quarter of that).
template <int BM>
__global__ void __launch_bounds__(BM * 4)
gemm_f32_exact_kernel(const float* __restrict__ A, const float* __restrict__ B,
                      float* __restrict__ C, int M, int N, int K, int64_t lda, int64_t ldb,
                      int64_t ldc, int64_t sa, int64_t sb, int64_t sc, int accumulate,
                      int tiles_n) {
  constexpr int THREADS = BM * 4;
  constexpr int A_PER = BM * F32_BK / THREADS;       // 8
  constexpr int B_PER = F32_BK * F32_BN / THREADS;   // 16 or 8
  __shared__ __align__(16) float As[F32_BK][BM + 4];  // transposed: As[k][m]
  __shared__ __align__(16) float Bs[F32_BK][F32_BN + 4];
  const int batch = blockIdx.y;
  const int tm = blockIdx.x / tiles_n, tn = blockIdx.x % tiles_n;
  A += batch * sa;
  B += batch * sb;
  C += batch * sc;
  const int m0 = tm * BM, n0 = tn * F32_BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 columns of threads, 4 x 4 outputs each

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = m0 + ty * 4 + i, c = n0 + tx * 4 + j;
      acc[i][j] = (accumulate && r < M && c < N) ? C[r * ldc + c] : 0.0f;
    }

  float ra[A_PER], rb[B_PER];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int e = 0; e < A_PER; ++e) {   // A slab: BM rows x 32 k
      const int idx = threadIdx.x + e * THREADS;
      const int gr = m0 + idx / F32_BK, gk = k0 + idx % F32_BK;
      ra[e] = (gr < M && gk < K) ? A[gr * lda + gk] : 0.0f;
    }
#pragma unroll
    for (int e = 0; e < B_PER; ++e) {   // B slab: 32 k x 64 columns
      const int idx = threadIdx.x + e * THREADS;
      const int gk = k0 + (idx >> 6), gc = n0 + (idx & 63);
      rb[e] = (gk < K && gc < N) ? B[gk * ldb + gc] : 0.0f;
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += F32_BK) {
#pragma unroll
    for (int e = 0; e < A_PER; ++e) {
      const int idx = threadIdx.x + e * THREADS;
      As[idx % F32_BK][idx / F32_BK] = ra[e];
    }
#pragma unroll
    for (int e = 0; e < B_PER; ++e) {
      const int idx = threadIdx.x + e * THREADS;
      Bs[idx >> 6][idx & 63] = rb[e];
    }
    __syncthreads();
    if (k0 + F32_BK < K) fetch(k0 + F32_BK);   // in flight while this slab is multiplied
    auto step = [&](int kk) {
      const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float a[4] = {av.x, av.y, av.z, av.w}, b[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], b[j]));
    };
    if (K - k0 >= F32_BK) {   // a whole slab: unrolled, so that the shared-memory loads run ahead of the arithmetic
#pragma unroll
      for (int kk = 0; kk < F32_BK; ++kk) step(kk);
    } else {
      for (int kk = 0; kk < K - k0; ++kk) step(kk);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = m0 + ty * 4 + i, c = n0 + tx * 4 + j;
      if (r < M && c < N) C[r * ldc + c] = acc[i][j];
    }
}

}  // namespace b200

int b200_gemm_f32_dispatch(const float* A, const float* B, float* C, int batch, int M, int N,
                           int K, int64_t lda, int64_t ldb, int64_t ldc, int64_t sa, int64_t sb,
                           int64_t sc, int accumulate, cudaStream_t stream) {
  using namespace b200;
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  if (batch > 65535)
    return b200h::set_error(B200_ERR_INVALID, "gemm(f32): batch %d exceeds 65535", batch);
  const int tiles_n = (N + F32_BN - 1) / F32_BN;
  const int64_t tiles64 = (int64_t)((M + 63) / 64) * tiles_n * batch;
  if (tiles64 < 2 * (int64_t)di->sm_count) {
    dim3 grid(((M + 31) / 32) * tiles_n, batch, 1);
    gemm_f32_exact_kernel<32><<<grid, 128, 0, stream>>>(A, B, C, M, N, K, lda, ldb, ldc, sa, sb, sc, accumulate, tiles_n);
  } else {
    dim3 grid(((M + 63) / 64) * tiles_n, batch, 1);
    gemm_f32_exact_kernel<64><<<grid, 256, 0, stream>>>(A, B, C, M, N, K, lda, ldb, ldc, sa, sb, sc, accumulate, tiles_n);
  }
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
