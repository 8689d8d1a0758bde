// Exact-fp32 GEMM:  C[b] (+)= A[b] * B[b]  with every product and sum rounded separately and the
// K loop walked in ascending order per output element.  That is the arithmetic of the
// reference's host check `cpu_gemm` (cutile-examples/examples/persistent_gemm.rs:140-152:
// `acc += x[row*k+inner] * y[inner*n+col]`, no fused multiply-add), so results are bit-identical
// to it.  This is the correctness configuration (f32, 512^3) and the f32 path of `gemm`,
// `gemm_persistent` and `batch_matmul`; it is CUDA-core work by design (TF32 tensor cores would
// not reproduce fp32 results).
#include "host_common.h"

namespace b200 {

constexpr int F32_BM = 64, F32_BN = 64, F32_BK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_exact_kernel(const float* __restrict__ A, const float* __restrict__ B,
                      float* __restrict__ C, int M, int N, int K, int64_t lda, int64_t ldb,
                      int64_t ldc, int64_t sa, int64_t sb, int64_t sc, int accumulate,
                      int tiles_n) {
  __shared__ float As[F32_BK][F32_BM + 4];  // transposed: As[k][m]
  __shared__ float Bs[F32_BK][F32_BN + 4];
  const int batch = blockIdx.y;
  const int tm = blockIdx.x / tiles_n, tn = blockIdx.x % tiles_n;
  A += batch * sa;
  B += batch * sb;
  C += batch * sc;
  const int m0 = tm * F32_BM, n0 = tn * F32_BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4 x 4 outputs each

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = m0 + ty * 4 + i, c = n0 + tx * 4 + j;
      acc[i][j] = (accumulate && r < M && c < N) ? C[r * ldc + c] : 0.0f;
    }

  for (int k0 = 0; k0 < K; k0 += F32_BK) {
    // A tile: 64 rows x 16 k  (256 threads x 4 elements)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = threadIdx.x + e * 256;
      const int r = idx >> 4, kk = idx & 15;
      const int gr = m0 + r, gk = k0 + kk;
      As[kk][r] = (gr < M && gk < K) ? A[gr * lda + gk] : 0.0f;
    }
    // B tile: 16 k x 64 columns
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = threadIdx.x + e * 256;
      const int kk = idx >> 6, c = idx & 63;
      const int gk = k0 + kk, gc = n0 + c;
      Bs[kk][c] = (gk < K && gc < N) ? B[gk * ldb + gc] : 0.0f;
    }
    __syncthreads();
    const int kmax = (K - k0) < F32_BK ? (K - k0) : F32_BK;
    for (int kk = 0; kk < kmax; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], b[j]));
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
  if (!b200h::device_info()) return B200_ERR_CUDA;
  const int tiles_m = (M + F32_BM - 1) / F32_BM, tiles_n = (N + F32_BN - 1) / F32_BN;
  if (batch > 65535)
    return b200h::set_error(B200_ERR_INVALID, "gemm(f32): batch %d exceeds 65535", batch);
  dim3 grid(tiles_m * tiles_n, batch, 1);
  gemm_f32_exact_kernel<<<grid, 256, 0, stream>>>(A, B, C, M, N, K, lda, ldb, ldc, sa, sb, sc,
                                                  accumulate, tiles_n);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
