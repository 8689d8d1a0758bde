// 16-bit GEMM on CTA PAIRS:  one 256x256 output tile per pair of SMs, tcgen05.mma cta_group::2.
//
// Same contract and reference as gemm_tc.cu (the `gemm_persistent` body with
// `num_cta_in_cga = 2`, tile 256x256x64, grouped-M 8 -- the configuration behind the reference's
// published B200 number, cutile-benchmarks/paper/sec5_exp1_safety_overhead/README.md:146-153).
// Each CTA of a pair loads its own 128 rows of A and its own 128 columns of B (every load has one
// destination CTA); the pair's leader issues 256x256x16 MMAs that read both CTAs' shared memory
// and write 128 accumulator rows into each CTA's Tensor Memory.  Halving the B operand per SM is
// what relieves shared-memory bandwidth compared with the single-CTA 128x256 tile.
//
//   warp 0      TMA producer (both CTAs); transaction bytes are counted on the leader's barrier
//   warp 1      MMA issuer (leader CTA only) -- releases a stage in BOTH CTAs with two commits
//   warps 2..5  epilogue of this CTA's 128 rows x 256 columns
#include "host_common.h"
#include "sm100_ptx.cuh"

namespace b200 {

constexpr int P_BM = 128;   // rows per CTA (256 per pair)
constexpr int P_BN = 256;   // columns per pair (128 loaded per CTA)
#ifndef B200_PAIR_BK
#define B200_PAIR_BK 128
#endif
constexpr int P_BK = B200_PAIR_BK;  // 128: two 128-byte swizzle rows per stage, 8 MMAs per pair of commits
constexpr int P_KH = P_BK / 64;  // 64-wide (128-byte) sub-blocks per stage
constexpr int P_THREADS = 192;
constexpr int P_STAGES = 384 / P_BK;  // 192 KiB of operand ring per CTA

struct PairSmem {
  static constexpr int A_BYTES = P_BM * P_BK * 2;        // 16 KiB
  static constexpr int B_BYTES = (P_BN / 2) * P_BK * 2;  // 16 KiB
  static constexpr int C_WARP_BYTES = 32 * 128;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + P_STAGES * A_BYTES;
  static constexpr int OFF_C = OFF_B + P_STAGES * B_BYTES;
  static constexpr int OFF_BAR = OFF_C + 4 * 2 * C_WARP_BYTES;
  static constexpr int NUM_BARS = 2 * P_STAGES + 4;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
  static constexpr int TOTAL = OFF_MISC + 16 + 1024;
};

__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int group_m,
                                                 int& bm, int& bn) {
  const int in_group = group_m * tiles_n;
  const int group = tile / in_group;
  const int first_m = group * group_m;
  const int rem = tiles_m - first_m;
  const int gsz = rem < group_m ? rem : group_m;
  bm = first_m + (tile % gsz);
  bn = (tile % in_group) / gsz;
}

template <bool B_KMAJOR, bool OUT_F16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, int M, int N, int K, int group_m,
                    uint32_t idesc, uint32_t* status) {
  using L = PairSmem;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sA = base + L::OFF_A;
  const uint32_t sB = base + L::OFF_B;
  const uint32_t sC = base + L::OFF_C;
  const uint32_t bar_full = base + L::OFF_BAR;              // meaningful in the leader only
  const uint32_t bar_empty = bar_full + P_STAGES * 8;       // one set per CTA
  const uint32_t bar_tfull = bar_empty + P_STAGES * 8;      // one set per CTA
  const uint32_t bar_tempty = bar_tfull + 2 * 8;            // meaningful in the leader only
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(gen_base + L::OFF_MISC);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  WaitCtx wctx{misc + 1, status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(bar_full + s * 8, 1);   // leader's producer arrives once with both CTAs' bytes
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + b * 8, 1);
      mbar_init(bar_tempty + b * 8, 8);  // four epilogue warps from each CTA of the pair
    }
    misc[1] = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc_2cta(smem_u32(const_cast<uint32_t*>(misc)), 512);
    tmem_relinquish_2cta();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = misc[0];

  const int tiles_m = (M + 2 * P_BM - 1) / (2 * P_BM);
  const int tiles_n = (N + P_BN - 1) / P_BN;
  const int total_tiles = tiles_m * tiles_n;
  const int num_kb = (K + P_BK - 1) / P_BK;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += num_pairs) {
        int bm, bn;
        pair_tile_coords(tile, tiles_m, tiles_n, group_m, bm, bn);
        const int m0 = bm * (2 * P_BM) + (int)rank * P_BM;
        const int n0 = bn * P_BN + (int)rank * (P_BN / 2);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(wctx, bar_empty + stage * 8, phase ^ 1, 1)) { ok = false; break; }
          const uint32_t full_leader = mapa_u32(bar_full + stage * 8, 0);
          if (leader) mbar_expect_tx(bar_full + stage * 8, 2 * (L::A_BYTES + L::B_BYTES));
          // A (and a K-major B): one [128 rows][128 B] box per 64-wide k sub-block
#pragma unroll
          for (int h = 0; h < P_KH; ++h)
            tma_load_2d_pair(sA + stage * L::A_BYTES + h * (P_BM * 128), &tmA, full_leader,
                             kb * P_BK + h * 64, m0);
          if (B_KMAJOR) {
#pragma unroll
            for (int h = 0; h < P_KH; ++h)
              tma_load_2d_pair(sB + stage * L::B_BYTES + h * ((P_BN / 2) * 128), &tmB, full_leader,
                               kb * P_BK + h * 64, n0);
          } else {
            // N-major B: one [P_BK k-rows][64 columns] box per 64-column chunk
#pragma unroll
            for (int j = 0; j < P_BN / 2 / 64; ++j)
              tma_load_2d_pair(sB + stage * L::B_BYTES + j * (P_BK * 128), &tmB, full_leader,
                               n0 + j * 64, kb * P_BK);
          }
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // --------------------------- MMA issuer (leader) ---------------------------
    if (leader && lane == 0) {
      uint32_t stage = 0, phase = 0, it = 0;
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += num_pairs, ++it) {
        const uint32_t buf = it & 1;
        if (!mbar_wait(wctx, bar_tempty + buf * 8, ((it >> 1) & 1) ^ 1, 2)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * P_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(wctx, bar_full + stage * 8, phase, 3)) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t adesc = make_smem_desc(sA + stage * L::A_BYTES, 16, 1024, SWZ_128B);
          const uint64_t bdesc =
              B_KMAJOR ? make_smem_desc(sB + stage * L::B_BYTES, 16, 1024, SWZ_128B)
                       : make_smem_desc(sB + stage * L::B_BYTES, P_BK * 128, 1024, SWZ_128B);
#pragma unroll
          for (int k = 0; k < P_BK / 16; ++k) {
            // K-major operands: 32 bytes per step inside a 64-wide sub-block, next sub-block one
            // [rows][128 B] slab further; N-major B: two 8-row groups (2 x 1024 bytes) per step
            const uint32_t kmaj_a = (uint32_t)((k & 3) * 2 + (k >> 2) * ((P_BM * 128) >> 4));
            const uint32_t kmaj_b = (uint32_t)((k & 3) * 2 + (k >> 2) * (((P_BN / 2) * 128) >> 4));
            const uint64_t a_k = adesc + (uint64_t)kmaj_a;
            const uint64_t b_k = bdesc + (uint64_t)(B_KMAJOR ? kmaj_b : (uint32_t)(k * 128));
            umma_f16_ss_2cta(d_tmem, a_k, b_k, idesc, (kb | k) != 0);
          }
          // free this stage in both CTAs once the MMAs have read it
          umma_commit_2cta(bar_empty + stage * 8);
          umma_commit_2cta(mapa_u32(bar_empty + stage * 8, 1));
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          umma_commit_2cta(bar_tfull + buf * 8);
          umma_commit_2cta(mapa_u32(bar_tfull + buf * 8, 1));
        }
      }
    }
  } else {
    // -------------------------------- epilogue ---------------------------------
    const int q = warp & 3;
    const uint32_t sCw = sC + q * (2 * L::C_WARP_BYTES);
    const uint32_t tempty_leader = mapa_u32(bar_tempty, 0);
    uint32_t it = 0;
    bool ok = true;
    for (int tile = pair; tile < total_tiles && ok; tile += num_pairs, ++it) {
      int bm, bn;
      pair_tile_coords(tile, tiles_m, tiles_n, group_m, bm, bn);
      const int m0 = bm * (2 * P_BM) + (int)rank * P_BM, n0 = bn * P_BN;
      const uint32_t buf = it & 1;
      if (!mbar_wait(wctx, bar_tfull + buf * 8, (it >> 1) & 1, 4)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + buf * P_BN;
#pragma unroll 1
      for (int c = 0; c < P_BN / 64; ++c) {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(t_row + c * 64, v0);
        tmem_ld_32x32b_x32(t_row + c * 64 + 32, v1);
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        tmem_wait_ld();
        const uint32_t sbuf = sCw + (c & 1) * L::C_WARP_BYTES;
        const uint32_t row_addr = sbuf + lane * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t* src = (j < 4) ? &v0[j * 8] : &v1[(j - 4) * 8];
          uint32_t p[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float lo = __uint_as_float(src[2 * e]), hi = __uint_as_float(src[2 * e + 1]);
            p[e] = OUT_F16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
          }
          const uint32_t dst = row_addr + ((uint32_t)(j ^ (lane & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(p[0]),
                       "r"(p[1]), "r"(p[2]), "r"(p[3])
                       : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&tmC, sbuf, n0 + c * 64, m0 + q * 32);
          tma_store_commit();
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster_addr(tempty_leader + buf * 8);
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while its partner may still touch its memory
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_2cta(tmem_base, 512);
  }
}

template <bool B_KMAJOR, bool OUT_F16>
static int launch_gemm_pair(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda,
                            int64_t ldb, int64_t ldc, int group_m, int max_ctas,
                            cudaStream_t stream) {
  using L = PairSmem;
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  const CUtensorMapDataType dt =
      OUT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if ((rc = b200h::encode_tmap_2d(&tmA, dt, 2, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, 64,
                                  P_BM, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  if (B_KMAJOR)
    rc = b200h::encode_tmap_2d(&tmB, dt, 2, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, 64,
                               P_BN / 2, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = b200h::encode_tmap_2d(&tmB, dt, 2, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64,
                               P_BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  if ((rc = b200h::encode_tmap_2d(&tmC, dt, 2, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 2, 64,
                                  32, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  auto kern = gemm_tc_pair_kernel<B_KMAJOR, OUT_F16>;
  static bool attr_done[64] = {};
  if (!attr_done[di->ordinal]) {
    B200_CUDA_CHECK(
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    attr_done[di->ordinal] = true;
  }
  const int tiles = ((M + 2 * P_BM - 1) / (2 * P_BM)) * ((N + P_BN - 1) / P_BN);
  int pairs = di->sm_count / 2;
  if (tiles < pairs) pairs = tiles;
  if (max_ctas > 0 && pairs > (max_ctas + 1) / 2) pairs = (max_ctas + 1) / 2;
  const uint32_t fmt = OUT_F16 ? FMT_F16 : FMT_BF16;
  const uint32_t idesc = make_idesc(fmt, fmt, 0, B_KMAJOR ? 0 : 1, 2 * P_BM, P_BN);
  kern<<<pairs * 2, P_THREADS, L::TOTAL, stream>>>(tmA, tmB, tmC, M, N, K, group_m, idesc,
                                                   di->status);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

}  // namespace b200

int b200_gemm_pair_dispatch(int dtype, int b_kmajor, const void* A, const void* B, void* C, int M,
                            int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int group_m,
                            int max_ctas, cudaStream_t stream) {
  using namespace b200;
  if (!b_kmajor && dtype == 0)
    return launch_gemm_pair<false, false>(A, B, C, M, N, K, lda, ldb, ldc, group_m, max_ctas, stream);
  if (!b_kmajor && dtype == 1)
    return launch_gemm_pair<false, true>(A, B, C, M, N, K, lda, ldb, ldc, group_m, max_ctas, stream);
  if (b_kmajor && dtype == 0)
    return launch_gemm_pair<true, false>(A, B, C, M, N, K, lda, ldb, ldc, group_m, max_ctas, stream);
  return launch_gemm_pair<true, true>(A, B, C, M, N, K, lda, ldb, ldc, group_m, max_ctas, stream);
}
