// Persistent 16-bit GEMM for sm_100a:  C[M,N] (+)= A[M,K] * B,  fp32 accumulation in TMEM.
//
// Replaces the machine code that the reference obtains by JIT-compiling its `gemm` /
// `gemm_persistent` DSL bodies (cutile-benchmarks/paper/sec5_exp1_safety_overhead/rust/gemm/
// src/main.rs:74-132, cutile-examples/examples/persistent_gemm.rs:26-58): one [BM,BN] output
// tile per persistent iteration, a K loop of tile MMAs, tiles visited in grouped-M order
// (main.rs:53-66).
//
// Structure of one CTA (192 threads, one CTA per SM):
//   warp 0      TMA producer: A and B k-slabs into a STAGES-deep shared-memory ring
//   warp 1      MMA issuer: tcgen05.mma kind::f16, two TMEM accumulator buffers
//   warps 2..5  epilogue: tcgen05.ld -> bf16/f16 -> swizzled smem -> TMA store
// The epilogue of tile i overlaps the main loop of tile i+1 through the two accumulator buffers.
// All waits are bounded; a wait that gives up records a status code and the CTA unwinds.
#include <cuda_fp16.h>

#include "host_common.h"
#include "sm100_ptx.cuh"

namespace b200 {

#ifdef B200TILE_TEST_HOOKS
// Test builds only (libb200tile_waittest.so, never the product library): when set, CTA 0 leaves the second
// k-slab of its first tile unloaded, so the MMA thread's wait for that stage runs out.  This is how the
// bounded-wait path is exercised without faulting, trapping or hanging anything.
__device__ int g_test_skip_stage;
#endif

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;  // 64 x 2 bytes = one 128-byte swizzle row
constexpr int GEMM_THREADS = 192;

template <int BN>
struct GemmSmem {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;  // 16 KiB
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int C_WARP_BYTES = 32 * 128;  // 32 rows x 64 columns of 16-bit
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_C = OFF_B + STAGES * B_BYTES;
  static constexpr int OFF_BAR = OFF_C + 4 * 2 * C_WARP_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
  static constexpr int TOTAL = OFF_MISC + 16 + 1024;  // + alignment slack
};

// Grouped-M tile order: bands of `group_m` tile rows are walked column by column.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_m,
                                            int& bm, int& bn) {
  const int in_group = group_m * tiles_n;
  const int group = tile / in_group;
  const int first_m = group * group_m;
  const int rem = tiles_m - first_m;
  const int gsz = rem < group_m ? rem : group_m;
  bm = first_m + (tile % gsz);
  bn = (tile % in_group) / gsz;
}

// silu(gate) * up on values that first pass through the 16-bit type, as they would between the GEMM
// and the pointwise kernel: y = gate / (1 + exp(-gate)) * up in fp32 (pointwise.rs:66-74).
template <bool OUT_F16>
__device__ __forceinline__ float swiglu_16bit(float gate, float up) {
  const uint32_t packed = OUT_F16 ? pack_f16x2(gate, up) : pack_bf16x2(gate, up);
  float g, u;
  if (OUT_F16) {
    asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %2; cvt.f32.f16 %0, lo; cvt.f32.f16 %1, hi;}"
        : "=f"(g), "=f"(u) : "r"(packed));
  } else {
    g = __uint_as_float(packed << 16);
    u = __uint_as_float(packed & 0xffff0000u);
  }
  const float sig = __fdividef(1.0f, 1.0f + __expf(-g));
  return sig * g * u;
}

// B_KMAJOR = false: B is [K,N] row-major (the reference GEMM layout; N-major operand)
// B_KMAJOR = true : B is [N,K] row-major (the reference `linear_tile` layout; K-major operand)
// OUT_F16 selects f16 instead of bf16 for the 16-bit output pack.
// SWIGLU (BN = 256, K-major B only): B is [2N, K] = N gate rows followed by N up rows; a tile takes 128
// rows of each as one 256-row operand, so accumulator columns [0,128) hold x.gate^T and [128,256)
// x.up^T for the same 128 output columns, and the epilogue stores silu(gate) * up -- the GEMM and
// `silu_mul_2d_f16` (cutile-kernels/src/pointwise.rs:50-77) in one pass, with gate and up rounded to
// the 16-bit type in between exactly as the two-kernel sequence does.
// EPI (K-major B only): the linear layer's additive epilogue.  `bias` [N] (or null) is added to the fp32
// accumulator before the result is rounded to the 16-bit type; `residual` [M, N] (or null) is then added the way
// `add_2d_f16` (cutile-kernels/src/pointwise.rs:20-36) adds two 16-bit tensors: both operands in their 16-bit
// form, one fp32 sum, one rounding -- so "linear, then add_2d_f16" and this epilogue give the same bits.
struct EpiArgs {
  const uint16_t* bias;
  const uint16_t* residual;
  int64_t ld_res;
};

template <bool OUT_F16>
__device__ __forceinline__ float round_trip_16(float x) {
  if (OUT_F16) return __half2float(__float2half_rn(x));
  return __uint_as_float(pack_bf16x2(x, 0.0f) << 16);
}
template <bool OUT_F16>
__device__ __forceinline__ float from_16(uint16_t h) {
  if (OUT_F16) return __half2float(__ushort_as_half(h));
  return __uint_as_float((uint32_t)h << 16);
}

template <int BN, bool B_KMAJOR, bool OUT_F16, bool SWIGLU = false, bool EPI = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, int M, int N, int K, int group_m,
               uint32_t idesc, uint32_t* status, EpiArgs epi) {
  static_assert(!EPI || (B_KMAJOR && !SWIGLU), "the additive epilogue belongs to the NT linear layer");
  static_assert(!SWIGLU || (BN == 256 && B_KMAJOR), "the fused SwiGLU epilogue pairs two 128-row K-major B blocks");
  constexpr int BN_OUT = SWIGLU ? BN / 2 : BN;   // output columns per tile
  using L = GemmSmem<BN>;
  constexpr int STAGES = L::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));

  const uint32_t sA = base + L::OFF_A;
  const uint32_t sB = base + L::OFF_B;
  const uint32_t sC = base + L::OFF_C;
  const uint32_t bar_full = base + L::OFF_BAR;
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_tfull = bar_empty + STAGES * 8;
  const uint32_t bar_tempty = bar_tfull + 2 * 8;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(gen_base + L::OFF_MISC);
  // misc[0] = TMEM base address, misc[1] = abort flag

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  WaitCtx wctx{misc + 1, status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + b * 8, 1);
      mbar_init(bar_tempty + b * 8, 4);
    }
    misc[1] = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(misc)), 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = misc[0];

  const int tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
  const int tiles_n = (N + BN_OUT - 1) / BN_OUT;
  const int total_tiles = tiles_m * tiles_n;
  const int num_kb = (K + GEMM_BK - 1) / GEMM_BK;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int bm, bn;
        tile_coords(tile, tiles_m, tiles_n, group_m, bm, bn);
        const int m0 = bm * GEMM_BM, n0 = bn * BN_OUT;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(wctx, bar_empty + stage * 8, phase ^ 1, 1)) { ok = false; break; }
#ifdef B200TILE_TEST_HOOKS
          if (g_test_skip_stage && blockIdx.x == 0 && tile == 0 && kb == 1) {
            ok = false;   // the producer stops here: this stage's barrier is never armed, and the only
            break;        // wait left to run out is the MMA thread's (one deterministic wait site)
          }
#endif
          const uint32_t full = bar_full + stage * 8;
          mbar_expect_tx(full, L::A_BYTES + L::B_BYTES);
          tma_load_2d(sA + stage * L::A_BYTES, &tmA, full, kb * GEMM_BK, m0);
          if (SWIGLU) {
            // 128 gate rows, then the 128 up rows that belong to the same output columns
            tma_load_2d(sB + stage * L::B_BYTES, &tmB, full, kb * GEMM_BK, n0);
            tma_load_2d(sB + stage * L::B_BYTES + BN_OUT * 128, &tmB, full, kb * GEMM_BK, N + n0);
          } else if (B_KMAJOR) {
            tma_load_2d(sB + stage * L::B_BYTES, &tmB, full, kb * GEMM_BK, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sB + stage * L::B_BYTES + j * (GEMM_BK * 128), &tmB, full, n0 + j * 64,
                          kb * GEMM_BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer --------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
        const uint32_t buf = it & 1;
        if (!mbar_wait(wctx, bar_tempty + buf * 8, ((it >> 1) & 1) ^ 1, 2)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(wctx, bar_full + stage * 8, phase, 3)) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t adesc = make_smem_desc(sA + stage * L::A_BYTES, 16, 1024, SWZ_128B);
          const uint64_t bdesc =
              B_KMAJOR ? make_smem_desc(sB + stage * L::B_BYTES, 16, 1024, SWZ_128B)
                       : make_smem_desc(sB + stage * L::B_BYTES, GEMM_BK * 128, 1024, SWZ_128B);
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            // K-major operands advance 32 bytes inside the swizzled row per K=16 step;
            // the N-major B operand advances two 8-row groups (2 x 1024 bytes).
            const uint64_t a_k = adesc + (uint64_t)(k * 2);
            const uint64_t b_k = bdesc + (uint64_t)(B_KMAJOR ? k * 2 : k * 128);
            umma_f16_ss(d_tmem, a_k, b_k, idesc, (kb | k) != 0);
          }
          umma_commit(bar_empty + stage * 8);  // frees the smem stage when the MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(bar_tfull + buf * 8);  // accumulator complete
      }
    }
  } else {
    // -------------------------------- epilogue ---------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const uint32_t sCw = sC + q * (2 * L::C_WARP_BYTES);
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
      int bm, bn;
      tile_coords(tile, tiles_m, tiles_n, group_m, bm, bn);
      const int m0 = bm * GEMM_BM, n0 = bn * BN_OUT;
      const uint32_t buf = it & 1;
      if (!mbar_wait(wctx, bar_tfull + buf * 8, (it >> 1) & 1, 4)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN_OUT / 64; ++c) {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(t_row + c * 64, v0);
        tmem_ld_32x32b_x32(t_row + c * 64 + 32, v1);
        if (SWIGLU) {
          uint32_t u0[32], u1[32];
          tmem_ld_32x32b_x32(t_row + BN_OUT + c * 64, u0);
          tmem_ld_32x32b_x32(t_row + BN_OUT + c * 64 + 32, u1);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            v0[i] = __float_as_uint(swiglu_16bit<OUT_F16>(__uint_as_float(v0[i]), __uint_as_float(u0[i])));
            v1[i] = __float_as_uint(swiglu_16bit<OUT_F16>(__uint_as_float(v1[i]), __uint_as_float(u1[i])));
          }
        }
        // staging buffer (c & 1): the store issued two chunks ago must have drained it.  Chunk parity is a
        // valid choice only because every tile stores an even number of chunks; a variant with an odd
        // count must pick the buffer by a count of committed stores instead.
        static_assert((BN_OUT / 64) % 2 == 0, "chunk-parity staging needs an even number of chunks per tile");
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        tmem_wait_ld();
        if (EPI) {
          const int col0 = n0 + c * 64;
          const int row_g = m0 + q * 32 + lane;
          if (epi.bias) {
#pragma unroll
            for (int i = 0; i < 64; i += 8) {
              uint16_t b8[8];
              if (col0 + i + 8 <= N) {
                *reinterpret_cast<uint4*>(b8) = __ldg(reinterpret_cast<const uint4*>(epi.bias + col0 + i));
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) b8[e] = col0 + i + e < N ? __ldg(epi.bias + col0 + i + e) : (uint16_t)0;
              }
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                uint32_t& dst = (i + e < 32) ? v0[(i + e) & 31] : v1[(i + e) & 31];
                dst = __float_as_uint(__uint_as_float(dst) + from_16<OUT_F16>(b8[e]));
              }
            }
          }
          if (epi.residual && row_g < M) {
            const uint16_t* rrow = epi.residual + (int64_t)row_g * epi.ld_res + col0;
#pragma unroll
            for (int i = 0; i < 64; i += 8) {
              uint16_t r8[8];
              // plain (coherent) loads: `out` may alias `residual`, so the data is not read-only for the kernel
              if (col0 + i + 8 <= N) {
                *reinterpret_cast<uint4*>(r8) = *reinterpret_cast<const uint4*>(rrow + i);
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) r8[e] = col0 + i + e < N ? rrow[i + e] : (uint16_t)0;
              }
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                uint32_t& dst = (i + e < 32) ? v0[(i + e) & 31] : v1[(i + e) & 31];
                dst = __float_as_uint(round_trip_16<OUT_F16>(__uint_as_float(dst)) + from_16<OUT_F16>(r8[e]));
              }
            }
          }
        }
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
      // all TMEM reads of this accumulator are complete: hand it back to the MMA warp
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + buf * 8);
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ---------------------------------------------------------------------------
// Host launch
// ---------------------------------------------------------------------------
template <int BN, bool B_KMAJOR, bool OUT_F16>
static int launch_gemm_tc(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda,
                          int64_t ldb, int64_t ldc, int group_m, int max_ctas,
                          cudaStream_t stream) {
  using L = GemmSmem<BN>;
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  const CUtensorMapDataType dt =
      OUT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if ((rc = b200h::encode_tmap_2d(&tmA, dt, 2, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2,
                                  GEMM_BK, GEMM_BM, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  if (B_KMAJOR)
    rc = b200h::encode_tmap_2d(&tmB, dt, 2, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2,
                               GEMM_BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = b200h::encode_tmap_2d(&tmB, dt, 2, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64,
                               GEMM_BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  if ((rc = b200h::encode_tmap_2d(&tmC, dt, 2, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 2, 64,
                                  32, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;

  auto kern = gemm_tc_kernel<BN, B_KMAJOR, OUT_F16>;
  static b200h::DeviceOnce attr_done;
  if (!attr_done.test(di->ordinal)) {
    B200_CUDA_CHECK(
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    attr_done.set(di->ordinal);
  }
  const int tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + BN - 1) / BN);
  int grid = tiles < di->sm_count ? tiles : di->sm_count;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  const uint32_t fmt = OUT_F16 ? FMT_F16 : FMT_BF16;
  const uint32_t idesc = make_idesc(fmt, fmt, 0, B_KMAJOR ? 0 : 1, GEMM_BM, BN);
  kern<<<grid, GEMM_THREADS, L::TOTAL, stream>>>(tmA, tmB, tmC, M, N, K, group_m, idesc,
                                                 di->status, EpiArgs{nullptr, nullptr, 0});
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// out[M, N] = x . w^T (+ bias[N]) (+ residual[M, N]); x [M,K], w [N,K]: the NT linear layer with its additive epilogue
template <int BN, bool OUT_F16>
static int launch_gemm_epi(const void* X, const void* W, const void* bias, const void* residual, void* O, int M, int N,
                           int K, int64_t ldx, int64_t ldw, int64_t ld_res, int64_t ldo, cudaStream_t stream) {
  using L = GemmSmem<BN>;
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  const CUtensorMapDataType dt = OUT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if ((rc = b200h::encode_tmap_2d(&tmA, dt, 2, X, (uint64_t)K, (uint64_t)M, (uint64_t)ldx * 2, GEMM_BK, GEMM_BM,
                                  CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  if ((rc = b200h::encode_tmap_2d(&tmB, dt, 2, W, (uint64_t)K, (uint64_t)N, (uint64_t)ldw * 2, GEMM_BK, BN,
                                  CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  if ((rc = b200h::encode_tmap_2d(&tmC, dt, 2, O, (uint64_t)N, (uint64_t)M, (uint64_t)ldo * 2, 64, 32,
                                  CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  auto kern = gemm_tc_kernel<BN, true, OUT_F16, false, true>;
  static b200h::DeviceOnce attr_done;
  if (!attr_done.test(di->ordinal)) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    attr_done.set(di->ordinal);
  }
  const int tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + BN - 1) / BN);
  const int grid = tiles < di->sm_count ? tiles : di->sm_count;
  const uint32_t fmt = OUT_F16 ? FMT_F16 : FMT_BF16;
  const uint32_t idesc = make_idesc(fmt, fmt, 0, 0, GEMM_BM, BN);
  EpiArgs epi{static_cast<const uint16_t*>(bias), static_cast<const uint16_t*>(residual), ld_res};
  kern<<<grid, GEMM_THREADS, L::TOTAL, stream>>>(tmA, tmB, tmC, M, N, K, 8, idesc, di->status, epi);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// out[M, I] = silu(x . w[0:I]^T) * (x . w[I:2I]^T), x [M,K], w [2I,K] (gate rows, then up rows)
template <bool OUT_F16>
static int launch_gemm_swiglu(const void* X, const void* W, void* O, int M, int I, int K, int64_t ldx, int64_t ldw,
                              int64_t ldo, cudaStream_t stream) {
  using L = GemmSmem<256>;
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  const CUtensorMapDataType dt = OUT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if ((rc = b200h::encode_tmap_2d(&tmA, dt, 2, X, (uint64_t)K, (uint64_t)M, (uint64_t)ldx * 2, GEMM_BK, GEMM_BM,
                                  CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  if ((rc = b200h::encode_tmap_2d(&tmB, dt, 2, W, (uint64_t)K, (uint64_t)2 * I, (uint64_t)ldw * 2, GEMM_BK, 128,
                                  CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  if ((rc = b200h::encode_tmap_2d(&tmC, dt, 2, O, (uint64_t)I, (uint64_t)M, (uint64_t)ldo * 2, 64, 32,
                                  CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  auto kern = gemm_tc_kernel<256, true, OUT_F16, true>;
  static b200h::DeviceOnce attr_done;
  if (!attr_done.test(di->ordinal)) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    attr_done.set(di->ordinal);
  }
  const int tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((I + 127) / 128);
  const int grid = tiles < di->sm_count ? tiles : di->sm_count;
  const uint32_t fmt = OUT_F16 ? FMT_F16 : FMT_BF16;
  const uint32_t idesc = make_idesc(fmt, fmt, 0, 0, GEMM_BM, 256);
  kern<<<grid, GEMM_THREADS, L::TOTAL, stream>>>(tmA, tmB, tmC, M, I, K, 8, idesc, di->status,
                                                 EpiArgs{nullptr, nullptr, 0});
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

}  // namespace b200

// dtype: 0 = bf16, 1 = f16.  b_kmajor: 0 = B[K,N] row-major, 1 = B[N,K] row-major.
// config: 0 = 128x256x64, 1 = 128x128x64.
int b200_gemm_tc_dispatch(int dtype, int b_kmajor, int config, const void* A, const void* B,
                          void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                          int group_m, int max_ctas, cudaStream_t stream) {
  using namespace b200;
#define B200_GEMM_CASE(BN_, KM_, F16_)                                                        \
  return launch_gemm_tc<BN_, KM_, F16_>(A, B, C, M, N, K, lda, ldb, ldc, group_m, max_ctas, \
                                        stream)
  if (config == 0) {
    if (!b_kmajor && dtype == 0) B200_GEMM_CASE(256, false, false);
    if (!b_kmajor && dtype == 1) B200_GEMM_CASE(256, false, true);
    if (b_kmajor && dtype == 0) B200_GEMM_CASE(256, true, false);
    if (b_kmajor && dtype == 1) B200_GEMM_CASE(256, true, true);
  } else if (config == 1) {
    if (!b_kmajor && dtype == 0) B200_GEMM_CASE(128, false, false);
    if (!b_kmajor && dtype == 1) B200_GEMM_CASE(128, false, true);
    if (b_kmajor && dtype == 0) B200_GEMM_CASE(128, true, false);
    if (b_kmajor && dtype == 1) B200_GEMM_CASE(128, true, true);
  }
#undef B200_GEMM_CASE
  return b200h::set_error(B200_ERR_UNSUPPORTED, "gemm: no kernel for dtype %d / config %d", dtype,
                          config);
}

// dtype: 0 = bf16, 1 = f16.
int b200_gemm_swiglu_dispatch(int dtype, const void* X, const void* W, void* O, int M, int I, int K, int64_t ldx,
                              int64_t ldw, int64_t ldo, cudaStream_t stream) {
  using namespace b200;
  return dtype ? launch_gemm_swiglu<true>(X, W, O, M, I, K, ldx, ldw, ldo, stream)
               : launch_gemm_swiglu<false>(X, W, O, M, I, K, ldx, ldw, ldo, stream);
}

// dtype: 0 = bf16, 1 = f16.  Small problems take 128-column tiles (more CTAs), the rest 256-column ones.
int b200_gemm_epilogue_dispatch(int dtype, const void* X, const void* W, const void* bias, const void* residual,
                                void* O, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ld_res, int64_t ldo,
                                cudaStream_t stream) {
  using namespace b200;
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  const long long tiles256 = (long long)((M + GEMM_BM - 1) / GEMM_BM) * ((N + 255) / 256);
  const bool narrow = tiles256 < di->sm_count;
  if (narrow)
    return dtype ? launch_gemm_epi<128, true>(X, W, bias, residual, O, M, N, K, ldx, ldw, ld_res, ldo, stream)
                 : launch_gemm_epi<128, false>(X, W, bias, residual, O, M, N, K, ldx, ldw, ld_res, ldo, stream);
  return dtype ? launch_gemm_epi<256, true>(X, W, bias, residual, O, M, N, K, ldx, ldw, ld_res, ldo, stream)
               : launch_gemm_epi<256, false>(X, W, bias, residual, O, M, N, K, ldx, ldw, ld_res, ldo, stream);
}

#ifdef B200TILE_TEST_HOOKS
int b200_test_set_skip_stage(int on) {
  return cudaMemcpyToSymbol(b200::g_test_skip_stage, &on, sizeof(int)) != cudaSuccess;
}
#endif
