// FP8 (e4m3) GEMM with one fp32 scale per 1x128 block of A and per 128x128 block of B:
//   Z[M,N] = alpha * sum_kb  sa[m,kb] * sb[n/128,kb] * ( A_q[m, kb*128 : +128] . B_q[n, kb*128 : +128] )
// A_q is [M,K] and B_q is [N,K] (both K-major, the layout of the reference's scaled linear kernels,
// cutile-examples/examples/mxfp8.rs:25-33).  The reference itself only ships the MXFP8 form
// (E8M0 scale per 32, `mmaf_scaled`, cutile/src/_core.rs:2288-2313); fp32 scales per 128-block are
// not a hardware block-scale mode, so each 128-deep k-block is multiplied exactly on the tensor
// cores (tcgen05.mma kind::f8f6f4, fp32 accumulation in TMEM) and "promoted" on CUDA cores:
// partial * sa * sb is added into fp32 register accumulators.
//
//   warp 0       TMA producer: 128x128 A and 256x128 B byte tiles, 3-stage ring
//   warp 1       MMA issuer: 4 MMAs (128x256x32) per k-block into one of two TMEM partial buffers
//   warps 4..7   promotion + epilogue of output columns   0..127 of the tile
//   warps 8..11  promotion + epilogue of output columns 128..255 (its own B scale block)
#include "host_common.h"
#include "sm100_ptx.cuh"

namespace b200 {

constexpr int F8_BM = 128, F8_BN = 256, F8_BK = 128;
constexpr int F8_THREADS = 384;
constexpr int F8_STAGES = 4;
// Register re-balancing (setmaxnreg).  The pool a CTA can re-balance is what it was GIVEN AT LAUNCH (threads x
// the kernel's register count, 384 x 168 here), not the SM's 64 K registers: an increase that does not fit
// into what the decrease released waits forever.
constexpr int F8_PROMO_REGS = 216, F8_OTHER_REGS = 40;  // 128 x 40 + 256 x 216 = 60416 <= 384 x 168 = 64512

struct Fp8Smem {
  static constexpr int A_BYTES = F8_BM * F8_BK;  // 16 KiB
  static constexpr int B_BYTES = F8_BN * F8_BK;  // 32 KiB
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + F8_STAGES * A_BYTES;
  // bf16 output staging for TMA stores: one [32 rows][128 B] swizzled buffer per promotion warp (rows stored
  // straight from registers reach L2 as half-filled sectors from all CTAs at once and hold up the next tile's loads)
  static constexpr int OFF_C = OFF_B + F8_STAGES * B_BYTES;
  static constexpr int C_WARP_BYTES = 32 * 128;
  static constexpr int OFF_BAR = OFF_C + 8 * C_WARP_BYTES;
  static constexpr int NUM_BARS = 2 * F8_STAGES + 4;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
  static constexpr int TOTAL = OFF_MISC + 16 + 1024;
};

template <bool OUT_F32>
__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_blk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const float* __restrict__ sa, const float* __restrict__ sb, void* __restrict__ Z,
                    int M, int N, int K, int64_t ldz, int ld_sa, int ld_sb, float alpha, int group_m,
                    uint32_t idesc, uint32_t* status) {
  using L = Fp8Smem;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sA = base + L::OFF_A, sB = base + L::OFF_B;
  const uint32_t bar_full = base + L::OFF_BAR;
  const uint32_t bar_empty = bar_full + F8_STAGES * 8;
  const uint32_t bar_pfull = bar_empty + F8_STAGES * 8;
  const uint32_t bar_pempty = bar_pfull + 2 * 8;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(gen_base + L::OFF_MISC);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx wctx{misc + 1, status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < F8_STAGES; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_pfull + b * 8, 1);
      mbar_init(bar_pempty + b * 8, 8);
    }
    misc[1] = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (!OUT_F32) tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(misc)), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = misc[0];

  const int tiles_m = (M + F8_BM - 1) / F8_BM;
  const int tiles_n = (N + F8_BN - 1) / F8_BN;
  const int total_tiles = tiles_m * tiles_n;
  const int num_kb = K / F8_BK;
  auto tile_coords = [&](int tile, int& bm, int& bn) {
    const int in_group = group_m * tiles_n;
    const int group = tile / in_group;
    const int first_m = group * group_m;
    const int rem = tiles_m - first_m;
    const int gsz = rem < group_m ? rem : group_m;
    bm = first_m + (tile % gsz);
    bn = (tile % in_group) / gsz;
  };

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(F8_OTHER_REGS));
    if (warp == 0 && lane == 0) {
      // ------------------------------ TMA producer ------------------------------
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int bm, bn;
        tile_coords(tile, bm, bn);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(wctx, bar_empty + stage * 8, phase ^ 1, 1)) { ok = false; break; }
          const uint32_t full = bar_full + stage * 8;
          mbar_expect_tx(full, L::A_BYTES + L::B_BYTES);
          tma_load_2d(sA + stage * L::A_BYTES, &tmA, full, kb * F8_BK, bm * F8_BM);
          tma_load_2d(sB + stage * L::B_BYTES, &tmB, full, kb * F8_BK, bn * F8_BN);
          if (++stage == F8_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    } else if (warp == 1 && lane == 0) {
      // ------------------------------- MMA issuer --------------------------------
      uint32_t stage = 0, phase = 0, g = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb, ++g) {
          const uint32_t buf = g & 1;
          if (!mbar_wait(wctx, bar_pempty + buf * 8, ((g >> 1) & 1) ^ 1, 2)) { ok = false; break; }
          if (!mbar_wait(wctx, bar_full + stage * 8, phase, 3)) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t adesc = make_smem_desc(sA + stage * L::A_BYTES, 16, 1024, SWZ_128B);
          const uint64_t bdesc = make_smem_desc(sB + stage * L::B_BYTES, 16, 1024, SWZ_128B);
#pragma unroll
          for (int k = 0; k < F8_BK / 32; ++k)
            umma_f8f6f4_ss(tmem_base + buf * F8_BN, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2),
                           idesc, k != 0);
          umma_commit(bar_empty + stage * 8);
          umma_commit(bar_pfull + buf * 8);
          if (++stage == F8_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else {
    // ---------------------- promotion + epilogue warpgroups ----------------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(F8_PROMO_REGS));
    const int wg = (warp - 4) >> 2;  // which 128-column half of the tile
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16) + wg * 128;
    uint32_t g = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      int bm, bn;
      tile_coords(tile, bm, bn);
      const int row_g = bm * F8_BM + row;
      const int col0 = bn * F8_BN + wg * 128;
      const bool row_ok = row_g < M;
      const float* sa_row = sa + (int64_t)(row_ok ? row_g : 0) * ld_sa;
      const int nb = col0 / 128;
      const bool col_ok = col0 < N;
      const float* sb_row = sb + (int64_t)(col_ok ? nb : 0) * ld_sb;
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.0f;
      float s_next = __ldg(sa_row) * __ldg(sb_row);
      for (int kb = 0; kb < num_kb; ++kb, ++g) {
        const uint32_t buf = g & 1;
        const float s = s_next;
        if (kb + 1 < num_kb) s_next = __ldg(sa_row + kb + 1) * __ldg(sb_row + kb + 1);
        if (!mbar_wait(wctx, bar_pfull + buf * 8, (g >> 1) & 1, 4)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t t_src = t_lane + buf * F8_BN;
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(t_src, v0);
        tmem_wait_ld();
        tmem_ld_32x32b_x32(t_src + 32, v1);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = fmaf(s, __uint_as_float(v0[i]), acc[i]);
        tmem_wait_ld();
        tmem_ld_32x32b_x32(t_src + 64, v0);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[32 + i] = fmaf(s, __uint_as_float(v1[i]), acc[32 + i]);
        tmem_wait_ld();
        tmem_ld_32x32b_x32(t_src + 96, v1);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[64 + i] = fmaf(s, __uint_as_float(v0[i]), acc[64 + i]);
        tmem_wait_ld();
        // every TMEM read of this partial buffer is done: hand it back before the last FMAs
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_pempty + buf * 8);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[96 + i] = fmaf(s, __uint_as_float(v1[i]), acc[96 + i]);
      }
      if (!ok) break;
      if constexpr (!OUT_F32) {
        // epilogue: registers -> bf16 -> swizzled staging -> TMA store (which clips at M and N), 64 columns at a time
        const uint32_t sbuf = base + L::OFF_C + (uint32_t)(warp - 4) * L::C_WARP_BYTES;
        const uint32_t row_addr = sbuf + lane * 128;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (lane == 0) tma_store_wait_read<0>();   // the previous store has read the buffer
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float* a = acc + c * 64 + j * 8;
            const uint32_t dst = row_addr + ((uint32_t)(j ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst),
                         "r"(pack_bf16x2(a[0] * alpha, a[1] * alpha)), "r"(pack_bf16x2(a[2] * alpha, a[3] * alpha)),
                         "r"(pack_bf16x2(a[4] * alpha, a[5] * alpha)), "r"(pack_bf16x2(a[6] * alpha, a[7] * alpha))
                         : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmC, sbuf, col0 + c * 64, bm * F8_BM + q * 32);
            tma_store_commit();
          }
        }
      } else if (row_ok && col_ok) {
        // f32 output: one output row (128 contiguous columns) per thread, written straight to global
        if (OUT_F32) {
          float* zrow = static_cast<float*>(Z) + (int64_t)row_g * ldz + col0;
#pragma unroll
          for (int i = 0; i < 128; i += 4) {
            if (col0 + i + 3 < N) {
              *reinterpret_cast<float4*>(zrow + i) =
                  make_float4(acc[i] * alpha, acc[i + 1] * alpha, acc[i + 2] * alpha, acc[i + 3] * alpha);
            } else {
              for (int e = 0; e < 4; ++e)
                if (col0 + i + e < N) zrow[i + e] = acc[i + e] * alpha;
            }
          }
        } else {
          uint16_t* zrow = static_cast<uint16_t*>(Z) + (int64_t)row_g * ldz + col0;
#pragma unroll
          for (int i = 0; i < 128; i += 8) {
            if (col0 + i + 7 < N) {
              uint4 w;
              w.x = pack_bf16x2(acc[i] * alpha, acc[i + 1] * alpha);
              w.y = pack_bf16x2(acc[i + 2] * alpha, acc[i + 3] * alpha);
              w.z = pack_bf16x2(acc[i + 4] * alpha, acc[i + 5] * alpha);
              w.w = pack_bf16x2(acc[i + 6] * alpha, acc[i + 7] * alpha);
              *reinterpret_cast<uint4*>(zrow + i) = w;
            } else {
              for (int e = 0; e < 8; ++e)
                if (col0 + i + e < N) zrow[i + e] = (uint16_t)(pack_bf16x2(acc[i + e] * alpha, 0.0f) & 0xFFFF);
            }
          }
        }
      }
    }
    if (!OUT_F32 && lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <bool OUT_F32>
static int launch_fp8(const void* x, const void* y, const float* xs, const float* ys, void* z, int M,
                      int N, int K, int64_t ldx, int64_t ldy, int64_t ldz, int ld_xs, int ld_ys,
                      float alpha, cudaStream_t stream) {
  using L = Fp8Smem;
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  CUtensorMap tmA, tmB;
  int rc;
  if ((rc = b200h::encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x, (uint64_t)K, (uint64_t)M,
                                  (uint64_t)ldx, F8_BK, F8_BM, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  if ((rc = b200h::encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, y, (uint64_t)K, (uint64_t)N,
                                  (uint64_t)ldy, F8_BK, F8_BN, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  CUtensorMap tmC = tmA;   // read only by the bf16 instantiation
  if (!OUT_F32 && (rc = b200h::encode_tmap_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, z, (uint64_t)N, (uint64_t)M,
                                              (uint64_t)ldz * 2, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  auto kern = gemm_fp8_blk_kernel<OUT_F32>;
  static b200h::DeviceOnce attr_done;
  if (!attr_done.test(di->ordinal)) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    attr_done.set(di->ordinal);
  }
  const int tiles = ((M + F8_BM - 1) / F8_BM) * ((N + F8_BN - 1) / F8_BN);
  const int grid = tiles < di->sm_count ? tiles : di->sm_count;
  const uint32_t idesc = make_idesc(FMT_E4M3, FMT_E4M3, 0, 0, F8_BM, F8_BN);
  kern<<<grid, F8_THREADS, L::TOTAL, stream>>>(tmA, tmB, tmC, xs, ys, z, M, N, K, ldz, ld_xs, ld_ys, alpha, 8,
                                               idesc, di->status);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

}  // namespace b200

int b200_gemm_fp8_blk_dispatch(int out_f32, const void* x, const void* y, const float* xs,
                               const float* ys, void* z, int M, int N, int K, int64_t ldx, int64_t ldy,
                               int64_t ldz, int ld_xs, int ld_ys, float alpha, cudaStream_t stream) {
  return out_f32 ? b200::launch_fp8<true>(x, y, xs, ys, z, M, N, K, ldx, ldy, ldz, ld_xs, ld_ys, alpha,
                                          stream)
                 : b200::launch_fp8<false>(x, y, xs, ys, z, M, N, K, ldx, ldy, ldz, ld_xs, ld_ys, alpha,
                                           stream);
}
