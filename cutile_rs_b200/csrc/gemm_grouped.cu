// Persistent grouped GEMM over per-group pointer and extent tables (MoE expert batches).
//
// Replaces `group_gemm_f16_nt_desc` (cutile-kernels/src/experimental/moe.rs:66-128): group g
// multiplies A_g [m_g, k_g] by B_g [k_g, n_g] into C_g [m_g, n_g], all row-major 16-bit; the
// pointers come from three device arrays of i64 and the extents from three device tables of
// eight i32 per group ({rows, cols, row stride, ...}, moe.rs:27-63).  Nothing about the groups is
// known on the host, so the work is split in two launches:
//
//   grouped_prepare_kernel   CTA 0: tile counts and their prefix sum; every warp of the grid: for one group three
//                            TMA descriptors made on the device from host-encoded templates
//                            (`tensormap.replace` in shared memory, published to the workspace with
//                            `tensormap.cp_fenceproxy`)
//   gemm_grouped_kernel      the persistent warp-specialised GEMM of gemm_tc.cu (TMA ring ->
//                            tcgen05.mma into two TMEM accumulators -> TMA-store epilogue) walking
//                            the concatenated tile list of all groups, tile t of the list going to
//                            CTA t mod grid like the reference's `tile_idx += NUM_SM`
#include "host_common.h"
#include "sm100_ptx.cuh"

namespace b200 {

constexpr int GG_BM = 128;
constexpr int GG_BK = 64;
constexpr int GG_THREADS = 192;
constexpr int GG_PREP_THREADS = 256;

// Workspace layout: descriptors first (128-byte records), then one int4 {m, n, k, first tile} per
// group and a closing record whose .w is the total tile count.
struct GroupedWs {
  CUtensorMap* desc;  // [groups][3]: A, B, C
  int4* info;         // [groups + 1]
};
__host__ __device__ inline size_t grouped_desc_bytes(int groups) { return (size_t)groups * 3 * 128; }
__host__ __device__ inline size_t grouped_ws_bytes(int groups) {
  return grouped_desc_bytes(groups) + (size_t)(groups + 1) * sizeof(int4);
}

__device__ __forceinline__ void tmap_replace_addr(uint32_t smem_desc, uint64_t addr) {
  asm volatile("tensormap.replace.tile.global_address.shared::cta.b1024.b64 [%0], %1;" ::"r"(smem_desc), "l"(addr)
               : "memory");
}
__device__ __forceinline__ void tmap_replace_dims(uint32_t smem_desc, uint32_t dim0, uint32_t dim1) {
  asm volatile("tensormap.replace.tile.global_dim.shared::cta.b1024.b32 [%0], 0, %1;" ::"r"(smem_desc), "r"(dim0)
               : "memory");
  asm volatile("tensormap.replace.tile.global_dim.shared::cta.b1024.b32 [%0], 1, %1;" ::"r"(smem_desc), "r"(dim1)
               : "memory");
}
// pitch of dimension 1 in bytes (a multiple of 16)
__device__ __forceinline__ void tmap_replace_stride(uint32_t smem_desc, uint64_t bytes) {
  asm volatile("tensormap.replace.tile.global_stride.shared::cta.b1024.b64 [%0], 0, %1;" ::"r"(smem_desc), "l"(bytes)
               : "memory");
}
// whole warp: copies the 128-byte record to global memory and releases it to the tensormap proxy
__device__ __forceinline__ void tmap_publish(void* gmem_desc, uint32_t smem_desc) {
  asm volatile(
      "tensormap.cp_fenceproxy.global.shared::cta.tensormap::generic.release.gpu.sync.aligned [%0], [%1], 128;"
      ::"l"(gmem_desc), "r"(smem_desc)
      : "memory");
}
__device__ __forceinline__ void tmap_acquire(const void* gmem_desc) {
  asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(gmem_desc) : "memory");
}

template <int BN>
__global__ void __launch_bounds__(GG_PREP_THREADS)
grouped_prepare_kernel(const __grid_constant__ CUtensorMap tplA, const __grid_constant__ CUtensorMap tplB,
                       const __grid_constant__ CUtensorMap tplC, const int64_t* a_ptrs, const int64_t* b_ptrs,
                       const int64_t* c_ptrs, const int32_t* a_metas, const int32_t* b_metas,
                       const int32_t* c_metas, int groups, GroupedWs ws) {
  __shared__ __align__(128) uint8_t s_desc[GG_PREP_THREADS / 32][3][128];
  __shared__ int s_warp_sum[GG_PREP_THREADS / 32];
  __shared__ int s_carry;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) s_carry = 0;
  __syncthreads();

  // ---- CTA 0: extents and the exclusive prefix sum of the tile counts ----
  if (blockIdx.x == 0) {
    for (int g0 = 0; g0 < groups; g0 += GG_PREP_THREADS) {
      const int g = g0 + tid;
      int m = 0, n = 0, k = 0, tiles = 0;
      if (g < groups) {
        m = a_metas[g * 8 + 0];
        k = a_metas[g * 8 + 1];
        n = b_metas[g * 8 + 1];
        if (m < 0) m = 0;
        if (n < 0) n = 0;
        if (k < 0) k = 0;
        tiles = ((m + GG_BM - 1) / GG_BM) * ((n + BN - 1) / BN);
      }
      int scan = tiles;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, scan, off);
        if (lane >= off) scan += v;
      }
      if (lane == 31) s_warp_sum[warp] = scan;
      __syncthreads();
      int before = s_carry;
      for (int w = 0; w < warp; ++w) before += s_warp_sum[w];
      if (g < groups) ws.info[g] = make_int4(m, n, k, before + scan - tiles);
      __syncthreads();
      if (tid == GG_PREP_THREADS - 1) s_carry = before + scan;
      __syncthreads();
    }
    if (tid == 0) ws.info[groups] = make_int4(0, 0, 0, s_carry);
  }

  // ---- descriptors: every warp of the grid builds ONE group's three records.  A warp's shared-memory
  // slot is written once and never reused, so nothing can overwrite a record that is still being
  // copied out (a loop that reused the slot produced corrupt descriptors now and then when there were
  // more groups than warps). ----
  const int g = blockIdx.x * (GG_PREP_THREADS / 32) + warp;
  if (g < groups) {
    const uint32_t sd = smem_u32(&s_desc[warp][0][0]);
    // templates -> shared memory, four bytes per lane and descriptor
    reinterpret_cast<uint32_t*>(&s_desc[warp][0][0])[lane] = reinterpret_cast<const uint32_t*>(&tplA)[lane];
    reinterpret_cast<uint32_t*>(&s_desc[warp][1][0])[lane] = reinterpret_cast<const uint32_t*>(&tplB)[lane];
    reinterpret_cast<uint32_t*>(&s_desc[warp][2][0])[lane] = reinterpret_cast<const uint32_t*>(&tplC)[lane];
    __syncwarp();
    if (lane == 0) {
      // extents of an empty group are never used by a copy; keep them legal for the descriptor
      const uint32_t m = max(a_metas[g * 8 + 0], 1), k = max(a_metas[g * 8 + 1], 1);
      const uint32_t n = max(b_metas[g * 8 + 1], 1);
      const uint64_t lda = (uint64_t)max(a_metas[g * 8 + 2], 8), ldb = (uint64_t)max(b_metas[g * 8 + 2], 8);
      const uint64_t ldc = (uint64_t)max(c_metas[g * 8 + 2], 8);
      tmap_replace_addr(sd, (uint64_t)a_ptrs[g]);
      tmap_replace_dims(sd, k, m);
      tmap_replace_stride(sd, lda * 2);
      tmap_replace_addr(sd + 128, (uint64_t)b_ptrs[g]);
      tmap_replace_dims(sd + 128, n, k);
      tmap_replace_stride(sd + 128, ldb * 2);
      tmap_replace_addr(sd + 256, (uint64_t)c_ptrs[g]);
      tmap_replace_dims(sd + 256, n, m);
      tmap_replace_stride(sd + 256, ldc * 2);
    }
    __syncwarp();
    tmap_publish(&ws.desc[g * 3 + 0], sd);
    tmap_publish(&ws.desc[g * 3 + 1], sd + 128);
    tmap_publish(&ws.desc[g * 3 + 2], sd + 256);
    __syncwarp();
  }
}

// Cursor over the concatenated tile list: advances to the group that holds `tile`.
struct GroupCursor {
  const int4* info;
  int groups;
  int g;
  int4 cur;      // {m, n, k, first tile}
  int next_first;
  __device__ GroupCursor(const int4* info_, int groups_) : info(info_), groups(groups_), g(0) {
    cur = __ldg(info);
    next_first = __ldg(info + 1).w;
  }
  // returns true when the group changed
  __device__ bool seek(int tile) {
    bool moved = false;
    while (tile >= next_first && g + 1 < groups) {
      ++g;
      cur = __ldg(info + g);
      next_first = __ldg(info + g + 1).w;
      moved = true;
    }
    return moved;
  }
};

template <int BN>
struct GroupedSmem {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = GG_BM * GG_BK * 2;
  static constexpr int B_BYTES = BN * GG_BK * 2;
  static constexpr int C_WARP_BYTES = 32 * 128;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_C = OFF_B + STAGES * B_BYTES;
  static constexpr int OFF_BAR = OFF_C + 4 * 2 * C_WARP_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
  static constexpr int TOTAL = OFF_MISC + 16 + 1024;
};

// B is [k, n] row-major (the N-major UMMA operand), as in the reference kernel's `b.partition([BK, BN])`.
template <int BN, bool OUT_F16>
__global__ void __launch_bounds__(GG_THREADS, 1)
gemm_grouped_kernel(GroupedWs ws, int groups, uint32_t idesc, uint32_t* status) {
  using L = GroupedSmem<BN>;
  constexpr int STAGES = L::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sA = base + L::OFF_A, sB = base + L::OFF_B, sC = base + L::OFF_C;
  const uint32_t bar_full = base + L::OFF_BAR;
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_tfull = bar_empty + STAGES * 8;
  const uint32_t bar_tempty = bar_tfull + 2 * 8;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(gen_base + L::OFF_MISC);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx wctx{misc + 1, status};

  const int total_tiles = __ldg(ws.info + groups).w;
  if ((int)blockIdx.x >= total_tiles) return;  // uniform for the CTA: nothing allocated yet

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
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(misc)), 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = misc[0];

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      GroupCursor cur(ws.info, groups);
      uint32_t stage = 0, phase = 0;
      bool ok = true, first = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const bool moved = cur.seek(tile);
        const CUtensorMap* dA = ws.desc + cur.g * 3;
        const CUtensorMap* dB = dA + 1;
        if (moved || first) {
          tmap_acquire(dA);
          tmap_acquire(dB);
          first = false;
        }
        const int tiles_n = (cur.cur.y + BN - 1) / BN;
        const int local = tile - cur.cur.w;
        const int m0 = (local / tiles_n) * GG_BM, n0 = (local % tiles_n) * BN;
        const int num_kb = (cur.cur.z + GG_BK - 1) / GG_BK;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(wctx, bar_empty + stage * 8, phase ^ 1, 1)) { ok = false; break; }
          const uint32_t full = bar_full + stage * 8;
          mbar_expect_tx(full, L::A_BYTES + L::B_BYTES);
          tma_load_2d(sA + stage * L::A_BYTES, dA, full, kb * GG_BK, m0);
#pragma unroll
          for (int j = 0; j < BN / 64; ++j)
            tma_load_2d(sB + stage * L::B_BYTES + j * (GG_BK * 128), dB, full, n0 + j * 64, kb * GG_BK);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer --------------------------------
    if (lane == 0) {
      GroupCursor cur(ws.info, groups);
      uint32_t stage = 0, phase = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
        cur.seek(tile);
        const int num_kb = (cur.cur.z + GG_BK - 1) / GG_BK;
        const uint32_t buf = it & 1;
        if (!mbar_wait(wctx, bar_tempty + buf * 8, ((it >> 1) & 1) ^ 1, 2)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(wctx, bar_full + stage * 8, phase, 3)) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t adesc = make_smem_desc(sA + stage * L::A_BYTES, 16, 1024, SWZ_128B);
          const uint64_t bdesc = make_smem_desc(sB + stage * L::B_BYTES, GG_BK * 128, 1024, SWZ_128B);
#pragma unroll
          for (int k = 0; k < GG_BK / 16; ++k)
            umma_f16_ss(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 128), idesc, (kb | k) != 0);
          umma_commit(bar_empty + stage * 8);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(bar_tfull + buf * 8);  // with k = 0 nothing was issued: completes at once
      }
    }
  } else {
    // -------------------------------- epilogue ---------------------------------
    const int q = warp & 3;
    const uint32_t sCw = sC + q * (2 * L::C_WARP_BYTES);
    GroupCursor cur(ws.info, groups);
    uint32_t it = 0;
    uint32_t nst = 0;   // stores committed by this warp: picks the staging buffer, so that `wait_read<1>` below
                        // always frees the buffer about to be written, whatever number of chunks a tile stored
    bool ok = true, first = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
      const bool moved = cur.seek(tile);
      const CUtensorMap* dC = ws.desc + cur.g * 3 + 2;
      if (moved || first) {
        // stores of the previous group must have read their staging before the descriptor changes hands
        if (lane == 0) tmap_acquire(dC);
        first = false;
      }
      const int tiles_n = (cur.cur.y + BN - 1) / BN;
      const int local = tile - cur.cur.w;
      const int m0 = (local / tiles_n) * GG_BM, n0 = (local % tiles_n) * BN;
      const bool zero = cur.cur.z <= 0;  // k = 0: C = 0 (the accumulator was never written)
      const uint32_t buf = it & 1;
      if (!mbar_wait(wctx, bar_tfull + buf * 8, (it >> 1) & 1, 4)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
      const bool rows_live = m0 + q * 32 < cur.cur.x;
#pragma unroll 1
      for (int c = 0; rows_live && c < BN / 64; ++c) {   // a warp whose rows lie past m stages and stores nothing
        if (n0 + c * 64 >= cur.cur.y) break;   // columns past n: nothing to store (uniform per warp)
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(t_row + c * 64, v0);
        tmem_ld_32x32b_x32(t_row + c * 64 + 32, v1);
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        tmem_wait_ld();
        const uint32_t sbuf = sCw + (nst & 1) * L::C_WARP_BYTES;
        ++nst;
        const uint32_t row_addr = sbuf + lane * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t* src = (j < 4) ? &v0[j * 8] : &v1[(j - 4) * 8];
          uint32_t p[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float lo = zero ? 0.0f : __uint_as_float(src[2 * e]);
            const float hi = zero ? 0.0f : __uint_as_float(src[2 * e + 1]);
            p[e] = OUT_F16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
          }
          const uint32_t dst = row_addr + ((uint32_t)(j ^ (lane & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(p[0]), "r"(p[1]), "r"(p[2]),
                       "r"(p[3])
                       : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(dC, sbuf, n0 + c * 64, m0 + q * 32);
          tma_store_commit();
        }
      }
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
template <int BN, bool OUT_F16>
static int launch_grouped(const int64_t* a_ptrs, const int64_t* b_ptrs, const int64_t* c_ptrs,
                          const int32_t* a_metas, const int32_t* b_metas, const int32_t* c_metas, int groups,
                          void* workspace, cudaStream_t stream) {
  using L = GroupedSmem<BN>;
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  const CUtensorMapDataType dt = OUT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  // Templates carry what is common to every group (element type, box, swizzle); address, extents
  // and pitch are placeholders that the prepare kernel replaces.
  CUtensorMap tA, tB, tC;
  int rc;
  if ((rc = b200h::encode_tmap_2d(&tA, dt, 2, workspace, 1024, 1024, 2048, GG_BK, GG_BM, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  if ((rc = b200h::encode_tmap_2d(&tB, dt, 2, workspace, 1024, 1024, 2048, 64, GG_BK, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  if ((rc = b200h::encode_tmap_2d(&tC, dt, 2, workspace, 1024, 1024, 2048, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  GroupedWs ws;
  ws.desc = static_cast<CUtensorMap*>(workspace);
  ws.info = reinterpret_cast<int4*>(static_cast<uint8_t*>(workspace) + grouped_desc_bytes(groups));
  grouped_prepare_kernel<BN><<<(groups + GG_PREP_THREADS / 32 - 1) / (GG_PREP_THREADS / 32), GG_PREP_THREADS, 0, stream>>>(tA, tB, tC, a_ptrs, b_ptrs, c_ptrs, a_metas, b_metas,
                                                               c_metas, groups, ws);
  const cudaError_t after_grouped_prepare_launch = cudaGetLastError();
  B200_CUDA_CHECK(after_grouped_prepare_launch);
  auto kern = gemm_grouped_kernel<BN, OUT_F16>;
  static bool attr_done[64] = {};
  if (!attr_done[di->ordinal]) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    attr_done[di->ordinal] = true;
  }
  const uint32_t fmt = OUT_F16 ? FMT_F16 : FMT_BF16;
  const uint32_t idesc = make_idesc(fmt, fmt, 0, 1, GG_BM, BN);
  // the tile count is only known on the device: one CTA per SM, CTAs without a tile leave at once
  kern<<<di->sm_count, GG_THREADS, L::TOTAL, stream>>>(ws, groups, idesc, di->status);
  const cudaError_t after_grouped_main_launch = cudaGetLastError();
  B200_CUDA_CHECK(after_grouped_main_launch);
  return B200_OK;
}

}  // namespace b200

size_t b200_grouped_workspace_bytes(int groups) { return b200::grouped_ws_bytes(groups < 0 ? 0 : groups); }

// dtype 0 = bf16, 1 = f16; bn 128 or 256.  All table pointers are device pointers.
int b200_gemm_grouped_dispatch(int dtype, int bn, const int64_t* a_ptrs, const int64_t* b_ptrs, const int64_t* c_ptrs,
                               const int32_t* a_metas, const int32_t* b_metas, const int32_t* c_metas, int groups,
                               void* workspace, cudaStream_t stream) {
  using namespace b200;
  if (groups == 0) return B200_OK;
  if (bn == 256)
    return dtype ? launch_grouped<256, true>(a_ptrs, b_ptrs, c_ptrs, a_metas, b_metas, c_metas, groups, workspace, stream)
                 : launch_grouped<256, false>(a_ptrs, b_ptrs, c_ptrs, a_metas, b_metas, c_metas, groups, workspace, stream);
  if (bn == 128)
    return dtype ? launch_grouped<128, true>(a_ptrs, b_ptrs, c_ptrs, a_metas, b_metas, c_metas, groups, workspace, stream)
                 : launch_grouped<128, false>(a_ptrs, b_ptrs, c_ptrs, a_metas, b_metas, c_metas, groups, workspace, stream);
  return b200h::set_error(B200_ERR_UNSUPPORTED, "group_gemm: BN=%d has no precompiled configuration (128, 256)", bn);
}
