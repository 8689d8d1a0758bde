// Persistent grouped GEMM over per-group pointer and extent tables (MoE expert batches).
//
// Replaces `group_gemm_f16_nt_desc` (cutile-kernels/src/experimental/moe.rs:66-128): group g
// multiplies A_g [m_g, k_g] by B_g [k_g, n_g] into C_g [m_g, n_g], all row-major 16-bit; the
// pointers come from three device arrays of i64 and the extents from three device tables of
// eight i32 per group ({rows, cols, row stride, ...}, moe.rs:27-63).  Nothing about the groups is
// known on the host, so the work is split in two launches:
//
//   grouped_prepare_kernel   one CTA: validates every group's pointers and pitches (16-byte rule),
//                            computes the tile counts and their exclusive prefix sum into the workspace
//   gemm_grouped_kernel      persistent warp-specialised GEMM walking the concatenated tile list of all
//                            groups, tile t of the list going to CTA t mod grid like the reference's
//                            `tile_idx += NUM_SM`
//
// No TMA descriptor is involved: with per-group base addresses, extents and pitches that exist only
// in device memory a descriptor would have to be built on the device for every group.  Instead four
// producer warps fill the operand ring with 16-byte `cp.async` copies whose addresses are computed
// from the table entries and checked against the group's extents in the kernel (rows, columns and
// k past the extents are zero-filled by the copy's source-size operand, never read), writing the
// same 128-byte-swizzled layout that the tensor core's shared-memory descriptors expect.  The
// epilogue goes tcgen05.ld -> 16-bit -> swizzled staging -> 16-byte global stores, clipped to
// [m_g, n_g].  Every address the kernel touches is therefore ptr_g + (row < rows_g) * pitch_g +
// (col < cols_g).
//
//   warps 0..3  producers: cp.async ring; every thread lets the hardware arrive on the stage's `full`
//               barrier when its copies have landed (cp.async.mbarrier.arrive.noinc), the MMA thread
//               crosses from the generic to the async proxy with fence.proxy.async after its wait
//   warp 4      MMA issuer: tcgen05.mma kind::f16 into two TMEM accumulator buffers
//   warps 5..8  epilogue
#include <atomic>

#include "host_common.h"
#include "sm100_ptx.cuh"
#include "trace.cuh"

namespace b200 {

#ifdef B200TILE_TRACE
// MMA warp of CTA 5: [0] accumulator waits, [1] stage-full waits, [2] fence + MMA issue + commit, [4] stages,
// [5] total cycles, [6] the same span in ns
__device__ long long g_trace_grouped[8];
#endif

constexpr int GG_BM = 128;
constexpr int GG_BK = 64;
constexpr int GG_PRODUCERS = 128;
constexpr int GG_THREADS = GG_PRODUCERS + 32 + 128;
constexpr int GG_PREP_THREADS = 256;

enum : uint32_t { ST_BAD_GROUP = 3 };   // status code: a group's pointer or pitch breaks the 16-byte rule

// Workspace: one int4 {m, n, k, first tile} per group and a closing record whose .w is the total
// tile count.  A group that fails validation gets m = 0 (no tiles, nothing stored).
struct GroupedWs {
  int4* info;  // [groups + 1]
};
__host__ __device__ inline size_t grouped_ws_bytes(int groups) { return (size_t)(groups + 1) * sizeof(int4); }

template <int BN>
__global__ void __launch_bounds__(GG_PREP_THREADS)
grouped_prepare_kernel(const int64_t* a_ptrs, const int64_t* b_ptrs, const int64_t* c_ptrs, const int32_t* a_metas,
                       const int32_t* b_metas, const int32_t* c_metas, int groups, GroupedWs ws, uint32_t* status) {
  __shared__ int s_warp_sum[GG_PREP_THREADS / 32];
  __shared__ int s_carry;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) s_carry = 0;
  __syncthreads();
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
      const int lda = a_metas[g * 8 + 2], ldb = b_metas[g * 8 + 2], ldc = c_metas[g * 8 + 2];
      const uint64_t pa = (uint64_t)a_ptrs[g], pb = (uint64_t)b_ptrs[g], pc = (uint64_t)c_ptrs[g];
      const bool live = m > 0 && n > 0;
      // 16-byte copies: bases and pitches must be multiples of 16 bytes, pitches must cover a row
      // (with k = 0 the operands are never read, only C is written)
      const bool bad_ab = k > 0 && (((pa | pb) & 15) != 0 || pa == 0 || pb == 0 || (lda & 7) || (ldb & 7) || lda < k ||
                                    ldb < n);
      const bool bad = live && (bad_ab || (pc & 15) != 0 || pc == 0 || (ldc & 7) || ldc < n);
      if (bad) {
        if (atomicCAS(status, 0u, (uint32_t)ST_BAD_GROUP) == 0u) {
          status[1] = 0;
          status[2] = (uint32_t)g;   // the offending group
          status[3] = 0;
        }
        m = 0;
      }
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

// 16-byte asynchronous copy global -> shared; bytes past `src_bytes` (0..16) are written as zeros and
// not read.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// Makes the mbarrier track the completion of all cp.async copies this thread has issued so far: one arrival
// (counted in the barrier's expected arrivals, hence .noinc) is performed when they have completed.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// B is [k, n] row-major (the N-major UMMA operand), as in the reference kernel's `b.partition([BK, BN])`.
template <int BN, bool OUT_F16>
__global__ void __launch_bounds__(GG_THREADS, 1)
gemm_grouped_kernel(GroupedWs ws, const int64_t* a_ptrs, const int64_t* b_ptrs, const int64_t* c_ptrs,
                    const int32_t* a_metas, const int32_t* b_metas, const int32_t* c_metas, int groups, uint32_t idesc,
                    uint32_t* status) {
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
      mbar_init(bar_full + s * 8, GG_PRODUCERS);
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + b * 8, 1);
      mbar_init(bar_tempty + b * 8, 4);
    }
    misc[1] = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(misc)), 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = misc[0];

  if (warp < 4) {
    // ------------------------------ producers ------------------------------
    // Thread t owns 16-byte chunk (t & 7) of rows (t >> 3) + 16 i of every 128-byte-wide operand box, so
    // the eight threads of a row read 128 contiguous bytes.  A box row r keeps chunk c at byte
    // r * 128 + ((c ^ (r & 7)) << 4): the 128-byte swizzle; r & 7 does not depend on i.
    const int t = threadIdx.x;
    const int ch = t & 7, r0 = t >> 3;
    const uint32_t soff = (uint32_t)r0 * 128u + (uint32_t)((ch ^ (r0 & 7)) << 4);
    GroupCursor cur(ws.info, groups);
    const uint16_t* pa = nullptr;
    const uint16_t* pb = nullptr;
    int64_t lda = 0, ldb = 0;
    uint32_t issued = 0;   // stages issued by this thread
    bool ok = true, first = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      if (cur.seek(tile) || first) {
        first = false;
        pa = reinterpret_cast<const uint16_t*>(__ldg(a_ptrs + cur.g));
        pb = reinterpret_cast<const uint16_t*>(__ldg(b_ptrs + cur.g));
        lda = __ldg(a_metas + cur.g * 8 + 2);
        ldb = __ldg(b_metas + cur.g * 8 + 2);
      }
      const int m = cur.cur.x, n = cur.cur.y, k = cur.cur.z;
      const int tiles_n = (n + BN - 1) / BN;
      const int local = tile - cur.cur.w;
      const int m0 = (local / tiles_n) * GG_BM, n0 = (local % tiles_n) * BN;
      const int num_kb = (k + GG_BK - 1) / GG_BK;
      // A: rows m0 + r0 + 16 i (i < 8); the row mask is fixed for the tile
      uint32_t a_rows = 0;
#pragma unroll
      for (int i = 0; i < GG_BM / 16; ++i)
        if (m0 + r0 + 16 * i < m) a_rows |= 1u << i;
      const uint16_t* a_src = pa + (int64_t)(m0 + r0) * lda + ch * 8;
      // B: box j holds columns n0 + 64 j + [0, 64); this thread's chunk starts at column bcol + 64 j
      const int bcol = n0 + ch * 8;
      const uint16_t* b_src = pb + bcol;
      for (int kb = 0; kb < num_kb; ++kb) {
        const uint32_t stage = issued % STAGES;
        if (!mbar_wait(wctx, bar_empty + stage * 8, ((issued / STAGES) & 1) ^ 1, 1)) { ok = false; break; }
        const int k0 = kb * GG_BK;
        // ---- A box: 128 rows x 64 k ----
        {
          const int left = (k - k0 - ch * 8) * 2;   // bytes of this chunk inside [0, k)
          const uint32_t kbytes = left >= 16 ? 16u : (left > 0 ? (uint32_t)left : 0u);
          const uint32_t dst = sA + stage * L::A_BYTES + soff;
#pragma unroll
          for (int i = 0; i < GG_BM / 16; ++i) {
            const bool live = ((a_rows >> i) & 1u) && kbytes;
            cp_async_16(dst + i * 2048, live ? (const void*)(a_src + (int64_t)(16 * i) * lda + k0) : (const void*)pa,
                        live ? kbytes : 0u);
          }
        }
        // ---- B boxes: 64 k rows x 64 columns each ----
        {
          const uint32_t dst = sB + stage * L::B_BYTES + soff;
#pragma unroll
          for (int j = 0; j < BN / 64; ++j) {
            const int left = (n - bcol - 64 * j) * 2;
            const uint32_t nbytes = left >= 16 ? 16u : (left > 0 ? (uint32_t)left : 0u);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int kr = k0 + r0 + 16 * i;
              const bool live = kr < k && nbytes;
              cp_async_16(dst + j * (GG_BK * 128) + i * 2048,
                          live ? (const void*)(b_src + (int64_t)kr * ldb + 64 * j) : (const void*)pb, live ? nbytes : 0u);
            }
          }
        }
        // hardware arrives on the stage's barrier once this thread's copies above have landed; the thread
        // itself moves on to the next free slot (every slot of the ring can be in flight)
        cp_async_arrive_noinc(bar_full + stage * 8);
        ++issued;
      }
    }
    // nothing of this thread may still be in flight when the CTA leaves (also after a wait that gave up)
    cp_async_wait_all();
  } else if (warp == 4) {
    // ------------------------------- MMA issuer --------------------------------
    {
      // the whole warp runs the loop, one elected lane issues (an issue loop under `if (lane == 0)` costs ~80 cycles
      // per MMA and per commit)
      const bool me = elect_one() != 0;
      GroupCursor cur(ws.info, groups);
      uint32_t stage = 0, phase = 0, it = 0;
      bool ok = true;
      B200_TR_DECL(5);
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
        cur.seek(tile);
        const int num_kb = (cur.cur.z + GG_BK - 1) / GG_BK;
        const uint32_t buf = it & 1;
        B200_TR_BEGIN();
        if (!__all_sync(0xffffffffu, mbar_wait(wctx, bar_tempty + buf * 8, ((it >> 1) & 1) ^ 1, 2))) { ok = false; break; }
        B200_TR_END(0);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          B200_TR_COUNT(4);
          B200_TR_BEGIN();
          if (!__all_sync(0xffffffffu, mbar_wait(wctx, bar_full + stage * 8, phase, 3))) { ok = false; break; }
          B200_TR_END(1);
          B200_TR_BEGIN();
          // the operands were written by cp.async (generic proxy) and are read by the tensor core (async proxy)
          fence_proxy_async_smem();
          tc_fence_after_sync();
          const uint64_t adesc = make_smem_desc(sA + stage * L::A_BYTES, 16, 1024, SWZ_128B);
          const uint64_t bdesc = make_smem_desc(sB + stage * L::B_BYTES, GG_BK * 128, 1024, SWZ_128B);
#pragma unroll
          for (int k = 0; k < GG_BK / 16; ++k)
            if (me) umma_f16_ss(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 128), idesc, (kb | k) != 0);
          if (me) umma_commit(bar_empty + stage * 8);
          B200_TR_END(2);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok && me) umma_commit(bar_tfull + buf * 8);  // with k = 0 nothing was issued: completes at once
      }
      B200_TR_FLUSH(g_trace_grouped, 5, blockIdx.x == 5 && lane == 0);
    }
  } else {
    // -------------------------------- epilogue ---------------------------------
    const int q = warp & 3;   // the TMEM lane quarter this warp may read
    const uint32_t sCw = sC + q * (2 * L::C_WARP_BYTES);
    GroupCursor cur(ws.info, groups);
    uint16_t* pc = nullptr;
    int64_t ldc = 0;
    uint32_t it = 0, nst = 0;
    bool ok = true, first = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
      if (cur.seek(tile) || first) {
        first = false;
        pc = reinterpret_cast<uint16_t*>(__ldg(c_ptrs + cur.g));
        ldc = __ldg(c_metas + cur.g * 8 + 2);
      }
      const int m = cur.cur.x, n = cur.cur.y;
      const int tiles_n = (n + BN - 1) / BN;
      const int local = tile - cur.cur.w;
      const int m0 = (local / tiles_n) * GG_BM, n0 = (local % tiles_n) * BN;
      const bool zero = cur.cur.z <= 0;  // k = 0: C = 0 (the accumulator was never written)
      const uint32_t buf = it & 1;
      if (!mbar_wait(wctx, bar_tfull + buf * 8, (it >> 1) & 1, 4)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
      const int row_base = m0 + q * 32;
      const bool rows_live = row_base < m;
#pragma unroll 1
      for (int c = 0; rows_live && c < BN / 64; ++c) {   // a warp whose rows lie past m stores nothing
        const int col0 = n0 + c * 64;
        if (col0 >= n) break;   // columns past n: nothing to store (uniform per warp)
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(t_row + c * 64, v0);
        tmem_ld_32x32b_x32(t_row + c * 64 + 32, v1);
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
        __syncwarp();
        // rows of 128 bytes leave as eight 16-byte stores by eight neighbouring lanes
        const int cch = lane & 7;
        const int col = col0 + cch * 8;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const int row = r * 4 + (lane >> 3);
          const int grow = row_base + row;
          if (grow < m && col < n) {
            uint4 w;
            const uint32_t src = sbuf + row * 128 + ((uint32_t)(cch ^ (row & 7)) << 4);
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w)
                         : "r"(src)
                         : "memory");
            uint16_t* dst = pc + (int64_t)grow * ldc + col;
            if (col + 8 <= n) {
              *reinterpret_cast<uint4*>(dst) = w;
            } else {
              const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
              for (int e = 0; e < 8 && col + e < n; ++e) dst[e] = (uint16_t)(ww[e >> 1] >> ((e & 1) * 16));
            }
          }
        }
        // the other staging buffer is written next; this one is rewritten two chunks later, after the
        // __syncwarp() that follows the next chunk's staging
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + buf * 8);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
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
  GroupedWs ws;
  ws.info = static_cast<int4*>(workspace);
  grouped_prepare_kernel<BN><<<1, GG_PREP_THREADS, 0, stream>>>(a_ptrs, b_ptrs, c_ptrs, a_metas, b_metas, c_metas,
                                                               groups, ws, di->status);
  const cudaError_t after_grouped_prepare_launch = cudaGetLastError();
  B200_CUDA_CHECK(after_grouped_prepare_launch);
  auto kern = gemm_grouped_kernel<BN, OUT_F16>;
  static b200h::DeviceOnce attr_done;
  if (!attr_done.test(di->ordinal)) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    attr_done.set(di->ordinal);
  }
  const uint32_t fmt = OUT_F16 ? FMT_F16 : FMT_BF16;
  const uint32_t idesc = make_idesc(fmt, fmt, 0, 1, GG_BM, BN);
  // the tile count is only known on the device: one CTA per SM, CTAs without a tile leave at once
  kern<<<di->sm_count, GG_THREADS, L::TOTAL, stream>>>(ws, a_ptrs, b_ptrs, c_ptrs, a_metas, b_metas, c_metas, groups,
                                                       idesc, di->status);
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

#ifdef B200TILE_TRACE
int b200_trace_read_grouped(long long* out) {
  return cudaMemcpyFromSymbol(out, b200::g_trace_grouped, 8 * sizeof(long long)) != cudaSuccess;
}
#endif
