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
// When the tile count does not fill the last wave, that wave's tiles are split along K over all
// pairs (stream-K).  The pair that holds the END of a tile's k range owns its output; a pair whose
// share stops inside a tile publishes that fp32 partial to global scratch and raises a flag.  Every
// pair publishes FIRST and only then works as an owner, and an owner only waits (bounded) for pairs
// with a lower index: a wait never depends on a CTA that has not been dispatched yet or that is
// itself waiting, so the launch makes progress even when other work shares the GPU.  The owner
// clears a flag once it has read the partial, which leaves the scratch ready for the next launch
// (or the next replay of a captured graph) without any host-side state.
//
//   warp 0      TMA producer (both CTAs); transaction bytes are counted on the leader's barrier
//   warp 1      MMA issuer (leader CTA only) -- releases a stage in BOTH CTAs with two commits
//   warps 2..   epilogue of this CTA's 128 rows: four warps per 256 columns (4 or 8 warps)
#include <stdlib.h>

#include <mutex>

#include "host_common.h"
#include "sm100_ptx.cuh"
#include "trace.cuh"

namespace b200 {

#ifdef B200TILE_TRACE
// MMA thread of pair 10: [0] accumulator-buffer waits, [1] stage-full waits, [2] MMA issue,
// [3] commits, [4] stages, [5] tiles, [6] total cycles, [7] the same span in ns
__device__ long long g_trace_gemm_pair[16];   // [8..13]: time line of CTA 20 in ns of the global timer
#endif

constexpr int P_BM = 128;   // rows per CTA (256 per pair)

// Two tile widths.  BN = 256: one 256x256 accumulator per tile, double-buffered (the epilogue of tile i overlaps
// the main loop of tile i+1), 128-deep stages.  BN = 512: the pair's tile is 256 rows x 512 columns, i.e. two
// N = 256 MMAs per k-step that share the A operand: each CTA loads 128 rows of A and 256 columns of B per
// stage, three quarters of the bytes per FLOP of the 256-wide tile, which is what a kernel bound by the
// L2 -> shared-memory stream at full clock needs; the accumulator then takes all 512 Tensor-Memory columns, so
// there is one of it and the epilogue does not overlap the next tile's main loop (a few per cent at K = 8192).
template <int BN>
struct PairCfg {
  static_assert(BN == 256 || BN == 512, "pair tiles are 256 or 512 columns wide");
  static constexpr int NB = BN / 256;              // N = 256 MMAs per k-step
  static constexpr int NACC = BN == 256 ? 2 : 1;   // accumulators in Tensor Memory
  static constexpr int BK = BN == 256 ? 128 : 64;  // k depth of a stage
  static constexpr int KH = BK / 64;               // 64-wide (128-byte) sub-blocks per stage
  static constexpr int STAGES = BN == 256 ? 3 : 4; // 192 KiB of operand ring per CTA either way
  // Epilogue: every warp drains 256 columns of its Tensor-Memory lane quarter into packed 16-bit registers,
  // hands the accumulator back, and only then stages and stores: EH warps per quarter (column halves).
  static constexpr int EH = BN / 256;
  static constexpr int EW = 4 * EH;                // epilogue warps
  static constexpr int THREADS = 64 + 32 * EW;     // TMA warp, MMA warp, epilogue warps
  static constexpr int NSB = 2 / EH;               // staging buffers per epilogue warp (32 KiB in total)
  static constexpr int A_BYTES = P_BM * BK * 2;
  static constexpr int BJ_BYTES = 128 * BK * 2;    // the 128 columns (rows, for a K-major B) this CTA feeds to ONE MMA
  static constexpr int B_BYTES = NB * BJ_BYTES;
  static constexpr int C_WARP_BYTES = 32 * 128;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_C = OFF_B + STAGES * B_BYTES;
  static constexpr int OFF_BAR = OFF_C + EW * NSB * C_WARP_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
  static constexpr int TOTAL = OFF_MISC + 16 + 1024;
  static constexpr int SLOT_FLOATS = P_BM * BN;    // fp32 stream-K partial of one CTA
  static_assert(TOTAL <= 232448, "exceeds the shared memory of a CTA");
};
constexpr int P_MAX_SLOT_FLOATS = P_BM * 512;

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

// Work list of one CTA pair.  The first `sk_tiles` tiles are the partial last wave: their
// (tile, k-block) units are dealt out evenly ("stream-K"), so a pair's share may hold the tail of one
// tile, whole tiles and the head of another.  A share that stops inside a tile yields that last
// segment FIRST (kb1 < nkb: a partial to publish), then the segments that reach a tile's end (the
// pair owns those tiles), then whole tiles strided over the pairs.  Every role of the CTA walks the
// same list.
struct PairSched {
  int nkb, sk_tiles, total_tiles, pair, num_pairs, dp_i;
  long long u, u_pub, u_end;
  bool pub_pending;
  __device__ void init(int nkb_, int sk_tiles_, int total_tiles_, int pair_, int num_pairs_) {
    nkb = nkb_; sk_tiles = sk_tiles_; total_tiles = total_tiles_; pair = pair_; num_pairs = num_pairs_;
    dp_i = 0;
    const long long units = (long long)sk_tiles * nkb;
    u = units * pair / num_pairs;
    u_end = units * (pair + 1) / num_pairs;
    // the segment to publish starts at the last tile boundary inside the share (or at the share's start)
    const long long boundary = (u_end / nkb) * nkb;
    u_pub = (u_end == boundary) ? u_end : (boundary > u ? boundary : u);
    pub_pending = u_pub < u_end;
  }
  // first stream-K unit of pair q (used to find which pairs contribute to a tile)
  __device__ long long first_unit(int q) const { return (long long)sk_tiles * nkb * q / num_pairs; }
  __device__ bool next(int& tile, int& kb0, int& kb1) {
    if (pub_pending) {
      pub_pending = false;
      tile = (int)(u_pub / nkb);
      kb0 = (int)(u_pub - (long long)tile * nkb);
      kb1 = (int)(u_end - (long long)tile * nkb);
      return true;
    }
    if (u < u_pub) {
      tile = (int)(u / nkb);
      kb0 = (int)(u - (long long)tile * nkb);
      kb1 = nkb;   // u_pub lies on a tile boundary whenever it is past u
      u += kb1 - kb0;
      return true;
    }
    const int t = sk_tiles + pair + dp_i * num_pairs;
    if (t >= total_tiles) return false;
    ++dp_i;
    tile = t; kb0 = 0; kb1 = nkb;
    return true;
  }
};

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait for another CTA's partial tile (status code 2 on expiry).
__device__ __forceinline__ bool wait_flag(const WaitCtx& ctx, const uint32_t* flag) {
  if (ld_acquire_gpu(flag) != 0u) return true;
  const long long t0 = clock64();
  for (uint32_t it = 0;; ++it) {
    if (ld_acquire_gpu(flag) != 0u) return true;
    if ((it & 0x3F) == 0x3F) {
      if (*ctx.abort_flag) return false;
      if (clock64() - t0 > B200_WAIT_LIMIT_CYCLES) break;
    }
  }
  *ctx.abort_flag = 1;
  if (atomicCAS(ctx.status, 0u, 2u) == 0u) {
    ctx.status[1] = blockIdx.x;
    ctx.status[2] = 50;
    ctx.status[3] = 0;
  }
  return false;
}

template <bool B_KMAJOR, bool OUT_F16, int BN, bool ACC16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg<BN>::THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, int M, int N, int K, int group_m,
                    uint32_t idesc, uint32_t* status, int sk_tiles, float* sk_partials,
                    uint32_t* sk_flags) {
  using L = PairCfg<BN>;
  constexpr int P_BK = L::BK, P_KH = L::KH, P_STAGES = L::STAGES;
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
#ifdef B200TILE_TRACE
  if (blockIdx.x == 20 && threadIdx.x == 0) g_trace_gemm_pair[8] = b200_globaltimer_ns();    // kernel entry
#endif

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(bar_full + s * 8, 1);   // leader's producer arrives once with both CTAs' bytes
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + b * 8, 1);
      mbar_init(bar_tempty + b * 8, 2 * L::EW);  // the epilogue warps of both CTAs of the pair
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
#ifdef B200TILE_TRACE
  if (blockIdx.x == 20 && threadIdx.x == 0) g_trace_gemm_pair[9] = b200_globaltimer_ns();    // set-up done
#endif

  const int tiles_m = (M + 2 * P_BM - 1) / (2 * P_BM);
  const int tiles_n = (N + BN - 1) / BN;
  const int total_tiles = tiles_m * tiles_n;
  const int num_kb = (K + P_BK - 1) / P_BK;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      PairSched sched;
      sched.init(num_kb, sk_tiles, total_tiles, pair, num_pairs);
      int tile, kb0, kb1;
      while (ok && sched.next(tile, kb0, kb1)) {
        int bm, bn;
        pair_tile_coords(tile, tiles_m, tiles_n, group_m, bm, bn);
        const int m0 = bm * (2 * P_BM) + (int)rank * P_BM;
        // MMA j of a k-step covers tile columns [256 j, 256 j + 256); this CTA feeds its 128 of them
        const int n0 = bn * BN + (int)rank * 128;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(wctx, bar_empty + stage * 8, phase ^ 1, 1)) { ok = false; break; }
          const uint32_t full_leader = mapa_u32(bar_full + stage * 8, 0);
          if (leader) mbar_expect_tx(bar_full + stage * 8, 2 * (L::A_BYTES + L::B_BYTES));
          // A (and a K-major B): one [128 rows][128 B] box per 64-wide k sub-block
#pragma unroll
          for (int h = 0; h < P_KH; ++h)
            tma_load_2d_pair(sA + stage * L::A_BYTES + h * (P_BM * 128), &tmA, full_leader,
                             kb * P_BK + h * 64, m0);
#pragma unroll
          for (int jn = 0; jn < L::NB; ++jn) {
            const uint32_t sBj = sB + stage * L::B_BYTES + jn * L::BJ_BYTES;
            if (B_KMAJOR) {
#pragma unroll
              for (int h = 0; h < P_KH; ++h)
                tma_load_2d_pair(sBj + h * (128 * 128), &tmB, full_leader, kb * P_BK + h * 64, n0 + jn * 256);
            } else {
              // N-major B: one [P_BK k-rows][64 columns] box per 64-column chunk
#pragma unroll
              for (int j = 0; j < 2; ++j)
                tma_load_2d_pair(sBj + j * (P_BK * 128), &tmB, full_leader, n0 + jn * 256 + j * 64, kb * P_BK);
            }
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
      PairSched sched;
      sched.init(num_kb, sk_tiles, total_tiles, pair, num_pairs);
      int tile, kb0, kb1;
      B200_TR_DECL(6);
      for (; ok && sched.next(tile, kb0, kb1); ++it) {
        const uint32_t buf = L::NACC == 2 ? (it & 1) : 0;
        const uint32_t tpar = L::NACC == 2 ? (((it >> 1) & 1) ^ 1) : ((it & 1) ^ 1);
        B200_TR_BEGIN();
        if (!mbar_wait(wctx, bar_tempty + buf * 8, tpar, 2)) { ok = false; break; }
        B200_TR_END(0);
        B200_TR_COUNT(5);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          B200_TR_BEGIN();
          if (!mbar_wait(wctx, bar_full + stage * 8, phase, 3)) { ok = false; break; }
          tc_fence_after_sync();
          B200_TR_END(1);
#ifdef B200TILE_TRACE
          if (blockIdx.x == 20 && it == 0 && kb == kb0) g_trace_gemm_pair[10] = b200_globaltimer_ns();   // first operands landed
#endif
          B200_TR_COUNT(4);
          B200_TR_BEGIN();
          const uint64_t adesc = make_smem_desc(sA + stage * L::A_BYTES, 16, 1024, SWZ_128B);
#pragma unroll
          for (int k = 0; k < P_BK / 16; ++k) {
            // K-major operands: 32 bytes per step inside a 64-wide sub-block, next sub-block one
            // [rows][128 B] slab further; N-major B: two 8-row groups (2 x 1024 bytes) per step
            const uint32_t kmaj_a = (uint32_t)((k & 3) * 2 + (k >> 2) * ((P_BM * 128) >> 4));
            const uint32_t kmaj_b = (uint32_t)((k & 3) * 2 + (k >> 2) * ((128 * 128) >> 4));
            const uint64_t a_k = adesc + (uint64_t)kmaj_a;
#pragma unroll
            for (int jn = 0; jn < L::NB; ++jn) {
              const uint32_t sBj = sB + stage * L::B_BYTES + jn * L::BJ_BYTES;
              const uint64_t bdesc = B_KMAJOR ? make_smem_desc(sBj, 16, 1024, SWZ_128B)
                                              : make_smem_desc(sBj, P_BK * 128, 1024, SWZ_128B);
              const uint64_t b_k = bdesc + (uint64_t)(B_KMAJOR ? kmaj_b : (uint32_t)(k * 128));
              umma_f16_ss_2cta(d_tmem + jn * 256, a_k, b_k, idesc, (kb != kb0) || (k != 0));
            }
          }
          B200_TR_END(2);
          B200_TR_BEGIN();
          // free this stage in both CTAs once the MMAs have read it
          umma_commit_2cta(bar_empty + stage * 8);
          umma_commit_2cta(mapa_u32(bar_empty + stage * 8, 1));
          B200_TR_END(3);
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          umma_commit_2cta(bar_tfull + buf * 8);
          umma_commit_2cta(mapa_u32(bar_tfull + buf * 8, 1));
        }
      }
      B200_TR_FLUSH(g_trace_gemm_pair, 6, blockIdx.x == 20);
#ifdef B200TILE_TRACE
      if (blockIdx.x == 20) g_trace_gemm_pair[11] = b200_globaltimer_ns();   // last commit issued
#endif
    }
  } else {
    // -------------------------------- epilogue ---------------------------------
    // Warp w may read Tensor-Memory lanes 32 (w % 4) ..; with BN = 512 two warps share a lane quarter and take
    // 256 columns each.
    const int q = warp & 3;
    const int ew = warp - 2;                 // 0 .. EW-1
    const int half = ew >> 2;                // which 256 columns of the tile
    constexpr int CW = 256;                  // columns per epilogue warp
    const uint32_t sCw = sC + ew * (L::NSB * L::C_WARP_BYTES);
    const uint32_t tempty_leader = mapa_u32(bar_tempty, 0);
    uint32_t it = 0, nst = 0;
    bool ok = true;
    PairSched sched;
    sched.init(num_kb, sk_tiles, total_tiles, pair, num_pairs);
    int tile, kb0, kb1;
    const int etid = threadIdx.x - 64;  // 0 .. 32 EW - 1 inside the epilogue warps
    for (; ok && sched.next(tile, kb0, kb1); ++it) {
      int bm, bn;
      pair_tile_coords(tile, tiles_m, tiles_n, group_m, bm, bn);
      const int m0 = bm * (2 * P_BM) + (int)rank * P_BM, n0 = bn * BN + half * CW;
      const uint32_t buf = L::NACC == 2 ? (it & 1) : 0;
      if (!mbar_wait(wctx, bar_tfull + buf * 8, L::NACC == 2 ? ((it >> 1) & 1) : (it & 1), 4)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + half * CW;
      const int row = q * 32 + lane;
      if (!ACC16 && kb1 < num_kb) {
        // ---- the share stops inside this tile: publish the fp32 partial, column-major so that the
        // 32 lanes of a warp write 128 contiguous bytes ----
        float* slot = sk_partials + (size_t)blockIdx.x * L::SLOT_FLOATS + (size_t)(half * CW) * P_BM;
#pragma unroll 1
        for (int c = 0; c < CW / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_row + c * 32, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) slot[(c * 32 + i) * P_BM + row] = __uint_as_float(v[i]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_addr(tempty_leader + buf * 8);
        __threadfence();
        named_bar_sync(1, 32 * L::EW);
        if (etid == 0) st_release_gpu(sk_flags + blockIdx.x, 1u);
        continue;
      }
      // ---- the share reaches the tile's end: owner of the output.  When it starts inside the tile,
      // the pairs before this one hold the rest of the k range (each published it as the first item
      // of its list); wait for each and add its partial. ----
      int q_first = 0, q_last = -1;
      if (kb0 > 0) {
        q_last = pair - 1;
        q_first = pair;
        const long long tile_begin = (long long)tile * num_kb;
        while (q_first > 0 && sched.first_unit(q_first) > tile_begin) --q_first;
        for (int qq = q_first; qq <= q_last && ok; ++qq) {
          if (sched.first_unit(qq) == sched.first_unit(qq + 1)) continue;  // that pair got no units
          ok = wait_flag(wctx, sk_flags + (2 * qq + (int)rank));
        }
        if (!ok) break;
      }
      // ---- pass 1: Tensor Memory -> packed 16-bit registers (fix-up partials added in fp32 first); then
      // the accumulator goes back to the MMA thread, long before the stores below are done ----
      uint32_t pk[CW / 2];
      if constexpr (ACC16) {
        // 16-bit accumulators: one value per Tensor-Memory column; the packing load delivers two adjacent
        // columns per register, which is already the output format
#pragma unroll
        for (int c = 0; c < CW / 64; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32_pack16(t_row + c * 64, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) pk[c * 32 + i] = v[i];
        }
      } else {
#pragma unroll
      for (int c = 0; c < CW / 64; ++c) {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(t_row + c * 64, v0);
        tmem_ld_32x32b_x32(t_row + c * 64 + 32, v1);
        tmem_wait_ld();
        for (int qq = q_first; qq <= q_last; ++qq) {
          if (sched.first_unit(qq) == sched.first_unit(qq + 1)) continue;
          const float* part = sk_partials + (size_t)(2 * qq + (int)rank) * L::SLOT_FLOATS +
                              (size_t)(half * CW) * P_BM + row;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            v0[i] = __float_as_uint(__uint_as_float(v0[i]) + __ldcg(part + (c * 64 + i) * P_BM));
            v1[i] = __float_as_uint(__uint_as_float(v1[i]) + __ldcg(part + (c * 64 + 32 + i) * P_BM));
          }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float a0 = __uint_as_float(v0[2 * i]), a1 = __uint_as_float(v0[2 * i + 1]);
          const float b0 = __uint_as_float(v1[2 * i]), b1 = __uint_as_float(v1[2 * i + 1]);
          pk[c * 32 + i] = OUT_F16 ? pack_f16x2(a0, a1) : pack_bf16x2(a0, a1);
          pk[c * 32 + 16 + i] = OUT_F16 ? pack_f16x2(b0, b1) : pack_bf16x2(b0, b1);
        }
      }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster_addr_cta_release(tempty_leader + buf * 8);   // the loads have completed (wait::ld): no cluster-scope release, which costs ~500 cycles
      if (q_last >= q_first) {
        // every epilogue thread of this CTA has read the partials: clear their flags for the next launch
        named_bar_sync(1, 32 * L::EW);
        if (etid == 0)
          for (int qq = q_first; qq <= q_last; ++qq)
            if (sched.first_unit(qq) != sched.first_unit(qq + 1)) st_release_gpu(sk_flags + (2 * qq + (int)rank), 0u);
      }
      // ---- pass 2: registers -> swizzled staging -> TMA store, 64 columns at a time; the staging buffer is
      // picked by a count of committed stores, so `wait_group.read NSB-1` has always drained it ----
#pragma unroll
      for (int c = 0; c < CW / 64; ++c) {
        if (lane == 0) tma_store_wait_read<L::NSB - 1>();
        __syncwarp();
        const uint32_t sbuf = sCw + (nst % L::NSB) * L::C_WARP_BYTES;
        ++nst;
        const uint32_t row_addr = sbuf + lane * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t dst = row_addr + ((uint32_t)(j ^ (lane & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[c * 32 + j * 4]),
                       "r"(pk[c * 32 + j * 4 + 1]), "r"(pk[c * 32 + j * 4 + 2]), "r"(pk[c * 32 + j * 4 + 3])
                       : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&tmC, sbuf, n0 + c * 64, m0 + q * 32);
          tma_store_commit();
        }
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
#ifdef B200TILE_TRACE
    if (blockIdx.x == 20 && threadIdx.x == 64) g_trace_gemm_pair[12] = b200_globaltimer_ns();   // epilogue warp 0 done
#endif
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while its partner may still touch its memory
#ifdef B200TILE_TRACE
  if (blockIdx.x == 20 && threadIdx.x == 0) g_trace_gemm_pair[13] = b200_globaltimer_ns();    // about to leave
#endif
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_2cta(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------
// Stream-K scratch: one fp32 partial slot (128 x 256) and one flag per CTA, per (device, stream).
// Streams are told apart by cudaStreamGetId, which is never reused within a process (a handle can be:
// a destroyed stream's address may come back for a new one).  Allocated on the first launch that needs
// it (never while that stream is capturing: the launch then falls back to whole tiles), kept until
// process exit; when all sets of a device are taken, further streams run whole tiles only.  The flags
// are zero between launches (the kernel clears what it raised), so a launch captured into a graph
// replays correctly; two launches that share a set must not overlap on the GPU (same-stream order
// guarantees that; a graph replayed concurrently with eager work of its capture stream does not).
// ---------------------------------------------------------------------------
namespace {
struct SkScratch {
  unsigned long long stream_id;
  cudaStream_t handle;   // the handle the id was read from; the only key usable while the stream is capturing
  bool handle_live;      // false once another stream has been seen under the same handle
  float* partials;
  uint32_t* flags;
  int slots;
  bool used;
};
constexpr int kSkPerDevice = 8;
SkScratch g_sk[64][kSkPerDevice];
std::mutex g_sk_mu;

SkScratch* sk_scratch_for(int dev, int slots, cudaStream_t stream) {
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_sk_mu);
  if (cs != cudaStreamCaptureStatusNone) {
    // a capturing stream is alive, so its handle names it; only queries that are legal inside a capture
    // are made, and nothing is allocated: without a set from an earlier eager launch, whole tiles
    for (int i = 0; i < kSkPerDevice; ++i)
      if (g_sk[dev][i].used && g_sk[dev][i].handle_live && g_sk[dev][i].handle == stream && g_sk[dev][i].slots >= slots)
        return &g_sk[dev][i];
    return nullptr;
  }
  unsigned long long id = 0;
  if (cudaStreamGetId(stream, &id) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  for (int i = 0; i < kSkPerDevice; ++i)
    if (g_sk[dev][i].used && g_sk[dev][i].stream_id == id && g_sk[dev][i].slots >= slots) return &g_sk[dev][i];
  for (int i = 0; i < kSkPerDevice; ++i) {
    SkScratch& e = g_sk[dev][i];
    if (e.used) continue;
    void *p = nullptr, *f = nullptr;
    if (cudaMalloc(&p, (size_t)slots * P_MAX_SLOT_FLOATS * sizeof(float)) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    if (cudaMalloc(&f, (size_t)slots * sizeof(uint32_t)) != cudaSuccess ||
        cudaMemset(f, 0, (size_t)slots * sizeof(uint32_t)) != cudaSuccess) {
      cudaGetLastError();
      cudaFree(p);
      return nullptr;
    }
    e.stream_id = id;
    e.handle = stream;
    e.handle_live = true;
    e.partials = static_cast<float*>(p);
    e.flags = static_cast<uint32_t*>(f);
    e.slots = slots;
    e.used = true;
    // a set whose handle has been reused by this new stream belonged to a destroyed stream: it must not
    // be found by handle any more
    for (int j = 0; j < kSkPerDevice; ++j)
      if (j != i && g_sk[dev][j].used && g_sk[dev][j].handle == stream) g_sk[dev][j].handle_live = false;
    return &e;
  }
  return nullptr;  // more streams than scratch sets: whole tiles only
}

bool streamk_enabled() {
  static const bool on = [] {
    const char* v = getenv("B200TILE_STREAMK");
    return !(v && v[0] == '0');
  }();
  return on;
}
}  // namespace

template <bool B_KMAJOR, bool OUT_F16, int BN, bool ACC16 = false>
static int launch_gemm_pair(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda,
                            int64_t ldb, int64_t ldc, int group_m, int max_ctas,
                            cudaStream_t stream) {
  using L = PairCfg<BN>;
  constexpr int P_BK = L::BK;
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
                               128, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = b200h::encode_tmap_2d(&tmB, dt, 2, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64,
                               P_BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  if ((rc = b200h::encode_tmap_2d(&tmC, dt, 2, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 2, 64,
                                  32, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  static_assert(!ACC16 || OUT_F16, "16-bit accumulators exist for f16 only");
  auto kern = gemm_tc_pair_kernel<B_KMAJOR, OUT_F16, BN, ACC16>;
  static b200h::DeviceOnce attr_done;
  if (!attr_done.test(di->ordinal)) {
    B200_CUDA_CHECK(
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    attr_done.set(di->ordinal);
  }
  const int tiles = ((M + 2 * P_BM - 1) / (2 * P_BM)) * ((N + BN - 1) / BN);
  const int all_pairs = di->sm_count / 2;
  int pairs = all_pairs;
  if (tiles < pairs) pairs = tiles;
  if (max_ctas > 0 && pairs > (max_ctas + 1) / 2) pairs = (max_ctas + 1) / 2;
  // Partial last wave: when whole tiles would leave more than 5 % of the SM-time idle, deal the
  // k-blocks of the remainder tiles out evenly over all pairs (an explicit grid size keeps the
  // plain whole-tile schedule).
  int sk_tiles = 0;
  SkScratch* sk = nullptr;
  const int num_kb = (K + P_BK - 1) / P_BK;
  // Also when the tiles do not even fill one wave (at least half of it): all of them are then split along K.
  const bool partial_last = tiles > all_pairs && tiles % all_pairs != 0;
  const bool under_one = tiles < all_pairs && 2 * tiles >= all_pairs;
  // (f16 accumulators: whole tiles only, the stream-K partials are fp32)
  if (!ACC16 && max_ctas <= 0 && streamk_enabled() && (partial_last || under_one) && num_kb >= 4) {
    const int waves = (tiles + all_pairs - 1) / all_pairs;
    if ((double)tiles / ((double)waves * all_pairs) < 0.95) {
      sk = sk_scratch_for(di->ordinal, 2 * all_pairs, stream);
      if (sk) {
        sk_tiles = tiles % all_pairs;   // == tiles when they fill less than one wave
        pairs = all_pairs;
      }
    }
  }
  const uint32_t fmt = OUT_F16 ? FMT_F16 : FMT_BF16;
  const uint32_t idesc = make_idesc(fmt, fmt, 0, B_KMAJOR ? 0 : 1, 2 * P_BM, 256, ACC16 ? 0 : 1);
  kern<<<pairs * 2, L::THREADS, L::TOTAL, stream>>>(tmA, tmB, tmC, M, N, K, group_m, idesc,
                                                   di->status, sk_tiles, sk ? sk->partials : nullptr,
                                                   sk ? sk->flags : nullptr);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

}  // namespace b200

// wide = 0: 256 x 256 tiles per CTA pair; wide = 1: 256 x 512 (two N = 256 MMAs per k-step sharing A);
// wide = 2: the 256 x 512 tile with f16 accumulators (f16 operands only)
int b200_gemm_pair_dispatch(int dtype, int b_kmajor, int wide, const void* A, const void* B, void* C, int M,
                            int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int group_m,
                            int max_ctas, cudaStream_t stream) {
  using namespace b200;
  if (wide == 2) {
    if (dtype != 1) return b200h::set_error(B200_ERR_UNSUPPORTED, "gemm: f16 accumulators need f16 operands");
    return b_kmajor ? launch_gemm_pair<true, true, 512, true>(A, B, C, M, N, K, lda, ldb, ldc, group_m, max_ctas, stream)
                    : launch_gemm_pair<false, true, 512, true>(A, B, C, M, N, K, lda, ldb, ldc, group_m, max_ctas, stream);
  }
#define B200_PAIR_CASE(KM_, F16_)                                                                          \
  return wide ? launch_gemm_pair<KM_, F16_, 512>(A, B, C, M, N, K, lda, ldb, ldc, group_m, max_ctas, stream) \
              : launch_gemm_pair<KM_, F16_, 256>(A, B, C, M, N, K, lda, ldb, ldc, group_m, max_ctas, stream)
  if (!b_kmajor && dtype == 0) B200_PAIR_CASE(false, false);
  if (!b_kmajor && dtype == 1) B200_PAIR_CASE(false, true);
  if (b_kmajor && dtype == 0) B200_PAIR_CASE(true, false);
  B200_PAIR_CASE(true, true);
#undef B200_PAIR_CASE
}

// Clears the stream-K flags of every scratch set of the current device (ordered on `stream`).  A launch
// that gave up a wait can leave a flag raised; the status reset calls this so that the next launch
// starts clean.
int b200_gemm_pair_reset_scratch(cudaStream_t stream) {
  using namespace b200;
  int dev = 0;
  B200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return B200_OK;
  std::lock_guard<std::mutex> lk(g_sk_mu);
  for (int i = 0; i < kSkPerDevice; ++i)
    if (g_sk[dev][i].used)
      B200_CUDA_CHECK(cudaMemsetAsync(g_sk[dev][i].flags, 0, (size_t)g_sk[dev][i].slots * sizeof(uint32_t), stream));
  return B200_OK;
}

#ifdef B200TILE_TRACE
int b200_trace_read_gemm_pair(long long* out) {
  return cudaMemcpyFromSymbol(out, b200::g_trace_gemm_pair, 16 * sizeof(long long)) != cudaSuccess;
}
#endif
