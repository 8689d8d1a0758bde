// Block-scaled GEMMs on CTA pairs: one 256 x 256 output tile per pair of SMs (tcgen05.mma.cta_group::2 with
// .block_scale, M = 256, N = 256), for the three formats of gemm_nvfp4.cu: NVFP4 (kind::mxf4nvf4, K = 64 per
// instruction, UE4M3 scale per 16), MXFP4 (kind::mxf4, K = 64, UE8M0 scale per 32) and MXFP8 (kind::mxf8f6f4,
// K = 32, UE8M0 scale per 32).
//
// Why pairs: a block-scaled stage is only 384-540 tensor-pipe cycles long, so what limits these kernels is not a
// memory level (L2 -> SM runs at a third of its peak) but the chain of hand-offs around every stage: copies issued,
// bytes landed, scales moved to Tensor Memory, MMAs issued, stage released.  A pair puts twice the tensor work
// (256 x 256 x 256 elements per stage) behind one such chain, with each CTA loading its own 128 rows of A and only
// HALF of the tile's B rows (the instruction reads the other half from the partner's shared memory): 32 KB + 6 KB of
// scales per CTA and stage.
//
// Same operand formats, scale arrangement in Tensor Memory and scratch layout of the re-laid-out scales as
// gemm_nvfp4.cu (Z = alpha * sum_k x*xs * y*ys; cutile-examples/examples/nvfp4.rs:37-76).  Per CTA:
//   warp 0        TMA producer: own A rows, own half of B, own A-scale blocks, the tile's B-scale blocks
//   warp 1        leader CTA only: issues the pair's MMAs; both: Tensor-Memory allocation
//   warps 2, 3    idle (roles are aligned to warpgroups so that registers can be re-balanced with setmaxnreg)
//   warps 4..11   epilogue: two warps per 32-lane quarter (128 columns each); the accumulator is drained
//                 into packed registers first and handed back, then staged and stored with TMA
//   warps 12..19  scale writers: shared memory -> Tensor Memory (tcgen05.st), two sets taking alternate
//                 stages; each CTA writes its own Tensor Memory and arrives on the LEADER's per-stage barrier
// Every CTA holds the scales of its own 128 A rows and of all 256 B rows of the tile.
#include "../../include/b200tile.h"
#include "host_common.h"
#include "sm100_ptx.cuh"
#include "trace.cuh"

namespace b200 {

#ifdef B200TILE_TRACE
// leader CTA of pair 5 -- MMA thread: [0] accumulator waits, [2] scale-region waits, [3] MMA issue, [4] commits,
// [5] stages, [6] total cycles, [7] the same span in ns; writer warp 12: [0] stage-full waits, [1] loads +
// store issue, [2] store completion, [3] region waits, [4] stages, [5] total; producer: [0] stage-empty waits,
// [1] issue of the copies, [2] stages, [3] total
__device__ long long g_trace_fp4p[8];
__device__ long long g_trace_fp4p_writer[8];
__device__ long long g_trace_fp4p_producer[8];
// time lines (clock64 of one SM) of global stages 96..103 of the leader CTA of pair 5, five events per stage:
// see b200_trace_read_fp4_pair_tl
__device__ long long g_trace_fp4p_tl[40];
#define B200_TL(e, g) if ((g) >= 96u && (g) < 104u && blockIdx.x == 10) g_trace_fp4p_tl[((g) - 96u) * 5 + (e)] = clock64()
#else
#define B200_TL(i, cond)
#endif

// FMT = 1: NVFP4, 2: MXFP4, 0: MXFP8 (as in gemm_nvfp4.cu)
template <int FMT>
struct F4P {
  static constexpr bool FP4 = FMT != 0;
  static constexpr int STAGE_ELEMS = FP4 ? 256 : 128;   // K elements per 128-byte row
  static constexpr int BM = 128;                 // rows per CTA (256 per pair)
  static constexpr int BN = 256;                 // tile columns
  static constexpr int STAGES = 5;               // 3 / 4 stages measured 16 % / 4 % slower
  static constexpr int EW = 8;                   // epilogue warps
  static constexpr int THREADS = 128 + 32 * EW + 256;   // 640: the kernel is compiled for 96 registers per thread
  // setmaxnreg pool = what the CTA was given at launch, 640 x 96 = 61440: 384 x 56 + 256 x 152 = 60416
  static constexpr int OTHER_REGS = 56, EPI_REGS = 152;
  static constexpr int CHUNKS = 2;               // 128-row scale blocks per B tile
  // 512-byte scale blocks (128 rows x 4 scale bytes) along K per stage: one per instruction for NVFP4, one per two
  // instructions for MXFP4 (a byte pair each), one per stage for MXFP8 (a byte per instruction)
  static constexpr int KQ_PER_STAGE = FMT == 1 ? 4 : (FMT == 2 ? 2 : 1);
  static constexpr int RK = FMT == 1 ? 2 : 1;    // blocks along K per scale region
  static constexpr int HALVES = KQ_PER_STAGE / RK, MMAS_PER_REGION = 4 / HALVES;
  // a region's columns (24 or 12) are padded to 32 / 16 so that ONE tcgen05.st writes it
  static constexpr int REGION_USED = 4 * RK * (1 + CHUNKS);
  static constexpr int REGION_COLS = REGION_USED <= 16 ? 16 : 32;
  static constexpr int SF_BASE = BN;             // one accumulator, the scale regions follow it
  static constexpr int NREG_FIT = (512 - SF_BASE) / REGION_COLS;
  static constexpr int NREG_CAP = STAGES * HALVES - 1;   // a writer's wait on `empty` stays within one phase
  static constexpr int NREG = NREG_FIT < NREG_CAP ? NREG_FIT : NREG_CAP;
  static_assert(NREG >= 2, "at least two scale regions");
  static_assert(SF_BASE + NREG * REGION_COLS <= 512, "scale regions must fit beside the accumulator");
  static constexpr int A_BYTES = BM * 128;
  static constexpr int B_BYTES = (BN / 2) * 128;
  static constexpr int SFA_BYTES = KQ_PER_STAGE * 512;
  static constexpr int SFB_BYTES = KQ_PER_STAGE * CHUNKS * 512;
  static constexpr int SFB_COL0 = 4 * RK;
  static constexpr int STAGE_TX = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int STAGE_BYTES = (STAGE_TX + 1023) / 1024 * 1024;
  // bf16 output staging: one [32 rows][128 B] swizzled buffer per epilogue warp, stored with TMA.  (Storing rows
  // straight from registers -- 16 bytes per lane, 32 different rows per instruction -- made every tile boundary a
  // burst of half-filled sectors from all 148 CTAs at once, behind which the next tile's loads waited up to 6000
  // cycles.)
  static constexpr int OFF_C = STAGES * STAGE_BYTES;
  static constexpr int C_WARP_BYTES = 32 * 128;
  static constexpr int OFF_BAR = OFF_C + EW * C_WARP_BYTES;
  static constexpr int NUM_BARS = 3 * STAGES + 2;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
  static constexpr int TOTAL = OFF_MISC + 16 + 1024;
};

__device__ __forceinline__ void bulk_load_1d_p(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void umma_nvfp4_ss_2cta(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                   uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_mxf4_ss_2cta(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                  uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_mxfp8_ss_2cta(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                   uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
// Instruction descriptors: E2M1 operands have code 1 (NVFP4, MXFP4), E4M3 code 0 (MXFP8); bit 23 selects UE8M0
// scales; `sf` picks the scale byte (MXFP8: 0..3) or byte pair (MXFP4: 0 or 2) of the Tensor-Memory word, for A in
// bits [29,31) and for B in bits [4,6)
template <int FMT>
__host__ __device__ constexpr uint32_t make_idesc_bs_pair(uint32_t M, uint32_t N, uint32_t sf) {
  return (FMT != 0 ? ((1u << 7) | (1u << 10)) : 0u) | (FMT != 1 ? (1u << 23) : 0u) | ((N >> 3) << 17) |
         ((M >> 4) << 24) | (sf << 4) | (sf << 29);
}

template <bool OUT_F32, int FMT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(F4P<FMT>::THREADS, 1)
gemm_nvfp4_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmC, const uint8_t* __restrict__ sfa,
                       const uint8_t* __restrict__ sfb, void* __restrict__ Z, int M, int N, int K, int64_t ldz,
                       float alpha, int group_m, uint32_t* status) {
  using C = F4P<FMT>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar_full = base + C::OFF_BAR;            // per CTA: its own TMA bytes
  const uint32_t bar_empty = bar_full + STAGES * 8;       // per CTA: the leader commits to both
  const uint32_t bar_tfull = bar_empty + STAGES * 8;      // per CTA
  const uint32_t bar_tempty = bar_tfull + 8;              // meaningful in the leader only
  // [STAGES], meaningful in the leader only: a stage's scales are in both Tensor Memories (which implies that its
  // operands are in both shared memories); ONE barrier per stage, not per scale region, because every wait costs
  // the MMA warp ~90 cycles
  const uint32_t bar_sf_ready = bar_tempty + 8;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(gen_base + C::OFF_MISC);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  WaitCtx wctx{misc + 1, status};
  auto stage_a = [&](uint32_t s) { return base + s * C::STAGE_BYTES; };
  auto stage_b = [&](uint32_t s) { return base + s * C::STAGE_BYTES + C::A_BYTES; };
  auto stage_sfa = [&](uint32_t s) { return base + s * C::STAGE_BYTES + C::A_BYTES + C::B_BYTES; };
  auto stage_sfb = [&](uint32_t s) { return stage_sfa(s) + C::SFA_BYTES; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, 1);
    }
    mbar_init(bar_tfull, 1);
    mbar_init(bar_tempty, 2 * C::EW);                                    // the epilogue warps of both CTAs
    for (int r = 0; r < STAGES; ++r) mbar_init(bar_sf_ready + r * 8, 8);   // four writer warps of each CTA
    misc[1] = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (!OUT_F32) tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc_2cta(smem_u32(const_cast<uint32_t*>(misc)), 512);
    tmem_relinquish_2cta();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // the partner's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = misc[0];

  const int tiles_m = (M + 2 * C::BM - 1) / (2 * C::BM);
  const int tiles_n = (N + C::BN - 1) / C::BN;
  const int total_tiles = tiles_m * tiles_n;
  const int num_kb = (K + C::STAGE_ELEMS - 1) / C::STAGE_ELEMS;
  const int kq_count = num_kb * C::KQ_PER_STAGE;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  auto tile_coords = [&](int tile, int& bm, int& bn) {
    const int in_group = group_m * tiles_n;
    const int group = tile / in_group;
    const int first_m = group * group_m;
    const int rem = tiles_m - first_m;
    const int gsz = rem < group_m ? rem : group_m;
    bm = first_m + (tile % gsz);
    bn = (tile % in_group) / gsz;
  };

  if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::OTHER_REGS));
  if (warp == 0) {
    {
      // converged warp, one elected lane issues the copies (as for the MMA warp below)
      const bool me = elect_one() != 0;
      // the scale blocks come from the pre-pass launched just before this kernel (programmatic dependent launch:
      // everything above overlapped its tail); nothing else in this kernel reads what that grid writes
      asm volatile("griddepcontrol.wait;" ::: "memory");
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      [[maybe_unused]] uint32_t gs = 0;
      B200_TR_DECL(3);
      for (int tile = pair; tile < total_tiles && ok; tile += num_pairs) {
        int bm, bn;
        tile_coords(tile, bm, bn);
        const int m0 = bm * (2 * C::BM) + (int)rank * C::BM;
        const int n0 = bn * C::BN + (int)rank * (C::BN / 2);
        const uint8_t* sfa_tile = sfa + (int64_t)(bm * 2 + (int)rank) * kq_count * 512;
        const uint8_t* sfb_tile = sfb + (int64_t)bn * kq_count * (C::CHUNKS * 512);
        for (int kb = 0; kb < num_kb; ++kb) {
          B200_TR_COUNT(2);
          B200_TR_BEGIN();
          if (!__all_sync(0xffffffffu, mbar_wait(wctx, bar_empty + stage * 8, phase ^ 1, 1))) { ok = false; break; }
          B200_TR_END(0);
          B200_TL(0, gs);
          B200_TR_BEGIN();
          const uint32_t full = bar_full + stage * 8;
          if (me) {
            // (a barrier of their own for the scale blocks, so that the writers start while the operands are still
            // in flight, was measured 4 % slower: one more wait per stage for the MMA warp)
            mbar_expect_tx(full, C::STAGE_TX);
            bulk_load_1d_p(stage_sfa(stage), sfa_tile + (int64_t)kb * C::SFA_BYTES, C::SFA_BYTES, full);
            bulk_load_1d_p(stage_sfb(stage), sfb_tile + (int64_t)kb * C::SFB_BYTES, C::SFB_BYTES, full);
            tma_load_2d(stage_a(stage), &tmA, full, kb * 128, m0);
            tma_load_2d(stage_b(stage), &tmB, full, kb * 128, n0);
          }
          __syncwarp();
          B200_TR_END(1);
          B200_TL(1, gs);
          ++gs;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      B200_TR_FLUSH(g_trace_fp4p_producer, 3, blockIdx.x == 10 && lane == 0);
    }
  } else if (warp == 1) {
    if (leader) {
      // The whole warp runs the control flow and the address arithmetic (so that it stays in uniform registers)
      // and one elected lane issues the tcgen05 instructions: a loop under `if (lane == 0)` costs ~80 cycles per
      // MMA and per commit, more per stage than the stage's 540 cycles of tensor work leave room for.
      const bool me = elect_one() != 0;
      uint32_t stage = 0, phase = 0, it = 0, reg = 0;
      bool ok = true;
      [[maybe_unused]] uint32_t gs = 0;
      B200_TR_DECL(6);
      for (int tile = pair; tile < total_tiles && ok; tile += num_pairs, ++it) {
        B200_TR_BEGIN();
        if (!__all_sync(0xffffffffu, mbar_wait(wctx, bar_tempty, (it & 1) ^ 1, 2))) { ok = false; break; }
        B200_TR_END(0);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base;
        for (int kb = 0; kb < num_kb; ++kb) {
          B200_TR_COUNT(5);
          const uint64_t adesc = make_smem_desc(stage_a(stage), 16, 1024, SWZ_128B);
          const uint64_t bdesc = make_smem_desc(stage_b(stage), 16, 1024, SWZ_128B);
          // both CTAs' writers arrive only after their stage's TMA bytes have landed, so this wait covers the
          // operands in both shared memories and the stage's scales in both Tensor Memories
          B200_TR_BEGIN();
          if (!__all_sync(0xffffffffu, mbar_wait(wctx, bar_sf_ready + stage * 8, phase, 6))) { ok = false; break; }
          tc_fence_after_sync();
          B200_TR_END(2);
          B200_TL(3, gs);
#pragma unroll
          for (int h = 0; h < C::HALVES; ++h) {
            const uint32_t sf_t = tmem_base + C::SF_BASE + reg * C::REGION_COLS;
            B200_TR_BEGIN();
#pragma unroll
            for (int kk = 0; kk < C::MMAS_PER_REGION; ++kk) {
              const int k = h * C::MMAS_PER_REGION + kk;
              if (!me) continue;
              const uint64_t a_k = adesc + (uint64_t)(k * 2), b_k = bdesc + (uint64_t)(k * 2);
              if (FMT == 1)
                umma_nvfp4_ss_2cta(d_tmem, a_k, b_k, make_idesc_bs_pair<1>(2 * C::BM, C::BN, 0), sf_t + kk * 4,
                                   sf_t + C::SFB_COL0 + kk * C::CHUNKS * 4, (kb | k) != 0);
              else if (FMT == 2)
                umma_mxf4_ss_2cta(d_tmem, a_k, b_k, make_idesc_bs_pair<2>(2 * C::BM, C::BN, (uint32_t)(kk * 2)), sf_t,
                                  sf_t + C::SFB_COL0, (kb | k) != 0);
              else
                umma_mxfp8_ss_2cta(d_tmem, a_k, b_k, make_idesc_bs_pair<0>(2 * C::BM, C::BN, (uint32_t)k), sf_t,
                                   sf_t + C::SFB_COL0, (kb | k) != 0);
            }
            B200_TR_END(3);
            if (++reg == C::NREG) reg = 0;
          }
          // frees the stage (and, later, the scale regions it used) in both CTAs
          B200_TR_BEGIN();
          if (me) {
            umma_commit_2cta(bar_empty + stage * 8);
            umma_commit_2cta(mapa_u32(bar_empty + stage * 8, 1));
          }
          __syncwarp();
          B200_TR_END(4);
          B200_TL(4, gs);
          ++gs;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok && me) {
          umma_commit_2cta(bar_tfull);
          umma_commit_2cta(mapa_u32(bar_tfull, 1));
        }
        __syncwarp();
      }
      B200_TR_FLUSH(g_trace_fp4p, 6, blockIdx.x == 10 && lane == 0);
    }
  } else if (warp >= 4 + C::EW) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::OTHER_REGS));
    // ---- scale writers: one warp per 32-lane quadrant of this CTA's Tensor Memory, two sets ----
    const int q = warp & 3;
    constexpr int NBLK = C::RK * (1 + C::CHUNKS);   // 512-byte blocks per region, A's first
    const uint32_t set = (uint32_t)(warp - (4 + C::EW)) >> 2;
    int tile = pair, kb = 0;
    uint32_t stage = 0, phase = 0, u = 0, reg = 0;
    auto advance = [&]() {
      if (++kb == num_kb) { kb = 0; tile += num_pairs; }
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
      u += C::HALVES;
      reg = (reg + C::HALVES) % C::NREG;
    };
    if (set == 1) advance();
    bool ok = true;
    [[maybe_unused]] uint32_t gs = set;
    [[maybe_unused]] const bool tl = q == 0 && lane == 0;   // first warp of either set
    B200_TR_DECL(5);
    while (tile < total_tiles && ok) {
      B200_TR_COUNT(4);
      B200_TR_BEGIN();
      if (!mbar_wait(wctx, bar_full + stage * 8, phase, 5)) { ok = false; break; }
      B200_TR_END(0);
      if (tl) { B200_TL(2, gs); }
      B200_TR_BEGIN();
#pragma unroll
      for (int h = 0; h < C::HALVES; ++h) {
        const uint32_t uu = u + h, rr = (reg + h) % C::NREG;
        // region rr was last read by the MMAs of unit uu - NREG; their stage's commit is `empty`
        if (uu >= (uint32_t)C::NREG) {
          const uint32_t gp = (uu - C::NREG) / C::HALVES;
          B200_TR_END(1);
          B200_TR_BEGIN();
          if (!mbar_wait(wctx, bar_empty + (gp % STAGES) * 8, (gp / STAGES) & 1, 7)) { ok = false; break; }
          B200_TR_END(3);
          B200_TR_BEGIN();
        }
        tc_fence_after_sync();
        const uint32_t dst = tmem_base + ((uint32_t)(q * 32) << 16) + C::SF_BASE + rr * C::REGION_COLS;
        const uint32_t src_a = stage_sfa(stage) + (h * C::RK) * 512 + lane * 16;
        const uint32_t src_b = stage_sfb(stage) + (h * C::RK) * C::CHUNKS * 512 + lane * 16;
        uint32_t regs[C::REGION_COLS];
#pragma unroll
        for (int i = NBLK * 4; i < C::REGION_COLS; ++i) regs[i] = 0u;
#pragma unroll
        for (int b = 0; b < C::RK; ++b)
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(regs[4 * b]), "=r"(regs[4 * b + 1]), "=r"(regs[4 * b + 2]), "=r"(regs[4 * b + 3])
                       : "r"(src_a + b * 512));
#pragma unroll
        for (int b = C::RK; b < NBLK; ++b)
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(regs[4 * b]), "=r"(regs[4 * b + 1]), "=r"(regs[4 * b + 2]), "=r"(regs[4 * b + 3])
                       : "r"(src_b + (b - C::RK) * 512));
        tmem_st_cols<C::REGION_COLS>(dst, regs);
      }
      if (!ok) break;
      B200_TR_END(1);
      B200_TR_BEGIN();
      tmem_wait_st();
      B200_TR_END(2);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        // the stores have completed (wait::st), so a CTA-scope release is enough for the arrive on the leader's
        // barrier; a cluster-scope release costs ~500 cycles per call
        mbar_arrive_cluster_addr_cta_release(mapa_u32(bar_sf_ready + stage * 8, 0));
      }
      gs += 2;
      advance();
      advance();
    }
    B200_TR_FLUSH(g_trace_fp4p_writer, 5, blockIdx.x == 10 && warp == 4 + C::EW && lane == 0);
  } else if (warp >= 4) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::EPI_REGS));
    // ---- epilogue ----
    const int q = warp & 3;
    const int half = (warp - 4) >> 2;     // which 128 columns of the tile
    const int row = q * 32 + lane;
    const uint32_t tempty_leader = mapa_u32(bar_tempty, 0);
    uint32_t it = 0;
    bool ok = true;
    for (int tile = pair; tile < total_tiles && ok; tile += num_pairs, ++it) {
      int bm, bn;
      tile_coords(tile, bm, bn);
      if (!mbar_wait(wctx, bar_tfull, it & 1, 4)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + half * 128;
      const int row_g = bm * (2 * C::BM) + (int)rank * C::BM + row;
      const int col0 = bn * C::BN + half * 128;
      if (OUT_F32) {
        float* zrow = static_cast<float*>(Z) + (int64_t)row_g * ldz;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_row + c * 32, v);
          tmem_wait_ld();
          const int cc = col0 + c * 32;
          if (row_g < M && cc < N) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              if (cc + i + 3 < N)
                *reinterpret_cast<float4*>(zrow + cc + i) =
                    make_float4(__uint_as_float(v[i]) * alpha, __uint_as_float(v[i + 1]) * alpha,
                                __uint_as_float(v[i + 2]) * alpha, __uint_as_float(v[i + 3]) * alpha);
              else
                for (int e = 0; e < 4; ++e)
                  if (cc + i + e < N) zrow[cc + i + e] = __uint_as_float(v[i + e]) * alpha;
            }
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_addr_cta_release(tempty_leader);   // the loads have completed (wait::ld)
      } else {
        // pass 1: Tensor Memory -> packed bf16 registers, then the accumulator goes back to the MMA thread
        uint32_t pk[64];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_row + c * 32, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i)
            pk[c * 16 + i] = pack_bf16x2(__uint_as_float(v[2 * i]) * alpha, __uint_as_float(v[2 * i + 1]) * alpha);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_addr_cta_release(tempty_leader);   // the loads have completed (wait::ld)
        // pass 2: registers -> swizzled staging -> TMA store (which clips at M and N), 64 columns at a time
        const uint32_t sbuf = base + C::OFF_C + (uint32_t)(warp - 4) * C::C_WARP_BYTES;
        const uint32_t row_addr = sbuf + lane * 128;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (lane == 0) tma_store_wait_read<0>();   // the previous store has read the buffer
          __syncwarp();
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
            tma_store_2d(&tmC, sbuf, col0 + c * 64, bm * (2 * C::BM) + (int)rank * C::BM + q * 32);
            tma_store_commit();
          }
        }
      }
    }
    if (!OUT_F32 && lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // neither CTA leaves while its partner may still touch its memory
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_2cta(tmem_base, 512);
  }
}

}  // namespace b200

// gemm_nvfp4.cu: re-lays out the row-major scales [rows][4 kq_valid bytes] of both operands as
// [tile][kq][chunk][512 B] blocks, in one launch
int b200_blockscale_relayout2(const void* src_a, int rows_a, int64_t ld_a, int tile_rows_a, int tiles_a, void* out_a,
                              const void* src_b, int rows_b, int64_t ld_b, int tile_rows_b, int tiles_b, void* out_b,
                              int kq, int kq_valid, cudaStream_t stream);

namespace {
// scale blocks along K: padded to whole stages / those the row-major tensors hold
inline void pair_kq(int fmt, int K, int* kq, int* kq_valid) {
  *kq = fmt == 1 ? ((K + 255) / 256) * 4 : (fmt == 2 ? ((K + 255) / 256) * 2 : (K + 127) / 128);
  *kq_valid = fmt == 1 ? K / 64 : K / 128;
}

template <bool OUT_F32, int FMT>
int launch_pair(const void* x, const void* y, const void* xs, const void* ys, void* z, int M, int N, int K, int64_t ldx,
                int64_t ldy, int64_t ldz, int64_t ld_xs, int64_t ld_ys, float alpha, void* scratch,
                cudaStream_t stream) {
  using namespace b200;
  using C = F4P<FMT>;
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  CUtensorMap tmA, tmB;
  int rc;
  const uint64_t row_bytes = C::FP4 ? (uint64_t)K / 2 : (uint64_t)K;
  if ((rc = b200h::encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x, row_bytes, (uint64_t)M, (uint64_t)ldx, 128,
                                  C::BM, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  if ((rc = b200h::encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, y, row_bytes, (uint64_t)N, (uint64_t)ldy, 128,
                                  C::BN / 2, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  CUtensorMap tmC = tmA;   // only the bf16 instantiations read it
  if (!OUT_F32 && (rc = b200h::encode_tmap_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, z, (uint64_t)N, (uint64_t)M,
                                              (uint64_t)ldz * 2, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  int kq, kq_valid;
  pair_kq(FMT, K, &kq, &kq_valid);
  const int tiles_m = (M + 255) / 256, tiles_n = (N + 255) / 256;
  uint8_t* s = static_cast<uint8_t*>(scratch);
  const size_t sfb_off = (size_t)2 * tiles_m * kq * 512;
  // A scales as 128-row tiles: 2 tiles_m of them (a last pair whose second CTA has no rows reads zeros); B scales
  // as 256-row tiles
  if ((rc = b200_blockscale_relayout2(xs, M, ld_xs, 128, 2 * tiles_m, s, ys, N, ld_ys, 256, tiles_n, s + sfb_off, kq,
                                      kq_valid, stream)))
    return rc;
  auto kern = gemm_nvfp4_pair_kernel<OUT_F32, FMT>;
  static b200h::DeviceOnce attr_done;
  if (!attr_done.test(di->ordinal)) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::TOTAL));
    attr_done.set(di->ordinal);
  }
  const int tiles = tiles_m * tiles_n;
  const int all_pairs = di->sm_count / 2;
  const int pairs = tiles < all_pairs ? tiles : all_pairs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pairs * 2);
  cfg.blockDim = dim3(C::THREADS);
  cfg.dynamicSmemBytes = C::TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // may start while the pre-pass drains
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  B200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, static_cast<const uint8_t*>(s),
                                     static_cast<const uint8_t*>(s + sfb_off), z, M, N, K, ldz, alpha, 8, di->status));
  return B200_OK;
}
}  // namespace

// Scratch: [2 ceil(M/256)] blocks of A scales (128-row tiles), then [ceil(N/256)] tiles of B scales (2 chunks).
// fmt = 1: NVFP4, 2: MXFP4, 0: MXFP8
size_t b200_blockscaled_pair_scratch_bytes(int fmt, int M, int N, int K) {
  int kq, kq_valid;
  pair_kq(fmt, K, &kq, &kq_valid);
  return ((size_t)2 * ((M + 255) / 256) + (size_t)2 * ((N + 255) / 256)) * (size_t)kq * 512;
}

int b200_gemm_blockscaled_pair_dispatch(int fmt, int out_f32, const void* x, const void* y, const void* xs,
                                        const void* ys, void* z, int M, int N, int K, int64_t ldx, int64_t ldy,
                                        int64_t ldz, int64_t ld_xs, int64_t ld_ys, float alpha, void* scratch,
                                        cudaStream_t stream) {
#define B200_PAIR_BS(F32_, FMT_) \
  return launch_pair<F32_, FMT_>(x, y, xs, ys, z, M, N, K, ldx, ldy, ldz, ld_xs, ld_ys, alpha, scratch, stream)
  if (fmt == 1 && out_f32) B200_PAIR_BS(true, 1);
  if (fmt == 1) B200_PAIR_BS(false, 1);
  if (fmt == 2 && out_f32) B200_PAIR_BS(true, 2);
  if (fmt == 2) B200_PAIR_BS(false, 2);
  if (fmt == 0 && out_f32) B200_PAIR_BS(true, 0);
  if (fmt == 0) B200_PAIR_BS(false, 0);
#undef B200_PAIR_BS
  return b200h::set_error(B200_ERR_UNSUPPORTED, "block-scaled pair GEMM: unknown format %d", fmt);
}

#ifdef B200TILE_TRACE
int b200_trace_read_fp4_pair(long long* out) {
  if (cudaMemcpyFromSymbol(out, b200::g_trace_fp4p, 8 * sizeof(long long)) != cudaSuccess) return 1;
  if (cudaMemcpyFromSymbol(out + 10, b200::g_trace_fp4p_writer, 7 * sizeof(long long)) != cudaSuccess) return 1;
  return cudaMemcpyFromSymbol(out + 17, b200::g_trace_fp4p_producer, 3 * sizeof(long long)) != cudaSuccess;
}
// out[5 g + e], g = 0..7 (global stages 96..103 of the leader CTA of pair 5), clock64 of event e -- 0: the producer
// sees the slot free, 1: it has issued the stage's copies, 2: a writer warp sees the stage landed, 3: the MMA warp
// sees the stage's first scale region ready, 4: it has committed the stage
int b200_trace_read_fp4_pair_tl(long long* out) {
  return cudaMemcpyFromSymbol(out, b200::g_trace_fp4p_tl, 40 * sizeof(long long)) != cudaSuccess;
}
#endif
