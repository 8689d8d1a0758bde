// NVFP4 block-scaled GEMM for sm_100a:
//   Z[M,N] = alpha * sum_k  x[m,k]*xs[m,k/16] * y[n,k]*ys[n,k/16]
// x, y: packed f4e2m1fnx2 (two values per byte, low nibble first) [M,K/2], [N,K/2];
// xs, ys: f8e4m3fn scales, logical row-major [M,K/16], [N,K/16]; fp32 accumulation.
// Replaces the machine code behind the reference's `linear_tile` + `mmaf_scaled`
// (cutile-examples/examples/nvfp4.rs:37-76; cutile/src/_core.rs:2288-2313; semantics
// cutile-book/tutorials/11-nvfp4-inference.md:58-82).
//
// The tensor core applies the scales itself (tcgen05.mma kind::mxf4nvf4.block_scale, one UE4M3
// scale per 16 elements, K = 64 per instruction) but wants them in Tensor Memory in a fixed
// arrangement: per 128 rows x 4 scale columns, lane (row % 32) of every 32-lane quadrant holds the
// four scale bytes of rows l, l+32, l+64, l+96 in four consecutive columns -- as a 512-byte block,
// byte (row%32)*16 + (row/32)*4 + col.  The row-major scale tensors are therefore re-laid out once
// per call by a small pre-pass into a SCRATCH buffer, [tile][K/64][chunk][512 B], from which the
// main kernel fetches whole stages with 1-D bulk copies.
//
//   warp 0      TMA producer: A (128 x 128 B), B (BN x 128 B) and both scale blocks per stage
//   warp 1      issuer: 4 block-scaled MMAs (K = 64 each) per stage, nothing else on its queue
//   warps 2..5  epilogue: tcgen05.ld -> alpha -> bf16/f32 -> global
//   warps 6..13 scale writers: shared memory -> Tensor Memory with tcgen05.st, one warp per quadrant,
//               two sets of four taking alternate stages
#include <mutex>

#include "../../include/b200tile.h"
#include "host_common.h"
#include "sm100_ptx.cuh"
#include "trace.cuh"

namespace b200 {

#ifdef B200TILE_TRACE
// MMA thread of CTA 5: [0] accumulator waits, [1] unused, [2] stage + scale ready waits, [3] MMA issue, [4] commits, [5] stages, [6] total cycles, [7] the same span in ns
__device__ long long g_trace_fp4[8];
// writer warp 6 of the same CTA: [0] stage-full waits, [1] region waits + loads + store issue, [2] store
// completion wait, [3] hand-off, [4] stages, [5] total cycles
__device__ long long g_trace_fp4_writer[8];
// TMA producer thread of the same CTA: [0] stage-empty waits, [1] issue of the stage's copies, [2] stages, [3] total
__device__ long long g_trace_fp4_producer[8];
#endif

constexpr int F4_BM = 128;
constexpr int F4_THREADS = 448;  // TMA, MMA, 4 epilogue warps, two sets of 4 scale-writer warps

// FMT = 1: NVFP4 (packed e2m1, UE4M3 scale per 16, K = 64 per MMA, 256 elements per stage)
// FMT = 0: MXFP8 (e4m3, UE8M0 scale per 32, K = 32 per MMA, 128 elements per stage)
// FMT = 2: MXFP4 (packed e2m1, UE8M0 scale per 32, K = 64 per MMA, 256 elements per stage; the operand /
//          scale pairing of cutile/tests/tensor_and_matrix_ops.rs:224-244)
// Either way a stage is 128 bytes per row and 4 MMAs; a 512-byte scale block holds 128 rows x 4
// scale bytes: one MMA's scales for NVFP4, two MMAs' (a byte pair each) for MXFP4, the whole stage's
// (one byte per MMA) for MXFP8.
// A_DIRECT: A's scales are read in place by the writer warps (no pre-pass, no scratch: decode-sized M
// and the prepared-weights entry); otherwise they come re-laid-out from scratch with the stage's TMA.
// AROWS: rows of the A tile that are loaded (the TMA box).  The MMA always reads 128 rows; with AROWS < 128
// (decode-sized M) the rows past the box are whatever follows in the stage (the B tile), their scales are
// zero and their results are never stored, and the shared memory saved buys a ring nearly twice as deep,
// which is what a call bound by the latency of the weight stream needs.
template <int BN, int FMT = 1, bool A_DIRECT = false, int AROWS = 128>
struct Fp4Cfg {
  static constexpr bool FP4 = FMT != 0;                      // packed 4-bit operands
  static_assert(AROWS == 128 || (AROWS % 8 == 0 && AROWS * 128 + BN * 128 >= 128 * 128),
                "a short A tile must be followed by enough of the B tile for the MMA's 128-row read");
  // The rows past a short A tile are bytes of the B tile multiplied by zero scales: harmless for E2M1, which has
  // no NaN or infinity encodings; an E4M3 operand (MXFP8) could turn 0 x NaN into NaN in those accumulator rows.
  static_assert(AROWS == 128 || FP4, "the short A tile is only valid for operand types without NaN / Inf encodings");
  static constexpr int CHUNKS = (BN + 127) / 128;            // 128-row scale blocks per B tile
  static constexpr int KQ_PER_STAGE = FMT == 1 ? 4 : (FMT == 2 ? 2 : 1);   // scale blocks along K per stage
  static constexpr int STAGES_ = AROWS < 128 ? ((BN <= 128) ? 9 : (BN <= 192 ? 6 : 5))
                                             : ((BN <= 128) ? 5 : 4);   // 3 instead of 4 measured 9 % slower at BN = 192
  // Scales travel to Tensor Memory in REGIONS of RK scale blocks along K (half a stage for NVFP4, a
  // whole one for MXFP8); the columns left beside the accumulators form a ring of NREG regions so
  // that the writers run ahead of the MMAs.  NREG < STAGES * HALVES keeps a writer's wait on a
  // stage's `empty` barrier within one phase of that barrier.
  static constexpr int RK = FMT == 1 ? 2 : 1;
  static constexpr int HALVES = KQ_PER_STAGE / RK;           // regions per stage
  static constexpr int MMAS_PER_REGION = 4 / HALVES;
  static constexpr int REGION_COLS = 4 * RK * (1 + CHUNKS);
  static constexpr int NACC = (2 * BN + 2 * REGION_COLS <= 512) ? 2 : 1;
  static constexpr int SF_BASE = NACC * BN;                  // scales sit after the accumulators
  static constexpr int NREG_FIT = (512 - NACC * BN) / REGION_COLS;
  static constexpr int NREG = NREG_FIT < STAGES_ * HALVES - 1 ? NREG_FIT : STAGES_ * HALVES - 1;
  static_assert(NREG >= 2, "at least two scale regions");
  static constexpr int A_BYTES = AROWS * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int SFA_BYTES = A_DIRECT ? 0 : KQ_PER_STAGE * 512;
  static constexpr int SFB_BYTES = KQ_PER_STAGE * CHUNKS * 512;
  static constexpr int SFB_COL0 = 4 * RK;                    // first column of the B scales inside a region
  static constexpr int STAGE_TX = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;  // bytes landed per stage
  static constexpr int STAGE_BYTES = (STAGE_TX + 1023) / 1024 * 1024;         // 1024-aligned stride
  static constexpr int STAGES = STAGES_;
  static constexpr int OFF_BAR = STAGES * STAGE_BYTES;
  static constexpr int NUM_BARS = 3 * STAGES + 4;   // + one `ready` barrier per stage
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
  static constexpr int XROW_BYTES = 4 * KQ_PER_STAGE;          // one row's A scales for one stage
  static constexpr int OFF_XBUF = (OFF_MISC + 16 + 15) / 16 * 16;   // [2][128 rows][XROW_BYTES]
  static constexpr int XBUF_BYTES = (A_DIRECT && AROWS <= 32) ? 0 : 4 * F4_BM * XROW_BYTES;   // two buffers per writer set
  static constexpr int TOTAL = OFF_XBUF + XBUF_BYTES + 1024;
  // bf16 output staging for TMA stores, one [32 rows][CW columns] swizzled buffer per epilogue warp, where shared
  // memory has room for it (every configuration but the short-A-tile one and 256-row B tiles).  Rows stored
  // straight from registers (16 bytes per lane, 32 rows per instruction) reach L2 as half-filled sectors from all
  // CTAs at once, and the next tile's loads queue behind them.
  static constexpr int CW = BN % 64 == 0 ? 64 : 32;                 // columns per store: 128- or 64-byte rows
  static constexpr int C_WARP_BYTES = 32 * CW * 2;
  static constexpr int OFF_CSTG = (OFF_XBUF + XBUF_BYTES + 1023) / 1024 * 1024;
  static constexpr int TOTAL_STG = OFF_CSTG + 4 * C_WARP_BYTES + 1024;
  static constexpr bool STG_FITS = AROWS == 128 && TOTAL_STG <= 232448;
};

// ---------------------------------------------------------------------------
// Pre-pass: row-major scales -> per-tile tcgen05 scale blocks in scratch memory.
// One thread per 4-byte word of the output.
// ---------------------------------------------------------------------------
struct RelayoutJob {
  const uint8_t* src;
  uint32_t* dst;
  int64_t ld;
  int rows, kq_count, kq_valid, tile_rows, chunks, num_tiles;
  int grid;   // CTAs that work on this job
};
// Work item = (tile, group of 8 scale blocks along K, chunk, block of the group, word): the 1024 threads of
// a CTA read 32 consecutive bytes of each of 128 rows (whole sectors, shared through L1) and every warp
// writes 128 consecutive bytes.  32-bit index arithmetic: the 64-bit divisions of a first version cost
// more than the copy itself.  Rows past `rows` and blocks past `kq_valid` are written as zeros.
__device__ __forceinline__ void relayout_scales(const RelayoutJob& j, uint32_t block, uint32_t nblocks) {
  const uint32_t kq_groups = (uint32_t)(j.kq_count + 7) / 8;
  const uint32_t total = (uint32_t)j.num_tiles * kq_groups * (uint32_t)j.chunks * 1024u;   // checked on the host
  for (uint32_t w = block * blockDim.x + threadIdx.x; w < total; w += nblocks * blockDim.x) {
    const uint32_t word = w & 127u;              // word inside the 512-byte block
    const uint32_t kq_lo = (w >> 7) & 7u;
    const uint32_t rest = w >> 10;
    const uint32_t c = rest % (uint32_t)j.chunks;
    const uint32_t t_kg = rest / (uint32_t)j.chunks;
    const uint32_t kq = (t_kg % kq_groups) * 8u + kq_lo;
    const uint32_t tile = t_kg / kq_groups;
    if (kq >= (uint32_t)j.kq_count) continue;
    const int r32 = (int)(word >> 2), g = (int)(word & 3u);
    const int local = (int)c * 128 + g * 32 + r32;
    const int row = (int)tile * j.tile_rows + local;
    uint32_t v = 0;
    if (local < j.tile_rows && row < j.rows && (int)kq < j.kq_valid)
      v = *reinterpret_cast<const uint32_t*>(j.src + (int64_t)row * j.ld + (int64_t)kq * 4);
    j.dst[((size_t)(tile * (uint32_t)j.kq_count + kq) * (uint32_t)j.chunks + c) * 128u + word] = v;
  }
}
__global__ void nvfp4_relayout_scales_kernel(const uint8_t* __restrict__ src, int rows, int kq_count,
                                             int kq_valid, int64_t ld, int tile_rows, int chunks,
                                             int num_tiles, uint32_t* __restrict__ dst) {
  const RelayoutJob j{src, dst, ld, rows, kq_count, kq_valid, tile_rows, chunks, num_tiles, (int)gridDim.x};
  relayout_scales(j, blockIdx.x, gridDim.x);
}
// Both operands' scales in one launch (a launch costs more than either copy)
__global__ void nvfp4_relayout_scales2_kernel(const RelayoutJob a, const RelayoutJob b) {
  // the GEMM that follows is launched with programmatic stream serialisation: let its CTAs set themselves up
  // (barriers, Tensor Memory, descriptor prefetch) while this grid runs; its producer warp waits for this grid's
  // completion (griddepcontrol.wait) before it reads the first scale block
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if ((int)blockIdx.x < a.grid) relayout_scales(a, blockIdx.x, (uint32_t)a.grid);
  else relayout_scales(b, blockIdx.x - (uint32_t)a.grid, (uint32_t)b.grid);
}

// Launch shape of the pre-pass: 1024-thread CTAs, one per 8 scale blocks along K of a 128-row chunk.
static inline int nvfp4_relayout_grid(int num_tiles, int kq_count, int chunks) {
  const long long ctas = (long long)num_tiles * ((kq_count + 7) / 8) * chunks;
  return (int)(ctas < 1 ? 1 : (ctas > 65535 ? 65535 : ctas));
}
static inline bool nvfp4_relayout_fits(int num_tiles, int kq_count, int chunks) {
  return (long long)num_tiles * ((kq_count + 7) / 8) * chunks * 1024 < 0x7fffffffLL;
}

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// 32 rows x 16 bytes of shared memory -> TMEM lanes 0..31 (4 columns), replicated into all four
// 32-lane quarters.
__device__ __forceinline__ void umma_nvfp4_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_mxfp8_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
// MXFP8 descriptor: E4M3 operands (code 0), UE8M0 scales (bit 23); `sf_byte` picks which of the four
// scale bytes of the TMEM word this K = 32 step uses (A: bits [29,31), B: bits [4,6)).
__host__ __device__ constexpr uint32_t make_idesc_mxfp8(uint32_t M, uint32_t N, uint32_t sf_byte) {
  return (sf_byte << 4) | ((N >> 3) << 17) | (1u << 23) | ((M >> 4) << 24) | (sf_byte << 29);
}
// Block-scaled instruction descriptor: E2M1 operands (code 1 for this kind), UE4M3 scales, K = 64.
__host__ __device__ constexpr uint32_t make_idesc_nvfp4(uint32_t M, uint32_t N) {
  return (1u << 7) | (1u << 10) | ((N >> 3) << 17) | (0u << 23) | ((M >> 4) << 24);
}

// MXFP4: E2M1 operands, UE8M0 scales, K = 64 per instruction, two scale bytes per row and instruction;
// `sf_half` (0 or 2) picks the byte pair of the TMEM word.
__device__ __forceinline__ void umma_mxf4_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
__host__ __device__ constexpr uint32_t make_idesc_mxf4(uint32_t M, uint32_t N, uint32_t sf_half) {
  return (sf_half << 4) | (1u << 7) | (1u << 10) | ((N >> 3) << 17) | (1u << 23) | ((M >> 4) << 24) | (sf_half << 29);
}

template <int BN, bool OUT_F32, int FMT, bool A_DIRECT, int AROWS>
__global__ void __launch_bounds__(F4_THREADS, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmC, const uint8_t* __restrict__ xs, int64_t ld_xs, int kq_valid, const uint8_t* __restrict__ sfa,
                  const uint8_t* __restrict__ sfb, void* __restrict__ Z,
                  int M, int N, int K, int64_t ldz, float alpha, int group_m, uint32_t* status, int weights_first) {
  using C = Fp4Cfg<BN, FMT, A_DIRECT, AROWS>;
  // Decode-sized calls (the short A tile) are chained back to back in a serving step, and ~4 us of each call are
  // fixed: launch, set-up, the first copies' latency, the drain.  So this instantiation takes part in programmatic
  // dependent launch: it lets its successor start early, and when ITS launch carries the attribute it sets itself up
  // and (weights_first: the weights and their scales are constants of the model) fills its ring with the weight tiles
  // before it waits for the predecessor, whose output it only needs for the activations.
  constexpr bool CHAINED = A_DIRECT && AROWS <= 32;
  constexpr bool FP4 = C::FP4;
  constexpr int STAGES = C::STAGES;
  constexpr int STAGE_ELEMS = FP4 ? 256 : 128;  // K elements per 128-byte row
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar_full = base + C::OFF_BAR;
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_tfull = bar_empty + STAGES * 8;
  const uint32_t bar_tempty = bar_tfull + 2 * 8;
  // [STAGES]: the stage has landed in shared memory AND its scales are in Tensor Memory.  One barrier per stage, not
  // per scale region: every wait costs the MMA warp ~90 cycles.
  const uint32_t bar_sf_ready = bar_tempty + 2 * 8;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(gen_base + C::OFF_MISC);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + b * 8, 1);
      mbar_init(bar_tempty + b * 8, 4);
    }
    for (int r = 0; r < STAGES; ++r) mbar_init(bar_sf_ready + r * 8, 4);   // one arrival per scale-writer warp
    misc[1] = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (!OUT_F32 && C::STG_FITS) tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(misc)), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = misc[0];
  if constexpr (CHAINED) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int tiles_m = (M + F4_BM - 1) / F4_BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int total_tiles = tiles_m * tiles_n;
  const int num_kb = (K + STAGE_ELEMS - 1) / STAGE_ELEMS;
  const int kq_count = num_kb * C::KQ_PER_STAGE;  // scale blocks along K (scratch is padded to this)
  auto tile_coords = [&](int tile, int& bm, int& bn) {
    const int in_group = group_m * tiles_n;
    const int group = tile / in_group;
    const int first_m = group * group_m;
    const int rem = tiles_m - first_m;
    const int gsz = rem < group_m ? rem : group_m;
    bm = first_m + (tile % gsz);
    bn = (tile % in_group) / gsz;
  };

  if (warp == 0) {
    {
      // converged warp, one elected lane issues the copies (as for the MMA warp below): 124 instead of 251 cycles per
      // stage
      const bool me = elect_one() != 0;
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      B200_TR_DECL(3);
      // stages of the first tile whose weight tile and weight scales are already on their way
      int prefetched = 0;
      if constexpr (CHAINED) {
        if (weights_first && (int)blockIdx.x < total_tiles) {
          int bm, bn;
          tile_coords(blockIdx.x, bm, bn);
          const uint8_t* sfb_tile = sfb + (int64_t)bn * kq_count * (C::CHUNKS * 512);
          prefetched = num_kb < STAGES ? num_kb : STAGES;
          if (me) {
            for (int kb = 0; kb < prefetched; ++kb) {
              const uint32_t full = bar_full + kb * 8;
              mbar_expect_tx(full, C::STAGE_TX);
              tma_load_2d(stage_b(kb), &tmB, full, kb * 128, bn * BN);
              bulk_load_1d(stage_sfb(kb), sfb_tile + (int64_t)kb * C::SFB_BYTES, C::SFB_BYTES, full);
            }
          }
          __syncwarp();
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");   // the activations are the predecessor's output
      }
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int bm, bn;
        tile_coords(tile, bm, bn);
        const uint8_t* sfa_tile = A_DIRECT ? nullptr : sfa + (int64_t)bm * kq_count * 512;
        const uint8_t* sfb_tile = sfb + (int64_t)bn * kq_count * (C::CHUNKS * 512);
        for (int kb = 0; kb < num_kb; ++kb) {
          B200_TR_COUNT(2);
          B200_TR_BEGIN();
          if (!__all_sync(0xffffffffu, mbar_wait(wctx, bar_empty + stage * 8, phase ^ 1, 1))) { ok = false; break; }
          B200_TR_END(0);
          B200_TR_BEGIN();
          const uint32_t full = bar_full + stage * 8;
          const bool half_done = CHAINED && tile == (int)blockIdx.x && kb < prefetched;
          if (me) {
            if (!half_done) mbar_expect_tx(full, C::STAGE_TX);
            tma_load_2d(stage_a(stage), &tmA, full, kb * 128, bm * F4_BM);
            if (!half_done) {
              tma_load_2d(stage_b(stage), &tmB, full, kb * 128, bn * BN);
              if (!A_DIRECT)
                bulk_load_1d(stage_sfa(stage), sfa_tile + (int64_t)kb * C::SFA_BYTES, C::SFA_BYTES, full);
              bulk_load_1d(stage_sfb(stage), sfb_tile + (int64_t)kb * C::SFB_BYTES, C::SFB_BYTES, full);
            }
          }
          __syncwarp();
          B200_TR_END(1);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      B200_TR_FLUSH(g_trace_fp4_producer, 3, blockIdx.x == 5 && lane == 0);
    }
  } else if (warp == 1) {
    {
      // The whole warp runs the control flow and the address arithmetic (which then stays in uniform registers) and
      // one elected lane issues the tcgen05 instructions: under `if (lane == 0)` the thread spent ~75 cycles per MMA
      // and ~60 per commit, 626 cycles per stage against the 384 the tensor pipe needs for the stage's MMAs.
      const bool me = elect_one() != 0;
      uint32_t stage = 0, phase = 0, it = 0, g = 0, reg = 0;
      bool ok = true;
      B200_TR_DECL(6);
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
        const uint32_t buf = (C::NACC == 2) ? (it & 1) : 0;
        const uint32_t par = (C::NACC == 2) ? (((it >> 1) & 1) ^ 1) : ((it & 1) ^ 1);
        B200_TR_BEGIN();
        if (!__all_sync(0xffffffffu, mbar_wait(wctx, bar_tempty + buf * 8, par, 2))) { ok = false; break; }
        B200_TR_END(0);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++g) {
          B200_TR_COUNT(5);
          const uint64_t adesc = make_smem_desc(stage_a(stage), 16, 1024, SWZ_128B);
          const uint64_t bdesc = make_smem_desc(stage_b(stage), 16, 1024, SWZ_128B);
          // the scale writers arrive only after the stage's TMA bytes have landed, so this wait covers the
          // operands in shared memory and the stage's scales in Tensor Memory
          B200_TR_BEGIN();
          if (!__all_sync(0xffffffffu, mbar_wait(wctx, bar_sf_ready + stage * 8, phase, 6))) { ok = false; break; }
          tc_fence_after_sync();
          B200_TR_END(2);
#pragma unroll
          for (int h = 0; h < C::HALVES; ++h) {
            const uint32_t sf_t = tmem_base + C::SF_BASE + reg * C::REGION_COLS;
            B200_TR_BEGIN();
#pragma unroll
            for (int kk = 0; kk < C::MMAS_PER_REGION; ++kk) {
              const int k = h * C::MMAS_PER_REGION + kk;
              if (!me) continue;
              if (FMT == 2)
                umma_mxf4_ss(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2),
                             make_idesc_mxf4(F4_BM, BN, (uint32_t)(kk * 2)), sf_t, sf_t + C::SFB_COL0, (kb | k) != 0);
              else if (FMT == 1)
                umma_nvfp4_ss(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2),
                              make_idesc_nvfp4(F4_BM, BN), sf_t + kk * 4, sf_t + C::SFB_COL0 + kk * C::CHUNKS * 4,
                              (kb | k) != 0);
              else
                umma_mxfp8_ss(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2),
                              make_idesc_mxfp8(F4_BM, BN, (uint32_t)k), sf_t, sf_t + C::SFB_COL0, (kb | k) != 0);
            }
            B200_TR_END(3);
            if (++reg == C::NREG) reg = 0;
          }
          B200_TR_BEGIN();
          if (me) umma_commit(bar_empty + stage * 8);   // frees the smem stage and, later, the TMEM scale regions it used
          __syncwarp();
          B200_TR_END(4);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok && me) umma_commit(bar_tfull + buf * 8);
        __syncwarp();
      }
      B200_TR_FLUSH(g_trace_fp4, 6, blockIdx.x == 5 && lane == 0);
    }
  } else if (warp >= 6) {
    // ---- scale writers: four warps, one per 32-lane quadrant of Tensor Memory ----
    // Lane l of every quadrant must hold bytes [16 l, 16 l + 16) of each 512-byte scale block (the
    // scales of rows l, l+32, l+64, l+96): what tcgen05.cp 32x128b.warpx4 would broadcast.  Written
    // with tcgen05.st instead, they stay off the tensor core's instruction queue, where each such
    // copy was measured at ~56 cycles with 12 of them per 4 MMAs.
    const int q = warp & 3;
    constexpr int NBLK = C::RK * (1 + C::CHUNKS);   // 512-byte blocks per region, A's first
    // A's scales come straight from the row-major tensor, no pre-pass: writer thread t = 32 q + lane
    // fetches row t's scale bytes of a stage (16 for NVFP4, 4 for MXFP8, one load, issued a stage
    // ahead), the four warps swap them through a small shared buffer, and lane l then picks up rows
    // l, l+32, l+64, l+96 -- the words its Tensor-Memory lane must hold.
    constexpr int AW = C::KQ_PER_STAGE * 4;     // A-scale words per lane and stage
    constexpr int XW = C::KQ_PER_STAGE;         // words per row and stage
    const uint32_t xbuf = base + C::OFF_XBUF;
    // Short A tile (AROWS <= 32, a single row of tiles): only rows 0..31 exist, every quadrant's lane l needs row l's
    // words and zeros for rows l+32, l+64, l+96, so each writer thread loads row `lane` itself and nothing is
    // swapped through shared memory (the swap, with its barrier over the four warps and the tile arithmetic, was 870
    // of the 1350 cycles a writer set spent per stage at M = 16).
    constexpr bool SHORT_A = A_DIRECT && AROWS <= 32;
    auto load_row_scales = [&](int tile, int kb, uint32_t (&dst)[XW]) {
      int row = lane;
      if constexpr (!SHORT_A) {
        int bm, bn;
        tile_coords(tile, bm, bn);
        row = bm * F4_BM + q * 32 + lane;
      }
      const int kq0 = kb * C::KQ_PER_STAGE;
#pragma unroll
      for (int k = 0; k < XW; ++k) dst[k] = 0u;
      if (row < M) {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(xs + (int64_t)row * ld_xs) + kq0;
        if (XW == 4 && kq0 + 3 < kq_valid && ((reinterpret_cast<uintptr_t>(src) & 15) == 0)) {
          const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
          dst[0] = v.x; dst[1] = v.y; dst[XW - 2] = v.z; dst[XW - 1] = v.w;
        } else {
#pragma unroll
          for (int k = 0; k < XW; ++k)
            if (kq0 + k < kq_valid) dst[k] = __ldg(src + k);
        }
      }
    };
    // Two sets of four warps take alternate stages: a set's tcgen05.st stream for one stage (issue
    // plus the wait for the region) was measured at ~650 cycles, longer than the MMA thread needs for
    // the stage's four MMAs, so one set alone was the pipeline's slowest member.
    const uint32_t set = (uint32_t)(warp - 6) >> 2;
    int tile = blockIdx.x, kb = 0;                      // position of the stage this set handles next
    uint32_t stage = 0, phase = 0, g = 0, u = 0, reg = 0;
    auto next_stage = [&](int& t_, int& kb_) {
      if (++kb_ == num_kb) { kb_ = 0; t_ += (int)gridDim.x; }
    };
    auto advance = [&]() {                              // ring / region bookkeeping of one stage
      next_stage(tile, kb);
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
      u += C::HALVES;
      reg = (reg + C::HALVES) % C::NREG;
      ++g;
    };
    if (set == 1) advance();
    bool ok = true;
    B200_TR_DECL(5);
    uint32_t x_next[XW];
    if constexpr (CHAINED) asm volatile("griddepcontrol.wait;" ::: "memory");   // the activation scales are the predecessor's output
    if (A_DIRECT && tile < total_tiles) load_row_scales(tile, kb, x_next);
    while (tile < total_tiles && ok) {
      {
        uint32_t a_cur[AW];
        if constexpr (SHORT_A) {
#pragma unroll
          for (int k = 0; k < XW; ++k) {
            a_cur[k * 4] = x_next[k];
            a_cur[k * 4 + 1] = a_cur[k * 4 + 2] = a_cur[k * 4 + 3] = 0u;
          }
          int nt = tile, nkb = kb;
          next_stage(nt, nkb);
          next_stage(nt, nkb);
          if (nt < total_tiles) load_row_scales(nt, nkb, x_next);
        } else if (A_DIRECT) {
          // publish this stage's row words, fetch those of the set's next stage, then gather the four
          // rows of the lane; two buffers per set so that a fast warp cannot overwrite a slow one's rows
          const uint32_t xb = xbuf + (set * 2 + ((g >> 1) & 1)) * (F4_BM * C::XROW_BYTES);
#pragma unroll
          for (int k = 0; k < XW; ++k)
            asm volatile("st.shared.b32 [%0], %1;" ::"r"(xb + (q * 32 + lane) * C::XROW_BYTES + k * 4), "r"(x_next[k])
                         : "memory");
          int nt = tile, nkb = kb;
          next_stage(nt, nkb);
          next_stage(nt, nkb);
          if (nt < total_tiles) load_row_scales(nt, nkb, x_next);
          named_bar_sync(1 + set, 128);   // the four warps of this set only
#pragma unroll
          for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int k = 0; k < XW; ++k)
              asm volatile("ld.shared.b32 %0, [%1];" : "=r"(a_cur[k * 4 + j])
                           : "r"(xb + (lane + 32 * j) * C::XROW_BYTES + k * 4));
        }
        B200_TR_COUNT(4);
        B200_TR_BEGIN();
        if (!mbar_wait(wctx, bar_full + stage * 8, phase, 5)) { ok = false; break; }
        B200_TR_END(0);
        B200_TR_BEGIN();
        // all stores of the stage first, one completion wait, then one arrival per region
#pragma unroll
        for (int h = 0; h < C::HALVES; ++h) {
          const uint32_t uu = u + h, rr = (reg + h) % C::NREG;
          // region rr was last read by the MMAs of unit uu - NREG; their stage's commit is `empty`
          if (uu >= (uint32_t)C::NREG) {
            const uint32_t gp = (uu - C::NREG) / C::HALVES;
            if (!mbar_wait(wctx, bar_empty + (gp % STAGES) * 8, (gp / STAGES) & 1, 7)) { ok = false; break; }
          }
          tc_fence_after_sync();
          const uint32_t dst = tmem_base + ((uint32_t)(q * 32) << 16) + C::SF_BASE + rr * C::REGION_COLS;
          const uint32_t src_b = stage_sfb(stage) + (h * C::RK) * C::CHUNKS * 512 + lane * 16;
          // region layout: RK blocks of A scales, then RK x CHUNKS blocks of B scales; gathered in
          // registers and stored as one or two wide column runs
          uint32_t regs[NBLK * 4];
          if (A_DIRECT) {
#pragma unroll
            for (int i = 0; i < C::RK * 4; ++i) regs[i] = a_cur[h * C::RK * 4 + i];
          } else {
            const uint32_t src_a = stage_sfa(stage) + (h * C::RK) * 512 + lane * 16;
#pragma unroll
            for (int b = 0; b < C::RK; ++b)
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(regs[4 * b]), "=r"(regs[4 * b + 1]), "=r"(regs[4 * b + 2]), "=r"(regs[4 * b + 3])
                           : "r"(src_a + b * 512));
          }
#pragma unroll
          for (int b = C::RK; b < NBLK; ++b) {
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(regs[4 * b]), "=r"(regs[4 * b + 1]), "=r"(regs[4 * b + 2]), "=r"(regs[4 * b + 3])
                         : "r"(src_b + (b - C::RK) * 512));
          }
          tmem_st_cols<NBLK * 4>(dst, regs);
        }
        if (!ok) break;
        B200_TR_END(1);
        B200_TR_BEGIN();
        tmem_wait_st();
        B200_TR_END(2);
        B200_TR_BEGIN();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_sf_ready + stage * 8);
        B200_TR_END(3);
      }
      advance();
      advance();
    }
    B200_TR_FLUSH(g_trace_fp4_writer, 5, blockIdx.x == 5 && warp == 6 && lane == 0);
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    uint32_t it = 0;
    bool ok = true;
    if constexpr (CHAINED) asm volatile("griddepcontrol.wait;" ::: "memory");   // the output may be the predecessor's too
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
      int bm, bn;
      tile_coords(tile, bm, bn);
      const uint32_t buf = (C::NACC == 2) ? (it & 1) : 0;
      const uint32_t par = (C::NACC == 2) ? ((it >> 1) & 1) : (it & 1);
      if (!mbar_wait(wctx, bar_tfull + buf * 8, par, 4)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
      const int row_g = bm * F4_BM + row;
      const int col0 = bn * BN;
      if constexpr (!OUT_F32 && C::STG_FITS) {
        // Tensor Memory -> bf16 -> swizzled staging -> TMA store (which clips at M and N), CW columns at a time
        constexpr int CW = C::CW;
        const uint32_t sbuf = base + C::OFF_CSTG + (uint32_t)q * C::C_WARP_BYTES;
        const uint32_t row_addr = sbuf + lane * (CW * 2);
#pragma unroll 1
        for (int c = 0; c < BN / CW; ++c) {
          uint32_t pk[CW / 2];
#pragma unroll
          for (int h = 0; h < CW / 32; ++h) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(t_row + c * CW + h * 32, v);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i)
              pk[h * 16 + i] = pack_bf16x2(__uint_as_float(v[2 * i]) * alpha, __uint_as_float(v[2 * i + 1]) * alpha);
          }
          if (c == BN / CW - 1) {   // the accumulator has been read: hand it back before the last store
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + buf * 8);
          }
          if (lane == 0) tma_store_wait_read<0>();   // the previous store has read the buffer
          __syncwarp();
#pragma unroll
          for (int j = 0; j < CW / 8; ++j) {
            // 16-byte chunk j of the row: 128-byte rows swizzle with row % 8, 64-byte rows with (row / 2) % 4
            const uint32_t sw = CW == 64 ? (uint32_t)(lane & 7) : (uint32_t)((lane >> 1) & 3);
            const uint32_t dst = row_addr + (((uint32_t)j ^ sw) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[j * 4]), "r"(pk[j * 4 + 1]),
                         "r"(pk[j * 4 + 2]), "r"(pk[j * 4 + 3]) : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmC, sbuf, col0 + c * CW, bm * F4_BM + q * 32);
            tma_store_commit();
          }
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(t_row + c * 32, v);
        tmem_wait_ld();
        const int cc = col0 + c * 32;
        if (row_g < M && cc < N) {
          if (OUT_F32) {
            float* zrow = static_cast<float*>(Z) + (int64_t)row_g * ldz + cc;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              if (cc + i + 3 < N)
                *reinterpret_cast<float4*>(zrow + i) =
                    make_float4(__uint_as_float(v[i]) * alpha, __uint_as_float(v[i + 1]) * alpha,
                                __uint_as_float(v[i + 2]) * alpha, __uint_as_float(v[i + 3]) * alpha);
              else
                for (int e = 0; e < 4; ++e)
                  if (cc + i + e < N) zrow[i + e] = __uint_as_float(v[i + e]) * alpha;
            }
          } else {
            uint16_t* zrow = static_cast<uint16_t*>(Z) + (int64_t)row_g * ldz + cc;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (cc + i + 7 < N) {
                uint4 w;
                w.x = pack_bf16x2(__uint_as_float(v[i]) * alpha, __uint_as_float(v[i + 1]) * alpha);
                w.y = pack_bf16x2(__uint_as_float(v[i + 2]) * alpha, __uint_as_float(v[i + 3]) * alpha);
                w.z = pack_bf16x2(__uint_as_float(v[i + 4]) * alpha, __uint_as_float(v[i + 5]) * alpha);
                w.w = pack_bf16x2(__uint_as_float(v[i + 6]) * alpha, __uint_as_float(v[i + 7]) * alpha);
                *reinterpret_cast<uint4*>(zrow + i) = w;
              } else {
                for (int e = 0; e < 8; ++e)
                  if (cc + i + e < N)
                    zrow[i + e] = (uint16_t)(pack_bf16x2(__uint_as_float(v[i + e]) * alpha, 0.0f) & 0xFFFF);
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + buf * 8);
      }
    }
    if (!OUT_F32 && C::STG_FITS && lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// Bytes of scratch needed for the re-laid-out B (weight) scales of an (M, N, K) problem with B tiles of BN rows.
static size_t nvfp4_scratch_layout(int M, int N, int K, int BN, size_t* sfb_offset, int fmt = 1) {
  const size_t kq = fmt == 1 ? (size_t)((K + 255) / 256) * 4
                             : (fmt == 2 ? (size_t)((K + 255) / 256) * 2 : (size_t)((K + 127) / 128));
  const size_t tiles_m = (M + F4_BM - 1) / F4_BM, tiles_n = (N + BN - 1) / BN;
  const size_t chunks = (BN + 127) / 128;
  // decode-sized M reads A's scales in place (no scratch for them)
  const size_t a_bytes = M <= F4_BM ? 0 : tiles_m * kq * 512;
  if (sfb_offset) *sfb_offset = a_bytes;
  return a_bytes + tiles_n * kq * chunks * 512;
}

// b_scales_prepared: `scratch` IS the tile layout of the B scales (written once by the caller); A's
// scales are then read in place whatever M is, so that the call needs no workspace at all.
template <int BN, bool OUT_F32, int FMT, bool A_DIRECT, int AROWS = 128>
static int launch_nvfp4_impl(const void* x, const void* y, const void* xs, const void* ys, void* z, int M, int N,
                             int K, int64_t ldx, int64_t ldy, int64_t ldz, int64_t ld_xs, int64_t ld_ys,
                             float alpha, uint8_t* scratch, cudaStream_t stream, bool b_scales_prepared) {
  using C = Fp4Cfg<BN, FMT, A_DIRECT, AROWS>;
  constexpr bool FP4 = C::FP4;
  const b200h::DeviceInfo* di = b200h::device_info();
  const uint64_t row_bytes = FP4 ? (uint64_t)K / 2 : (uint64_t)K;
  if (!di) return B200_ERR_CUDA;
  CUtensorMap tmA, tmB;
  int rc;
  if ((rc = b200h::encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x, row_bytes, (uint64_t)M,
                                  (uint64_t)ldx, 128, AROWS, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  if ((rc = b200h::encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, y, row_bytes, (uint64_t)N,
                                  (uint64_t)ldy, 128, BN, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  // scale blocks (4 scale bytes per row) along K: padded to whole stages / those the tensors hold
  constexpr bool STG = !OUT_F32 && C::STG_FITS;
  constexpr int SMEM = STG ? C::TOTAL_STG : C::TOTAL;
  CUtensorMap tmC = tmA;   // read only by the instantiations that stage their bf16 output
  if (STG && (rc = b200h::encode_tmap_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, z, (uint64_t)N, (uint64_t)M,
                                         (uint64_t)ldz * 2, C::CW, 32,
                                         C::CW == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B)))
    return rc;
  const int kq = FP4 ? ((K + 255) / 256) * C::KQ_PER_STAGE : (K + 127) / 128;
  const int kq_valid = FMT == 1 ? K / 64 : K / 128;
  const int tiles_m = (M + F4_BM - 1) / F4_BM, tiles_n = (N + BN - 1) / BN;
  const size_t sfb_off = A_DIRECT ? 0 : (size_t)tiles_m * kq * 512;
  if (!A_DIRECT) {
    if (!nvfp4_relayout_fits(tiles_m, kq, 1))
      return b200h::set_error(B200_ERR_UNSUPPORTED, "block-scaled GEMM: scale tensor of A too large for the pre-pass");
    nvfp4_relayout_scales_kernel<<<nvfp4_relayout_grid(tiles_m, kq, 1), 1024, 0, stream>>>(
        static_cast<const uint8_t*>(xs), M, kq, kq_valid, ld_xs, F4_BM, 1, tiles_m, reinterpret_cast<uint32_t*>(scratch));
  }
  if (!b_scales_prepared) {
    if (!nvfp4_relayout_fits(tiles_n, kq, C::CHUNKS))
      return b200h::set_error(B200_ERR_UNSUPPORTED, "block-scaled GEMM: scale tensor of B too large for the pre-pass");
    nvfp4_relayout_scales_kernel<<<nvfp4_relayout_grid(tiles_n, kq, C::CHUNKS), 1024, 0, stream>>>(
        static_cast<const uint8_t*>(ys), N, kq, kq_valid, ld_ys, BN, C::CHUNKS, tiles_n,
        reinterpret_cast<uint32_t*>(scratch + sfb_off));
  }
  B200_CUDA_CHECK(cudaGetLastError());
  auto kern = gemm_nvfp4_kernel<BN, OUT_F32, FMT, A_DIRECT, AROWS>;
  static b200h::DeviceOnce attr_done;
  if (!attr_done.test(di->ordinal)) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    attr_done.set(di->ordinal);
  }
  const int tiles = tiles_m * tiles_n;
  const int grid = tiles < di->sm_count ? tiles : di->sm_count;
  if constexpr (A_DIRECT && AROWS <= 32) {
    // decode-sized call: programmatic stream serialisation (see CHAINED in the kernel); the weight tiles go first only
    // when their scales were prepared ahead of the call, i.e. when nothing of the weights is written on this stream
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(F4_THREADS);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, static_cast<const uint8_t*>(xs), ld_xs, kq_valid,
                                       static_cast<const uint8_t*>(scratch), static_cast<const uint8_t*>(scratch + sfb_off), z,
                                       M, N, K, ldz, alpha, 8, di->status, b_scales_prepared ? 1 : 0));
    return B200_OK;
  }
  kern<<<grid, F4_THREADS, SMEM, stream>>>(tmA, tmB, tmC, static_cast<const uint8_t*>(xs), ld_xs, kq_valid, scratch,
                                               scratch + sfb_off, z, M, N, K, ldz, alpha, 8, di->status, 0);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

template <int BN, bool OUT_F32, int FMT = 1>
static int launch_nvfp4(const void* x, const void* y, const void* xs, const void* ys, void* z, int M, int N,
                        int K, int64_t ldx, int64_t ldy, int64_t ldz, int64_t ld_xs, int64_t ld_ys, float alpha,
                        uint8_t* scratch, cudaStream_t stream, bool b_scales_prepared = false) {
  // same rule as nvfp4_scratch_layout: one tile row of A, or prepared weights => A's scales in place
  if constexpr (FMT == 1 && BN == 128) {
    if (M <= 32)   // decode: short A tile, deep ring
      return launch_nvfp4_impl<BN, OUT_F32, FMT, true, 32>(x, y, xs, ys, z, M, N, K, ldx, ldy, ldz, ld_xs, ld_ys,
                                                           alpha, scratch, stream, b_scales_prepared);
  }
  if (M <= F4_BM || b_scales_prepared)
    return launch_nvfp4_impl<BN, OUT_F32, FMT, true>(x, y, xs, ys, z, M, N, K, ldx, ldy, ldz, ld_xs, ld_ys, alpha,
                                                     scratch, stream, b_scales_prepared);
  return launch_nvfp4_impl<BN, OUT_F32, FMT, false>(x, y, xs, ys, z, M, N, K, ldx, ldy, ldz, ld_xs, ld_ys, alpha,
                                                    scratch, stream, false);
}

}  // namespace b200

// Writes the tile layout of the B (weight) scales for B tiles of `bn` rows into `out`.
int b200_nvfp4_prepare_b_scales(const void* ys, int N, int K, int64_t ld_ys, int bn, void* out, cudaStream_t stream) {
  using namespace b200;
  const int kq = ((K + 255) / 256) * 4, kq_valid = K / 64;
  const int tiles_n = (N + bn - 1) / bn, chunks = (bn + 127) / 128;
  if (!nvfp4_relayout_fits(tiles_n, kq, chunks))
    return b200h::set_error(B200_ERR_UNSUPPORTED, "nvfp4_prepare_weight_scales: scale tensor too large for the pre-pass");
  nvfp4_relayout_scales_kernel<<<nvfp4_relayout_grid(tiles_n, kq, chunks), 1024, 0, stream>>>(
      static_cast<const uint8_t*>(ys), N, kq, kq_valid, ld_ys, bn, chunks, tiles_n, static_cast<uint32_t*>(out));
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// Row-major scales [rows][4 kq_valid bytes] -> [tile of tile_rows][kq][128-row chunk][512 B] blocks (a block is
// 128 rows x 4 scale bytes, whatever the format), for both operands of a GEMM in one launch; `tiles_a` / `tiles_b`
// may exceed what the rows need (the extra tiles are written as zeros).
int b200_blockscale_relayout2(const void* src_a, int rows_a, int64_t ld_a, int tile_rows_a, int tiles_a, void* out_a,
                              const void* src_b, int rows_b, int64_t ld_b, int tile_rows_b, int tiles_b, void* out_b,
                              int kq, int kq_valid, cudaStream_t stream) {
  using namespace b200;
  const int ca = (tile_rows_a + 127) / 128, cb = (tile_rows_b + 127) / 128;
  if (!nvfp4_relayout_fits(tiles_a, kq, ca) || !nvfp4_relayout_fits(tiles_b, kq, cb))
    return b200h::set_error(B200_ERR_UNSUPPORTED, "block-scaled GEMM: scale tensor too large for the pre-pass");
  const RelayoutJob a{static_cast<const uint8_t*>(src_a), static_cast<uint32_t*>(out_a), ld_a, rows_a, kq, kq_valid,
                      tile_rows_a, ca, tiles_a, nvfp4_relayout_grid(tiles_a, kq, ca)};
  const RelayoutJob b{static_cast<const uint8_t*>(src_b), static_cast<uint32_t*>(out_b), ld_b, rows_b, kq, kq_valid,
                      tile_rows_b, cb, tiles_b, nvfp4_relayout_grid(tiles_b, kq, cb)};
  nvfp4_relayout_scales2_kernel<<<a.grid + b.grid, 1024, 0, stream>>>(a, b);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

size_t b200_nvfp4_scratch_bytes(int M, int N, int K, int bn) {
  return b200::nvfp4_scratch_layout(M, N, K, bn, nullptr);
}

size_t b200_mxfp8_scratch_bytes(int M, int N, int K) {
  return b200::nvfp4_scratch_layout(M, N, K, 224, nullptr, 0);
}

size_t b200_mxf4_scratch_bytes(int M, int N, int K) {
  return b200::nvfp4_scratch_layout(M, N, K, 192, nullptr, 2);
}

// MXFP4 (E2M1 operands with UE8M0 scales per 32 elements): B tiles of 192 rows, as for NVFP4
int b200_gemm_mxf4_dispatch(int out_f32, const void* x, const void* y, const void* xs, const void* ys, void* z,
                            int M, int N, int K, int64_t ldx, int64_t ldy, int64_t ldz, int64_t ld_xs,
                            int64_t ld_ys, float alpha, void* scratch, cudaStream_t stream) {
  using namespace b200;
  uint8_t* s = static_cast<uint8_t*>(scratch);
  if (out_f32)
    return launch_nvfp4<192, true, 2>(x, y, xs, ys, z, M, N, K, ldx, ldy, ldz, ld_xs, ld_ys, alpha, s, stream);
  return launch_nvfp4<192, false, 2>(x, y, xs, ys, z, M, N, K, ldx, ldy, ldz, ld_xs, ld_ys, alpha, s, stream);
}

// MXFP8: B tiles of 224 rows -- the widest that keeps two accumulators plus the scales in TMEM
int b200_gemm_mxfp8_dispatch(int out_f32, const void* x, const void* y, const void* xs, const void* ys, void* z,
                             int M, int N, int K, int64_t ldx, int64_t ldy, int64_t ldz, int64_t ld_xs,
                             int64_t ld_ys, float alpha, void* scratch, cudaStream_t stream) {
  using namespace b200;
  uint8_t* s = static_cast<uint8_t*>(scratch);
  if (out_f32)
    return launch_nvfp4<224, true, 0>(x, y, xs, ys, z, M, N, K, ldx, ldy, ldz, ld_xs, ld_ys, alpha, s, stream);
  return launch_nvfp4<224, false, 0>(x, y, xs, ys, z, M, N, K, ldx, ldy, ldz, ld_xs, ld_ys, alpha, s, stream);
}

int b200_gemm_nvfp4_dispatch(int bn, int out_f32, const void* x, const void* y, const void* xs, const void* ys,
                             void* z, int M, int N, int K, int64_t ldx, int64_t ldy, int64_t ldz, int64_t ld_xs,
                             int64_t ld_ys, float alpha, void* scratch, cudaStream_t stream, int b_scales_prepared) {
  using namespace b200;
  uint8_t* s = static_cast<uint8_t*>(scratch);
#define B200_F4_CASE(BN_, F32_)                                                                            \
  return launch_nvfp4<BN_, F32_>(x, y, xs, ys, z, M, N, K, ldx, ldy, ldz, ld_xs, ld_ys, alpha, s, stream, \
                                 b_scales_prepared != 0)
  if (bn == 128 && out_f32) B200_F4_CASE(128, true);
  if (bn == 128 && !out_f32) B200_F4_CASE(128, false);
  if (bn == 192 && out_f32) B200_F4_CASE(192, true);
  if (bn == 192 && !out_f32) B200_F4_CASE(192, false);
  if (bn == 256 && out_f32) B200_F4_CASE(256, true);
  if (bn == 256 && !out_f32) B200_F4_CASE(256, false);
#undef B200_F4_CASE
  return b200h::set_error(B200_ERR_UNSUPPORTED, "linear_nvfp4: no kernel for BN = %d", bn);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant: the scale scratch lives inside the library image.
//
// Some callers are not in a position to hand over device memory: code running between
// cudaStreamBeginCapture and EndCapture on a thread that must not touch an allocator, plugins
// loaded into a host process whose memory pool they may not draw from, and start-up paths that run
// before the host's allocator exists.  For them the re-laid-out scales go into the fixed array
// below instead of a caller workspace.  The price: every GPU that loads this library reserves
// B200TILE_NVFP4_STATIC_SCRATCH_BYTES for as long as the process lives, problems whose scales do
// not fit are refused, and all calls on one GPU share the one array -- it still holds the previous
// call's scales when the next call starts (every word a call reads is first rewritten by that
// call's own pre-pass, so nothing needs clearing), and two calls that overlap on the GPU (different
// streams, or graph branches) would overwrite each other's scales.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) uint8_t g_nvfp4_static_scratch[B200TILE_NVFP4_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_mu;
uint8_t* g_static_ptr[64] = {};

// In host code `g_nvfp4_static_scratch` is only a handle for the runtime, not a device address;
// the address a kernel can use comes from cudaGetSymbolAddress, once per device, with that
// device current.
int nvfp4_static_scratch_ptr(uint8_t** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return b200h::set_error(B200_ERR_CUDA, "linear_nvfp4_static: no usable CUDA device is current");
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_nvfp4_static_scratch);
    if (e != cudaSuccess || !p)
      return b200h::set_error(B200_ERR_CUDA, "linear_nvfp4_static: cudaGetSymbolAddress failed: %s",
                              cudaGetErrorString(e));
    g_static_ptr[dev] = static_cast<uint8_t*>(p);
  }
  *out = g_static_ptr[dev];
  return B200_OK;
}
}  // namespace

extern "C" int b200tile_linear_nvfp4_static(const void* x, const void* y, const void* x_scales,
                                            const void* y_scales, void* z, const char* out_dtype, int m,
                                            int n, int k, int64_t ldx, int64_t ldy, int64_t ldz,
                                            int64_t ld_xs, int64_t ld_ys, float alpha, int config,
                                            void* cu_stream) {
  if (m <= 0 || n <= 0 || k <= 0)
    return b200h::set_error(B200_ERR_INVALID, "linear_nvfp4_static: Shape dimensions must be positive");
  if (config < -1 || config > 2)
    return b200h::set_error(B200_ERR_UNSUPPORTED, "linear_nvfp4_static: unknown config %d", config);
  static const int kBn[3] = {128, 192, 256};
  if (config < 0) config = m <= 32 ? 0 : 1;   // this entry's own default: single-CTA tiles (its scratch is sized for them)
  const int bn = kBn[config];
  const size_t need = b200::nvfp4_scratch_layout(m, n, k, bn, nullptr);
  if (need > (size_t)B200TILE_NVFP4_STATIC_SCRATCH_BYTES)
    return b200h::set_error(B200_ERR_INVALID,
                            "linear_nvfp4_static: the scales of a %d x %d x %d problem need %llu bytes of "
                            "scratch, the built-in buffer holds %llu; use b200tile_linear_nvfp4 with a "
                            "caller workspace",
                            m, n, k, (unsigned long long)need,
                            (unsigned long long)B200TILE_NVFP4_STATIC_SCRATCH_BYTES);
  uint8_t* scratch = nullptr;
  if (int rc = nvfp4_static_scratch_ptr(&scratch)) return rc;
  return b200tile_linear_nvfp4(x, y, x_scales, y_scales, z, out_dtype, m, n, k, ldx, ldy, ldz, ld_xs, ld_ys,
                               alpha, scratch, (uint64_t)B200TILE_NVFP4_STATIC_SCRATCH_BYTES, config,
                               cu_stream);
}

#ifdef B200TILE_TRACE
int b200_trace_read_fp4(long long* out) {
  if (cudaMemcpyFromSymbol(out, b200::g_trace_fp4, 8 * sizeof(long long)) != cudaSuccess) return 1;
  if (cudaMemcpyFromSymbol(out + 10, b200::g_trace_fp4_writer, 7 * sizeof(long long)) != cudaSuccess) return 1;
  return cudaMemcpyFromSymbol(out + 17, b200::g_trace_fp4_producer, 3 * sizeof(long long)) != cudaSuccess;
}
#endif
