// Attention forward for head_dim 128 with the softmax taken off the tensor-core chain.
//
// fmha_fwd.cu keeps S and P of a query tile in the same Tensor Memory columns, so per key tile the
// chain softmax -> P.V -> next Q.K^T runs in series and two query tiles per CTA only half hide it.
// Here a CTA owns ONE 128-row query tile at a time, two S buffers and two separate P buffers
// (2 x 128 + 2 x 64 + 128 columns of O fill the 512-column Tensor Memory).  An S buffer is free
// again as soon as the softmax has read it into registers, so S(j+2) is computed while the softmax
// of tiles j and j+1 is running; two softmax warpgroups take the key tiles alternately, and the
// Q.K^T and P.V MMAs are issued by two different threads (issuing one tcgen05.mma costs the issuing
// thread about as long as the MMA keeps the tensor pipe busy, so one thread with its waits and
// commits cannot keep the pipe fed).
//
// With one query tile per CTA the Q.K^T MMAs would need twice the shared-memory operand bandwidth
// per flop, so the CTAs work in pairs (cta_group::2): the leader issues M = 256 MMAs covering the
// query tile of each CTA, and each CTA loads and feeds only 64 of the 128 keys (S = Q K^T) and 64
// of the 128 value columns (O += P V) of every K/V tile.
//
// The kernel is persistent: a CTA pair walks a strided list of (256 query rows, batch*head) items,
// all barriers and rings run on across items, Q is double-buffered, and the only thing one item
// waits for from the previous one is the drained accumulator.  Pipeline fill and drain, which cost
// as much as five key tiles per item, are hidden that way.
//
// The two warpgroups share one running reference maximum per row: a thread decides the reference
// for its tile from the row maximum and the reference its partner thread (same row, other
// warpgroup) published for the previous tile, publishes it, and only then does the expensive part.
// The accumulator O is rescaled in place only when the reference moves by more than 2^8 (rare
// after the first tiles); each warpgroup keeps its own partial row sum relative to the reference it
// last saw and the two are merged at the end of the item.  Numerics are those of fmha_fwd.cu.
#include "fmha_common.cuh"
#include "host_common.h"
#include "sm100_ptx.cuh"
#include "trace.cuh"

namespace b200 {

#ifdef B200TILE_TRACE
// One CTA: the P.V thread's [0] V waits, [1] P waits, [2] P.V issue, [5] stage-release commits,
// [6] key tiles, [7] total cycles; the Q.K thread's [3] K waits, [4] waits for a free S buffer;
// [8] the total span in ns; softmax lane 0 of warpgroup 0 from [10]: S wait, TMEM load, max +
// reference hand-off, exp2 loop, store wait, P hand-off, key tiles, total.
__device__ long long g_trace_fmha_alt[20];
// Time line of the same CTA: for warpgroup 0 then warpgroup 1, (scores loaded, P handed over) of their
// tiles number 10..14, as SM clock values.
__device__ long long g_trace_fmha_alt_t[20];
#endif

struct FmhaAltSmem {
  static constexpr int D = 128;
  static constexpr int HALF_BYTES = 128 * 128;          // 128 rows x 128 bytes (one 64-wide column block)
  static constexpr int TILE_BYTES = 2 * HALF_BYTES;     // a 128 x 128 Q tile
  static constexpr int K_HALF = 64 * 128;               // this CTA's 64 keys, one column block
  static constexpr int K_BYTES = 2 * K_HALF;            // 64 keys x 128 dims
  static constexpr int V_BYTES = 128 * 128;             // 128 keys x this CTA's 64 value columns
  // K is consumed two key tiles before V: separate rings, each released as early as possible
  static constexpr int K_STAGES = 5;
  static constexpr int V_STAGES = 4;
  static constexpr int OFF_Q = 0;                       // two Q tiles: this item's and the next one's
  static constexpr int OFF_K = OFF_Q + 2 * TILE_BYTES;
  static constexpr int OFF_V = OFF_K + K_STAGES * K_BYTES;
  static constexpr int OFF_BAR = OFF_V + V_STAGES * V_BYTES;
  // q_full[2], q_empty[2], k_full[KS], k_empty[KS], v_full[VS], v_empty[VS], s_full[2], s_free[2],
  // p_full[2], o_free, m_pub[2][4]
  static constexpr int NUM_BARS = 4 + 2 * K_STAGES + 2 * V_STAGES + 6 + 1 + 8 + 2;
  static constexpr int OFF_MREF = OFF_BAR + NUM_BARS * 8;       // float[128] shared reference maximum
  static constexpr int OFF_LSUM = OFF_MREF + 128 * 4;           // float[2][128] partial sums, float[2][128] their references
  static constexpr int OFF_MISC = OFF_LSUM + 4 * 128 * 4;
  static constexpr int TOTAL = OFF_MISC + 16 + 1024;
};

// One work item of a CTA pair.
struct AltItem {
  int bh, kv_bh, q0, n_kv;
};

__device__ __forceinline__ AltItem alt_item(const FmhaParams& p, int idx, int rank, int input_pos, int n_total) {
  const int per_chunk = p.num_q_pairs * p.head_group;
  const int chunk = idx / per_chunk;
  const int r = idx - chunk * per_chunk;
  const int left = p.bh_total - chunk * p.head_group;
  const int gsz = left < p.head_group ? left : p.head_group;
  int qpair = r / gsz;
  AltItem it;
  it.bh = chunk * p.head_group + (r - qpair * gsz);
  if (p.causal) qpair = p.num_q_pairs - 1 - qpair;   // long rows first
  it.kv_bh = (it.bh / p.heads) * p.heads_kv + (it.bh % p.heads) / p.group;
  it.q0 = (qpair * 2 + rank) * FA_BM;
  // both CTAs walk the same key tiles: the count is that of the pair's last row
  it.n_kv = n_total;
  if (p.causal) {
    const int last = (qpair * 2 * FA_BM + 2 * FA_BM - 1 + input_pos) / FA_BN + 1;
    it.n_kv = last < n_total ? last : n_total;
  }
  return it;
}

template <bool OUT_F16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(FA_THREADS, 1)
fmha_fwd_alt_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, uint16_t* __restrict__ out, long long o_stride_bh,
                    long long o_stride_row, const FmhaParams p, uint32_t* status) {
  using L = FmhaAltSmem;
  constexpr int D = L::D;
  constexpr int KST = L::K_STAGES;
  constexpr int VST = L::V_STAGES;
  constexpr uint32_t HALF = L::HALF_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));

  const uint32_t sQ = base + L::OFF_Q;
  const uint32_t sK = base + L::OFF_K;
  const uint32_t sV = base + L::OFF_V;
  const uint32_t bar_q_full = base + L::OFF_BAR;            // leader [2]
  const uint32_t bar_q_empty = bar_q_full + 2 * 8;          // each CTA [2]
  const uint32_t bar_k_full = bar_q_empty + 2 * 8;          // leader
  const uint32_t bar_k_empty = bar_k_full + KST * 8;        // each CTA
  const uint32_t bar_v_full = bar_k_empty + KST * 8;        // leader
  const uint32_t bar_v_empty = bar_v_full + VST * 8;        // each CTA; also "P.V of that key tile has retired"
  const uint32_t bar_s_full = bar_v_empty + VST * 8;        // each CTA [2]
  const uint32_t bar_s_free = bar_s_full + 2 * 8;           // leader [2], 8 arrivals: S buffer read into registers
  const uint32_t bar_p_full = bar_s_free + 2 * 8;           // leader [2], 8 arrivals
  const uint32_t bar_o_free = bar_p_full + 2 * 8;           // leader, 16 arrivals: O read out of Tensor Memory
  const uint32_t bar_m_pub = bar_o_free + 8;                // each CTA: [warpgroup][quadrant]
  // each CTA [2], 4 arrivals: warpgroup w may start the exponentials of its next key tile, the other warpgroup has
  // finished its own.  The two warpgroups share the special-function unit; taking turns makes each exp2 loop ~1.5 k
  // cycles instead of ~1.75 k and measured 2-3 % on the whole kernel.
  const uint32_t bar_turn = bar_m_pub + 8 * 8;

  float* m_ref = reinterpret_cast<float*>(gen_base + L::OFF_MREF);
  float* l_part_sm = reinterpret_cast<float*>(gen_base + L::OFF_LSUM);
  float* m_part_sm = l_part_sm + 256;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(gen_base + L::OFF_MISC);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  WaitCtx wctx{misc + 1, status};

  const int input_pos = p.pos_ptr ? (int)__ldg(p.pos_ptr) : p.input_pos;
  const int n_total = (p.kv_len + FA_BN - 1) / FA_BN;
  const int total_items = p.num_q_pairs * p.bh_total;
  const int first_item = blockIdx.x >> 1;
  const int item_stride = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_q_full + i * 8, 1);
      mbar_init(bar_q_empty + i * 8, 1);
      mbar_init(bar_s_full + i * 8, 1);
      mbar_init(bar_s_free + i * 8, 8);   // four softmax warps from each CTA
      mbar_init(bar_p_full + i * 8, 8);
    }
    for (int s = 0; s < KST; ++s) {
      mbar_init(bar_k_full + s * 8, 1);
      mbar_init(bar_k_empty + s * 8, 1);
    }
    for (int s = 0; s < VST; ++s) {
      mbar_init(bar_v_full + s * 8, 1);
      mbar_init(bar_v_empty + s * 8, 1);
    }
    mbar_init(bar_o_free, 16);            // eight softmax warps from each CTA
    for (int i = 0; i < 8; ++i) mbar_init(bar_m_pub + i * 8, 1);
    for (int i = 0; i < 2; ++i) mbar_init(bar_turn + i * 8, 4);
    misc[1] = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
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
  // Tensor Memory columns: S[2] (fp32, 128 each), P[2] (16-bit pairs, 64 each), O (fp32, 128)
  auto S_COL = [](uint32_t b) { return b * 128u; };
  auto P_COL = [](uint32_t b) { return 256u + b * 64u; };
  constexpr uint32_t O_COL = 384;

  if (warp < 4) reg_dealloc<80>();   // 128 x 80 + 256 x 208 registers
  if (warp == 0) {
    // ---------------------------- TMA loader: Q and K ----------------------------
    if (lane == 0) {
      const uint32_t q_full_l = mapa_u32(bar_q_full, 0);
      const uint32_t k_full_l = mapa_u32(bar_k_full, 0);
      uint32_t stage = 0, phase = 0, n_item = 0;
      bool ok = true;
      for (int idx = first_item; idx < total_items && ok; idx += item_stride) {
        const AltItem it = alt_item(p, idx, (int)rank, input_pos, n_total);
        if (it.n_kv <= 0) continue;
        const uint32_t qb = n_item & 1, qph = (n_item >> 1) & 1;
        ++n_item;
        if (!mbar_wait(wctx, bar_q_empty + qb * 8, qph ^ 1, 12)) break;
        if (leader) mbar_expect_tx(bar_q_full + qb * 8, 2 * L::TILE_BYTES);
#pragma unroll
        for (int h = 0; h < 2; ++h)
          tma_load_3d_pair(sQ + qb * L::TILE_BYTES + h * HALF, &tmQ, q_full_l + qb * 8, h * 64, it.q0, it.bh);
        for (int j = 0; j < it.n_kv; ++j) {
          if (!mbar_wait(wctx, bar_k_empty + stage * 8, phase ^ 1, 10)) { ok = false; break; }
          const uint32_t k_dst = sK + stage * L::K_BYTES;
          if (leader) mbar_expect_tx(bar_k_full + stage * 8, 2 * L::K_BYTES);
#pragma unroll
          for (int h = 0; h < 2; ++h)
            tma_load_3d_pair(k_dst + h * L::K_HALF, &tmK, k_full_l + stage * 8, h * 64,
                             j * FA_BN + (int)rank * 64, it.kv_bh);
          if (++stage == KST) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 3) {
    // ------------------------------- TMA loader: V -------------------------------
    if (lane == 0) {
      const uint32_t v_full_l = mapa_u32(bar_v_full, 0);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int idx = first_item; idx < total_items && ok; idx += item_stride) {
        const AltItem it = alt_item(p, idx, (int)rank, input_pos, n_total);
        for (int j = 0; j < it.n_kv; ++j) {
          if (!mbar_wait(wctx, bar_v_empty + stage * 8, phase ^ 1, 11)) { ok = false; break; }
          if (leader) mbar_expect_tx(bar_v_full + stage * 8, 2 * L::V_BYTES);
          tma_load_3d_pair(sV + stage * L::V_BYTES, &tmV, v_full_l + stage * 8, (int)rank * 64, j * FA_BN, it.kv_bh);
          if (++stage == VST) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------- S = Q K^T issuer (leader CTA only), runs ahead of the softmax -------------
    if (leader) {
      // whole warp runs the loop, one elected lane issues (an issue loop under `if (lane == 0)` costs ~80 cycles
      // per MMA and per commit)
      const bool me = elect_one() != 0;
      constexpr uint32_t fmt = OUT_F16 ? FMT_F16 : FMT_BF16;
      constexpr uint32_t idesc_qk = make_idesc(fmt, fmt, 0, 0, 2 * FA_BM, FA_BN);
      const uint32_t s_full_peer = mapa_u32(bar_s_full, 1);
      const uint32_t k_empty_peer = mapa_u32(bar_k_empty, 1);
      const uint32_t q_empty_peer = mapa_u32(bar_q_empty, 1);
      uint32_t ks = 0, kph = 0, g = 0, n_item = 0;   // g: key tiles issued so far, over all items
      bool ok = true;
#ifdef B200TILE_TRACE
      long long qk_wait_k = 0, qk_wait_s = 0;
#endif
      for (int idx = first_item; idx < total_items && ok; idx += item_stride) {
        const AltItem it = alt_item(p, idx, 0, input_pos, n_total);
        if (it.n_kv <= 0) continue;
        const uint32_t qb = n_item & 1, qph = (n_item >> 1) & 1;
        ++n_item;
        if (!__all_sync(0xffffffffu, mbar_wait(wctx, bar_q_full + qb * 8, qph, 21))) break;
        const uint32_t q_addr = sQ + qb * L::TILE_BYTES;
        for (int j = 0; j < it.n_kv; ++j, ++g) {
          const uint32_t sb = g & 1;
#ifdef B200TILE_TRACE
          const long long c0 = clock64();
#endif
          if (!__all_sync(0xffffffffu, mbar_wait(wctx, bar_k_full + ks * 8, kph, 20))) { ok = false; break; }
#ifdef B200TILE_TRACE
          const long long c1 = clock64();
          qk_wait_k += c1 - c0;
#endif
          if (g >= 2) {
            // the softmax warps of both CTAs have read S(g - 2) out of buffer sb
            if (!__all_sync(0xffffffffu, mbar_wait(wctx, bar_s_free + sb * 8, ((g >> 1) - 1) & 1u, 23))) { ok = false; break; }
          }
#ifdef B200TILE_TRACE
          qk_wait_s += clock64() - c1;
#endif
          tc_fence_after_sync();
          const uint32_t k_addr = sK + ks * L::K_BYTES;
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t a = make_smem_desc(q_addr + (kk / 4) * HALF + (kk % 4) * 32, 16, 1024, SWZ_128B);
            const uint64_t bd = make_smem_desc(k_addr + (kk / 4) * L::K_HALF + (kk % 4) * 32, 16, 1024, SWZ_128B);
            if (me) umma_f16_ss_2cta(tmem_base + S_COL(sb), a, bd, idesc_qk, kk != 0);
          }
          if (me) umma_commit_2cta(bar_s_full + sb * 8);
          if (me) umma_commit_2cta(s_full_peer + sb * 8);
          if (me) umma_commit_2cta(bar_k_empty + ks * 8);
          if (me) umma_commit_2cta(k_empty_peer + ks * 8);
          if (++ks == KST) { ks = 0; kph ^= 1; }
        }
        // every Q.K^T of the item has been issued: its Q tile is free once they retire
        if (me) umma_commit_2cta(bar_q_empty + qb * 8);
        if (me) umma_commit_2cta(q_empty_peer + qb * 8);
      }
#ifdef B200TILE_TRACE
      if (lane == 0) {
        misc[2] = (uint32_t)qk_wait_k;   // read by the P.V thread, which finishes later
        misc[3] = (uint32_t)qk_wait_s;
      }
#endif
    }
  } else if (warp == 2) {
    // ------------------------- O += P V issuer (leader CTA only) -------------------------
    if (leader) {
      const bool me = elect_one() != 0;
      constexpr uint32_t fmt = OUT_F16 ? FMT_F16 : FMT_BF16;
      constexpr uint32_t idesc_pv = make_idesc(fmt, fmt, 0, 1, 2 * FA_BM, D);
      const uint32_t v_empty_peer = mapa_u32(bar_v_empty, 1);
      bool ok = true;
      B200_TR_DECL(7);
      uint32_t vs = 0, vph = 0, g = 0, n_item = 0;
      for (int idx = first_item; idx < total_items && ok; idx += item_stride) {
        const AltItem it = alt_item(p, idx, 0, input_pos, n_total);
        if (it.n_kv <= 0) continue;
        // the previous item's accumulator has been read out by all softmax warps of both CTAs
        if (n_item > 0 && !__all_sync(0xffffffffu, mbar_wait(wctx, bar_o_free, (n_item - 1) & 1u, 25))) break;
        ++n_item;
        for (int j = 0; j < it.n_kv; ++j, ++g) {
          const uint32_t pb = g & 1, pph = (g >> 1) & 1;
          B200_TR_COUNT(6);
          B200_TR_BEGIN();
          if (!__all_sync(0xffffffffu, mbar_wait(wctx, bar_v_full + vs * 8, vph, 22))) { ok = false; break; }
          B200_TR_END(0);
          B200_TR_BEGIN();
          if (!__all_sync(0xffffffffu, mbar_wait(wctx, bar_p_full + pb * 8, pph, 24))) { ok = false; break; }
          tc_fence_after_sync();
          B200_TR_END(1);
          B200_TR_BEGIN();
          const uint32_t v_addr = sV + vs * L::V_BYTES;
#pragma unroll
          for (int kk = 0; kk < FA_BN / 16; ++kk) {
            // V is the N-major B operand; each CTA holds one 64-column block, 16 key rows per step
            const uint64_t bd = make_smem_desc(v_addr + kk * 2048, HALF, 1024, SWZ_128B);
            if (me) umma_f16_ts_2cta(tmem_base + O_COL, tmem_base + P_COL(pb) + kk * 8, bd, idesc_pv, j > 0 || kk != 0);
          }
          B200_TR_END(2);
          // V(g) is free in both CTAs; the same signal tells the softmax warps that O holds key tile g
          B200_TR_BEGIN();
          if (me) umma_commit_2cta(bar_v_empty + vs * 8);
          if (me) umma_commit_2cta(v_empty_peer + vs * 8);
          B200_TR_END(5);
          if (++vs == VST) { vs = 0; vph ^= 1; }
        }
      }
#ifdef B200TILE_TRACE
      tr_[3] = misc[2];
      tr_[4] = misc[3];
#endif
      B200_TR_FLUSH(g_trace_fmha_alt, 7, blockIdx.x == 14 && lane == 0);
    }
  } else if (warp >= 4) {
    // -------------------------------- softmax ----------------------------------
    reg_alloc<FA_SOFTMAX_REGS>();
    const uint32_t w = (uint32_t)(warp - 4) >> 2;   // warpgroup: key tiles with (running index & 1) == w
    const int q = warp & 3;
    const int row = q * 32 + lane;                  // row inside the tile == TMEM lane
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    const uint32_t tS = lane_base + S_COL(w);
    const uint32_t tP = lane_base + P_COL(w);
    const uint32_t tO = lane_base + O_COL;
    const uint32_t my_pub = bar_m_pub + (w * 4 + (uint32_t)q) * 8;
    const uint32_t other_pub = bar_m_pub + ((1 - w) * 4 + (uint32_t)q) * 8;
    const uint32_t s_free_l = mapa_u32(bar_s_free + w * 8, 0);
    const uint32_t p_full_l = mapa_u32(bar_p_full + w * 8, 0);
    const uint32_t o_free_l = mapa_u32(bar_o_free, 0);
    const float scale = p.scale_log2;
    bool ok = true;
    uint32_t g0 = 0;                                // key tiles of the items before this one
    B200_TR_DECL(7);
    for (int idx = first_item; idx < total_items; idx += item_stride) {
      const AltItem it = alt_item(p, idx, (int)rank, input_pos, n_total);
      if (it.n_kv <= 0) continue;
      const int row_g = it.q0 + row;                // query position
      float m_seen = -CUDART_INF_F, l_part = 0.0f;  // this warpgroup's row sum, relative to m_seen
      for (int j = (int)((g0 ^ w) & 1u); j < it.n_kv && ok; j += 2) {
        const uint32_t g = g0 + (uint32_t)j;
        B200_TR_COUNT(6);
        B200_TR_BEGIN();
        if (!mbar_wait(wctx, bar_s_full + w * 8, (g >> 1) & 1u, 30)) { ok = false; break; }
        tc_fence_after_sync();
        B200_TR_END(0);
        B200_TR_BEGIN();
        // the whole score row lives in registers: one TMEM read per element
        uint32_t v[FA_BN];
#pragma unroll
        for (int c = 0; c < FA_BN / 32; ++c)
          tmem_ld_32x32b_x32(tS + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
        // last key column this row may see inside this tile (>= 127: nothing masked)
        int lim = p.kv_len - 1 - j * FA_BN;
        if (p.causal) {
          const int c = row_g + input_pos - j * FA_BN;
          lim = c < lim ? c : lim;
        }
        const bool masked_tile = __any_sync(0xffffffffu, lim < FA_BN - 1);
        tmem_wait_ld();
#ifdef B200TILE_TRACE
        if (blockIdx.x == 14 && q == 0 && lane == 0 && (g >> 1) >= 10 && (g >> 1) < 15)
          g_trace_fmha_alt_t[w * 10 + ((g >> 1) - 10) * 2] = clock64();
#endif
        // the scores are in registers: the buffer can take S(g + 2) while this tile is worked on
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_addr_cta_release(s_free_l);
        B200_TR_END(1);
        B200_TR_BEGIN();
        if (masked_tile) {
#pragma unroll
          for (int i = 0; i < FA_BN; ++i)
            if (i > lim) v[i] = 0xff800000u;  // -inf
        }
        // row maximum: four independent chains
        float mx[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
        for (int i = 0; i < FA_BN; i += 8) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            mx[u] = max3(mx[u], __uint_as_float(v[i + 2 * u]), __uint_as_float(v[i + 2 * u + 1]));
        }
        const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale;
        // reference maximum of this tile: the partner's reference unless the row maximum outgrew it
        float m_new, alpha = 1.0f;
        bool need = false;
        if (j == 0) {
          m_new = m_tile == -CUDART_INF_F ? 0.0f : m_tile;  // fully masked row: keep exp2 arguments finite
        } else {
          if (!mbar_wait(wctx, other_pub, ((g - 1) >> 1) & 1u, 32)) { ok = false; break; }
          const float m_old = m_ref[row];
          m_new = m_old;
          if (m_tile - m_old > FA_RESCALE_THRESHOLD) {
            need = true;
            m_new = m_tile;
            alpha = ex2_approx(m_old - m_new);
          }
        }
        m_ref[row] = m_new;
        __syncwarp();
        if (lane == 0) mbar_arrive(my_pub);
        if (m_new != m_seen) {
          l_part *= ex2_approx(m_seen - m_new);
          m_seen = m_new;
        }
        if (j > 0 && __any_sync(0xffffffffu, need)) {
          // O must hold key tile g-1 before it is rescaled; P.V of tile g cannot start before this
          // warp has handed over P(g), and the partner's rescale for tile g+1 waits for that P.V
          const uint32_t gp = g - 1;
          if (!mbar_wait(wctx, bar_v_empty + (gp % VST) * 8, (gp / VST) & 1u, 33)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(tO + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32b_x32(tO + c * 32, o);
          }
        }
        B200_TR_END(2);
        B200_TR_BEGIN();
        if (g >= 2) {
          // P(g - 2) must have been consumed before its buffer is overwritten
          const uint32_t gp = g - 2;
          if (!mbar_wait(wctx, bar_v_empty + (gp % VST) * 8, (gp / VST) & 1u, 34)) { ok = false; break; }
          tc_fence_after_sync();
        }
        // the exponentials of key tile g - 1 (the other warpgroup's) are done: the special-function unit is ours
        if (g >= 1 && !mbar_wait(wctx, bar_turn + w * 8, ((g - 1) >> 1) & 1u, 35)) { ok = false; break; }
        // probabilities: exp2(s*scale - m); masked entries are exp2(-inf) = 0
        const float neg_m = -m_new;
        const uint64_t scale2 = pack2(scale, scale), negm2 = pack2(neg_m, neg_m);
        uint64_t ls2[4] = {0ull, 0ull, 0ull, 0ull};  // four packed (even, odd) partial sums
#pragma unroll
        for (int c = 0; c < FA_BN / 32; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const uint64_t x2 = fma2(pack2(__uint_as_float(v[c * 32 + 2 * i]),
                                           __uint_as_float(v[c * 32 + 2 * i + 1])), scale2, negm2);
            float xa, xb;
            unpack2(x2, xa, xb);
            const float a = ex2_approx(xa), bb = ex2_approx(xb);
            ls2[i & 3] = add2(ls2[i & 3], pack2(a, bb));
            pk[i] = OUT_F16 ? pack_f16x2(a, bb) : pack_bf16x2(a, bb);
          }
          tmem_st_32x32b_x16(tP + c * 16, pk);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_turn + (1 - w) * 8);
        float ls[4];
        {
          const uint64_t s01 = add2(ls2[0], ls2[1]), s23 = add2(ls2[2], ls2[3]);
          unpack2(s01, ls[0], ls[1]);
          unpack2(s23, ls[2], ls[3]);
        }
        l_part += (ls[0] + ls[1]) + (ls[2] + ls[3]);
        B200_TR_END(3);
        B200_TR_BEGIN();
        tmem_wait_st();
        B200_TR_END(4);
        B200_TR_BEGIN();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_addr_cta_release(p_full_l);
#ifdef B200TILE_TRACE
        if (blockIdx.x == 14 && q == 0 && lane == 0 && (g >> 1) >= 10 && (g >> 1) < 15)
          g_trace_fmha_alt_t[w * 10 + ((g >> 1) - 10) * 2 + 1] = clock64();
#endif
        B200_TR_END(5);
      }
      // ---- end of the item: merge the two warpgroups' row sums under the final reference ----
      l_part_sm[w * 128 + row] = l_part;
      m_part_sm[w * 128 + row] = m_seen;
      named_bar_sync(1, 256);
      const float m_fin = m_ref[row];
      const float l_run = l_part_sm[row] * ex2_approx(m_part_sm[row] - m_fin) +
                          l_part_sm[128 + row] * ex2_approx(m_part_sm[128 + row] - m_fin);
      named_bar_sync(1, 256);   // the next item may overwrite the reference and the partial sums
      const uint32_t g_last = g0 + (uint32_t)it.n_kv - 1;
      g0 += (uint32_t)it.n_kv;
      if (ok && mbar_wait(wctx, bar_v_empty + (g_last % VST) * 8, (g_last / VST) & 1u, 31)) {
        tc_fence_after_sync();
        // warpgroup w takes value columns [64w, 64w + 64) of its 32 rows per warp
        uint32_t o[64];
        tmem_ld_32x32b_x32(tO + w * 64, *reinterpret_cast<uint32_t(*)[32]>(&o[0]));
        tmem_ld_32x32b_x32(tO + w * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&o[32]));
        tmem_wait_ld();
        // the accumulator is in registers: the next item's first P.V may overwrite it
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_addr_cta_release(o_free_l);
        if (row_g < p.q_len) {
          const float inv_l = 1.0f / fmaxf(l_run, 1e-8f);  // attention.rs:385-390
          uint16_t* dst = out + (long long)it.bh * o_stride_bh + (long long)row_g * o_stride_row + w * 64;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            uint32_t wd[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              const float lo = __uint_as_float(o[e * 8 + 2 * x]) * inv_l;
              const float hi = __uint_as_float(o[e * 8 + 2 * x + 1]) * inv_l;
              wd[x] = OUT_F16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
            }
            *reinterpret_cast<uint4*>(dst + e * 8) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
          }
        }
      } else {
        ok = false;
      }
    }
    B200_TR_FLUSH(g_trace_fmha_alt + 10, 7, blockIdx.x == 14 && warp == 4 && lane == 0);
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while its partner may still signal its barriers
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_2cta(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------
// Host launch
// ---------------------------------------------------------------------------
template <bool OUT_F16>
static int launch_fmha_alt(const void* q, const void* k, const void* v, void* o, int batch, int heads, int heads_kv,
                           int q_len, int kv_len, const int64_t* qs, const int64_t* ks, const int64_t* vs,
                           const int64_t* os, float qk_scale, int causal, int input_pos, const uint32_t* pos_ptr,
                           cudaStream_t stream) {
  using L = FmhaAltSmem;
  constexpr int D = L::D;
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  const CUtensorMapDataType dt = OUT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmQ, tmK, tmV;
  int rc;
  const uint64_t bh = (uint64_t)batch * heads, bhkv = (uint64_t)batch * heads_kv;
  if ((rc = b200h::encode_tmap_3d(&tmQ, dt, 2, q, D, q_len, bh, qs[1] * 2, qs[0] * 2, 64, FA_BM, 1,
                                  CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  // K arrives as 64-key boxes (one per CTA of the pair), V as 128 keys x one 64-column block
  if ((rc = b200h::encode_tmap_3d(&tmK, dt, 2, k, D, kv_len, bhkv, ks[1] * 2, ks[0] * 2, 64, 64, 1,
                                  CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  if ((rc = b200h::encode_tmap_3d(&tmV, dt, 2, v, D, kv_len, bhkv, vs[1] * 2, vs[0] * 2, 64, FA_BN, 1,
                                  CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  // the output is written with 16-byte stores straight from registers
  if ((reinterpret_cast<uintptr_t>(o) & 15) || (os[0] & 7) || (os[1] & 7))
    return b200h::set_error(B200_ERR_ALIGN, "fmha: output base and pitches must be multiples of 16 bytes");
  auto kern = fmha_fwd_alt_kernel<OUT_F16>;
  static b200h::DeviceOnce attr_done;
  if (!attr_done.test(di->ordinal)) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    attr_done.set(di->ordinal);
  }
  FmhaParams p;
  p.q_len = q_len;
  p.kv_len = kv_len;
  p.num_q_pairs = (q_len + 2 * FA_BM - 1) / (2 * FA_BM);   // 256-row pairs per (batch, head)
  p.bh_total = (int)bh;
  p.heads = heads;
  p.heads_kv = heads_kv;
  p.group = heads / heads_kv;
  p.causal = causal;
  p.input_pos = input_pos;
  p.pos_ptr = pos_ptr;
  p.head_group = 8;
  p.scale_log2 = qk_scale * 1.4426950408889634f;
  const long long items = (long long)p.num_q_pairs * p.bh_total;
  if (items > 0x3fffffffLL) return b200h::set_error(B200_ERR_INVALID, "fmha: grid too large");
  // one CTA pair per two SMs, each walking items pair, pair + pairs, ...
  const long long pairs = items < di->sm_count / 2 ? items : di->sm_count / 2;
  if (pairs <= 0) return B200_OK;
  kern<<<(unsigned)(2 * pairs), FA_THREADS, L::TOTAL, stream>>>(tmQ, tmK, tmV, static_cast<uint16_t*>(o),
                                                                (long long)os[0], (long long)os[1], p, di->status);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

}  // namespace b200

// dtype: 0 = bf16, 1 = f16; head_dim 128 only.  Same argument meaning as b200_fmha_fwd_dispatch.
int b200_fmha_fwd_alt_dispatch(int dtype, const void* q, const void* k, const void* v, void* o, int batch, int heads,
                               int heads_kv, int q_len, int kv_len, const int64_t* qs, const int64_t* ks,
                               const int64_t* vs, const int64_t* os, float qk_scale, int causal, int input_pos,
                               const uint32_t* pos_ptr, cudaStream_t stream) {
  using namespace b200;
  return dtype ? launch_fmha_alt<true>(q, k, v, o, batch, heads, heads_kv, q_len, kv_len, qs, ks, vs, os, qk_scale,
                                       causal, input_pos, pos_ptr, stream)
               : launch_fmha_alt<false>(q, k, v, o, batch, heads, heads_kv, q_len, kv_len, qs, ks, vs, os, qk_scale,
                                        causal, input_pos, pos_ptr, stream);
}

#ifdef B200TILE_TRACE
int b200_trace_read_fmha_alt(long long* out) {
  return cudaMemcpyFromSymbol(out, b200::g_trace_fmha_alt, 20 * sizeof(long long)) != cudaSuccess;
}
int b200_trace_read_fmha_alt_t(long long* out) {
  return cudaMemcpyFromSymbol(out, b200::g_trace_fmha_alt_t, 20 * sizeof(long long)) != cudaSuccess;
}
#endif
