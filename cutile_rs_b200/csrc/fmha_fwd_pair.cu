// Attention forward on CTA pairs (cta_group::2) for head_dim 128.
//
// Same algorithm, numerics and role layout as fmha_fwd.cu (which documents them and cites the
// reference kernels it replaces); what changes is the MMA shape.  A 128x128x16 MMA with both
// operands in shared memory asks one SM for 8 KiB of operands every 64 tensor-pipe cycles, more
// than shared memory delivers to the tensor core (measured: ~100 cycles per such MMA against 63
// for the P.V MMAs whose A operand sits in Tensor Memory).  Two CTAs of a cluster therefore share
// every K and V tile: one thread of the leader issues M = 256 MMAs that cover one query tile of
// each CTA; the B operand is split between the CTAs by the hardware, so each CTA loads and feeds
// only 64 of the 128 keys (S = Q K^T) and 64 of the 128 value columns (O += P V).  Per CTA that
// is 6 KiB instead of 8 KiB of operands per S MMA and half the K/V traffic into shared memory.
//
// A cluster owns FOUR consecutive 128-row query tiles of one (batch, head): CTA r works on tiles
// 4c + r and 4c + 2 + r (slot 0 and slot 1), ping-ponging between its two slots exactly like the
// single-CTA kernel does.  Barriers that the MMA thread waits on live in the leader and count both
// CTAs; barriers that release shared memory or publish S / O live in each CTA and are signalled
// with one commit per CTA.
#include "fmha_common.cuh"
#include "host_common.h"
#include "sm100_ptx.cuh"
#include "trace.cuh"

namespace b200 {

#ifdef B200TILE_TRACE
// One CTA: MMA thread [0] K/V waits, [1] P waits, [2] P.V issue, [3] Q.K issue, [4] S commits,
// [5] stage-release commits, [6] key tiles, [7] total cycles; [8] the same span in ns; softmax lane 0 of tile 0 from [10]:
// S wait, TMEM load, max and rescale, exp2 loop, store wait, hand-off, key tiles, total.
__device__ long long g_trace_fmha_pair[20];
#endif

struct FmhaPairSmem {
  static constexpr int D = 128;
  static constexpr int HALF_BYTES = 128 * 128;          // 128 rows x 128 bytes (one 64-wide column block)
  static constexpr int TILE_BYTES = 2 * HALF_BYTES;     // a 128 x 128 Q tile
  static constexpr int K_HALF = 64 * 128;               // this CTA's 64 keys, one column block
  static constexpr int K_BYTES = 2 * K_HALF;            // 64 keys x 128 dims
  static constexpr int V_BYTES = 128 * 128;             // 128 keys x this CTA's 64 value columns
  static constexpr int STAGE_BYTES = K_BYTES + V_BYTES;
  static constexpr int STAGES = 4;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_KV = OFF_Q + 2 * TILE_BYTES;
  static constexpr int OFF_BAR = OFF_KV + STAGES * STAGE_BYTES;
  // q_full[2], k_full[S], v_full[S], kv_empty[S], s_full[2], p_full[2], o_done[2]
  static constexpr int NUM_BARS = 2 + 3 * STAGES + 6;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
  static constexpr int TOTAL = OFF_MISC + 16 + 1024;
};

template <bool OUT_F16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(FA_THREADS, 1)
fmha_fwd_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                     const FmhaParams p, uint32_t* status) {
  using L = FmhaPairSmem;
  constexpr int D = L::D;
  constexpr int STAGES = L::STAGES;
  constexpr uint32_t HALF = L::HALF_BYTES;
  constexpr uint32_t TILE = L::TILE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));

  const uint32_t sQ = base + L::OFF_Q;
  const uint32_t sKV = base + L::OFF_KV;
  const uint32_t bar_q_full = base + L::OFF_BAR;            // leader
  const uint32_t bar_k_full = bar_q_full + 2 * 8;           // leader
  const uint32_t bar_v_full = bar_k_full + STAGES * 8;      // leader
  const uint32_t bar_kv_empty = bar_v_full + STAGES * 8;    // each CTA
  const uint32_t bar_s_full = bar_kv_empty + STAGES * 8;    // each CTA
  const uint32_t bar_p_full = bar_s_full + 2 * 8;           // leader, 8 arrivals
  const uint32_t bar_o_done = bar_p_full + 2 * 8;           // each CTA
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(gen_base + L::OFF_MISC);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  WaitCtx wctx{misc + 1, status};

  // ---- work item of the cluster: head-group swizzle, longest causal rows first ----
  int quad, bh;
  {
    const int idx = blockIdx.x >> 1;
    const int per_chunk = p.num_q_pairs * p.head_group;   // num_q_pairs holds the number of 512-row quads here
    const int chunk = idx / per_chunk;
    const int r = idx - chunk * per_chunk;
    const int left = p.bh_total - chunk * p.head_group;
    const int gsz = left < p.head_group ? left : p.head_group;
    quad = r / gsz;
    bh = chunk * p.head_group + (r - quad * gsz);
    if (p.causal) quad = p.num_q_pairs - 1 - quad;
  }
  const int input_pos = p.pos_ptr ? (int)__ldg(p.pos_ptr) : p.input_pos;
  const int kv_bh = (bh / p.heads) * p.heads_kv + (bh % p.heads) / p.group;
  const int n_total = (p.kv_len + FA_BN - 1) / FA_BN;
  // slot t: this CTA's tile 4*quad + 2t + rank; the key-tile count is the slot's (the later tile's)
  int q0[2], n_kv[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    q0[t] = (quad * 4 + 2 * t + (int)rank) * FA_BM;
    const int first_row = (quad * 4 + 2 * t) * FA_BM;       // CTA 0's tile of the slot
    if (first_row >= p.q_len) {
      n_kv[t] = 0;
    } else if (p.causal) {
      const int last = (first_row + 2 * FA_BM - 1 + input_pos) / FA_BN + 1;
      n_kv[t] = last < n_total ? last : n_total;
    } else {
      n_kv[t] = n_total;
    }
  }
  const int n_max = n_kv[0] > n_kv[1] ? n_kv[0] : n_kv[1];

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_q_full + i * 8, 1);
      mbar_init(bar_s_full + i * 8, 1);
      mbar_init(bar_p_full + i * 8, 8);   // four softmax warps from each CTA
      mbar_init(bar_o_done + i * 8, 1);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_k_full + s * 8, 1);
      mbar_init(bar_v_full + s * 8, 1);
      mbar_init(bar_kv_empty + s * 8, 1);
    }
    misc[1] = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmO);
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
  auto S_COL = [](int t) { return (uint32_t)(t * 128); };
  auto O_COL = [](int t) { return (uint32_t)(256 + t * 128); };

  if (warp < 4) reg_dealloc<FA_OTHER_REGS>();
  if (warp == 0) {
    // ------------------------------- TMA loader -------------------------------
    if (lane == 0) {
      const uint32_t q_full_l = mapa_u32(bar_q_full, 0);
      const uint32_t k_full_l = mapa_u32(bar_k_full, 0);
      const uint32_t v_full_l = mapa_u32(bar_v_full, 0);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (n_kv[t] == 0) continue;
        if (leader) mbar_expect_tx(bar_q_full + t * 8, 2 * TILE);
#pragma unroll
        for (int h = 0; h < 2; ++h)
          tma_load_3d_pair(sQ + t * TILE + h * HALF, &tmQ, q_full_l + t * 8, h * 64, q0[t], bh);
      }
      uint32_t stage = 0, phase = 0;
      for (int j = 0; j < n_max; ++j) {
        if (!mbar_wait(wctx, bar_kv_empty + stage * 8, phase ^ 1, 10)) break;
        const uint32_t k_dst = sKV + stage * L::STAGE_BYTES, v_dst = k_dst + L::K_BYTES;
        if (leader) mbar_expect_tx(bar_k_full + stage * 8, 2 * L::K_BYTES);
#pragma unroll
        for (int h = 0; h < 2; ++h)
          tma_load_3d_pair(k_dst + h * L::K_HALF, &tmK, k_full_l + stage * 8, h * 64,
                           j * FA_BN + (int)rank * 64, kv_bh);
        if (leader) mbar_expect_tx(bar_v_full + stage * 8, 2 * L::V_BYTES);
        tma_load_3d_pair(v_dst, &tmV, v_full_l + stage * 8, (int)rank * 64, j * FA_BN, kv_bh);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---------------------- MMA issuer (leader CTA only) -----------------------
    if (leader && lane == 0 && n_max > 0) {
      constexpr uint32_t fmt = OUT_F16 ? FMT_F16 : FMT_BF16;
      constexpr uint32_t idesc_qk = make_idesc(fmt, fmt, 0, 0, 2 * FA_BM, FA_BN);
      constexpr uint32_t idesc_pv = make_idesc(fmt, fmt, 0, 1, 2 * FA_BM, D);
      auto commit_both = [&](uint32_t bar) {
        umma_commit_2cta(bar);
        umma_commit_2cta(mapa_u32(bar, 1));
      };
      auto issue_qk = [&](int t, uint32_t k_addr) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t a = make_smem_desc(sQ + t * TILE + (kk / 4) * HALF + (kk % 4) * 32, 16, 1024, SWZ_128B);
          const uint64_t b = make_smem_desc(k_addr + (kk / 4) * L::K_HALF + (kk % 4) * 32, 16, 1024, SWZ_128B);
          umma_f16_ss_2cta(tmem_base + S_COL(t), a, b, idesc_qk, kk != 0);
        }
      };
      auto issue_pv = [&](int t, uint32_t v_addr, bool acc) {
#pragma unroll
        for (int kk = 0; kk < FA_BN / 16; ++kk) {
          // V is the N-major B operand; each CTA holds one 64-column block, 16 key rows per step
          const uint64_t b = make_smem_desc(v_addr + kk * 2048, HALF, 1024, SWZ_128B);
          umma_f16_ts_2cta(tmem_base + O_COL(t), tmem_base + S_COL(t) + kk * 8, b, idesc_pv, acc || kk != 0);
        }
      };
      bool ok = true;
      B200_TR_DECL(7);
      // prologue: S_t(0) = Q_t K(0)^T
      ok = mbar_wait(wctx, bar_k_full + 0, 0, 20);
#pragma unroll
      for (int t = 0; t < 2 && ok; ++t) {
        if (n_kv[t] == 0) continue;
        if (!mbar_wait(wctx, bar_q_full + t * 8, 0, 21)) { ok = false; break; }
        tc_fence_after_sync();
        issue_qk(t, sKV);
        commit_both(bar_s_full + t * 8);
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const uint32_t vs = j % STAGES, vph = (j / STAGES) & 1;
        const uint32_t ks = (j + 1) % STAGES, kph = ((j + 1) / STAGES) & 1;
        const bool have_next = j + 1 < n_max;
        B200_TR_COUNT(6);
        B200_TR_BEGIN();
        if (!mbar_wait(wctx, bar_v_full + vs * 8, vph, 22)) { ok = false; break; }
        if (have_next && !mbar_wait(wctx, bar_k_full + ks * 8, kph, 23)) { ok = false; break; }
        tc_fence_after_sync();
        B200_TR_END(0);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j < n_kv[t]) {
            B200_TR_BEGIN();
            if (!mbar_wait(wctx, bar_p_full + t * 8, j & 1, 24)) { ok = false; break; }
            tc_fence_after_sync();
            B200_TR_END(1);
            B200_TR_BEGIN();
            issue_pv(t, sKV + vs * L::STAGE_BYTES + L::K_BYTES, j > 0);
            B200_TR_END(2);
            if (j == n_kv[t] - 1) commit_both(bar_o_done + t * 8);
          }
          if (j + 1 < n_kv[t]) {
            B200_TR_BEGIN();
            issue_qk(t, sKV + ks * L::STAGE_BYTES);
            B200_TR_END(3);
            B200_TR_BEGIN();
            commit_both(bar_s_full + t * 8);
            B200_TR_END(4);
          }
        }
        if (!ok) break;
        // K(j) was consumed an iteration ago and V(j) just now: stage j is free in both CTAs
        B200_TR_BEGIN();
        commit_both(bar_kv_empty + vs * 8);
        B200_TR_END(5);
      }
      B200_TR_FLUSH(g_trace_fmha_pair, 7, blockIdx.x == 14);
    }
  } else if (warp >= 4) {
    // -------------------------------- softmax ----------------------------------
    reg_alloc<FA_SOFTMAX_REGS>();
    const int t = (warp - 4) >> 2;
    const int q = warp & 3;
    const int row = q * 32 + lane;          // row inside the tile == TMEM lane
    const int row_g = q0[t] + row;          // query position
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    const uint32_t tS = lane_base + S_COL(t);
    const uint32_t tO = lane_base + O_COL(t);
    const int n_mine = n_kv[t];
    const uint32_t p_full_leader = mapa_u32(bar_p_full + t * 8, 0);
    const float scale = p.scale_log2;
    float m_run = -CUDART_INF_F, l_run = 0.0f;
    bool ok = true;
    B200_TR_DECL(7);
    for (int j = 0; j < n_mine && ok; ++j) {
      B200_TR_COUNT(6);
      B200_TR_BEGIN();
      if (!mbar_wait(wctx, bar_s_full + t * 8, j & 1, 30)) { ok = false; break; }
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
      const float rmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      const float m_tile = rmax * scale;
      float m_new = fmaxf(m_run, m_tile);
      if (m_new == -CUDART_INF_F) m_new = 0.0f;  // fully masked row: keep exp2 arguments finite
      float alpha = 1.0f;
      bool need = false;
      if (j == 0) {
        m_run = m_new;
      } else if (m_new - m_run > FA_RESCALE_THRESHOLD) {
        need = true;
        alpha = ex2_approx(m_run - m_new);
        l_run *= alpha;
        m_run = m_new;
      }
      if (j > 0 && __any_sync(0xffffffffu, need)) {
        // S_t(j) complete implies O_t += P_t(j-1) V(j-1) complete (MMAs retire in issue order)
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
      // probabilities: exp2(s*scale - m); masked entries are exp2(-inf) = 0
      B200_TR_END(2);
      B200_TR_BEGIN();
      const float neg_m = -m_run;
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
          const float a = ex2_approx(xa), b = ex2_approx(xb);
          ls2[i & 3] = add2(ls2[i & 3], pack2(a, b));
          pk[i] = OUT_F16 ? pack_f16x2(a, b) : pack_bf16x2(a, b);
        }
        tmem_st_32x32b_x16(tS + c * 16, pk);
      }
      float ls[4];
      {
        const uint64_t s01 = add2(ls2[0], ls2[1]), s23 = add2(ls2[2], ls2[3]);
        unpack2(s01, ls[0], ls[1]);
        unpack2(s23, ls[2], ls[3]);
      }
      l_run += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      B200_TR_END(3);
      B200_TR_BEGIN();
      tmem_wait_st();
      B200_TR_END(4);
      B200_TR_BEGIN();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster_addr_cta_release(p_full_leader);
      B200_TR_END(5);
    }
    B200_TR_FLUSH(g_trace_fmha_pair + 10, 7, blockIdx.x == 14 && warp == 4 && lane == 0);
    // ------------------------------- epilogue ----------------------------------
    if (n_mine > 0 && ok) {
      if (mbar_wait(wctx, bar_o_done + t * 8, 0, 31)) {
        tc_fence_after_sync();
        const float inv_l = 1.0f / fmaxf(l_run, 1e-8f);  // attention.rs:385-390
        // Q_t's shared memory is free now (all S_t MMAs retired): stage O there
        const uint32_t stage_row = sQ + t * TILE + (uint32_t)row * 128;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(tO + c * 32, o);
          tmem_wait_ld();
          const uint32_t half_base = stage_row + (c >> 1) * HALF;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint32_t w[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              const float lo = __uint_as_float(o[e * 8 + 2 * x]) * inv_l;
              const float hi = __uint_as_float(o[e * 8 + 2 * x + 1]) * inv_l;
              w[x] = OUT_F16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
            }
            const uint32_t chunk = (uint32_t)((c & 1) * 4 + e);
            const uint32_t dst = half_base + ((chunk ^ (uint32_t)(lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[0]),
                         "r"(w[1]), "r"(w[2]), "r"(w[3])
                         : "memory");
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && q0[t] + q * 32 < p.q_len) {   // a slot may reach past the last query row
#pragma unroll
          for (int h = 0; h < 2; ++h)
            tma_store_3d(&tmO, sQ + t * TILE + h * HALF + (uint32_t)(q * 32) * 128, h * 64,
                         q0[t] + q * 32, bh);
          tma_store_commit();
          tma_store_wait_all<0>();
        }
      }
    }
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
static int launch_fmha_pair(const void* q, const void* k, const void* v, void* o, int batch, int heads, int heads_kv,
                            int q_len, int kv_len, const int64_t* qs, const int64_t* ks, const int64_t* vs,
                            const int64_t* os, float qk_scale, int causal, int input_pos, const uint32_t* pos_ptr,
                            cudaStream_t stream) {
  using L = FmhaPairSmem;
  constexpr int D = L::D;
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  const CUtensorMapDataType dt = OUT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmQ, tmK, tmV, tmO;
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
  if ((rc = b200h::encode_tmap_3d(&tmO, dt, 2, o, D, q_len, bh, os[1] * 2, os[0] * 2, 64, 32, 1,
                                  CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  auto kern = fmha_fwd_pair_kernel<OUT_F16>;
  static bool attr_done[64] = {};
  if (!attr_done[di->ordinal]) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    attr_done[di->ordinal] = true;
  }
  FmhaParams p;
  p.q_len = q_len;
  p.kv_len = kv_len;
  p.num_q_pairs = (q_len + 4 * FA_BM - 1) / (4 * FA_BM);   // 512-row quads per (batch, head)
  p.bh_total = (int)bh;
  p.heads = heads;
  p.heads_kv = heads_kv;
  p.group = heads / heads_kv;
  p.causal = causal;
  p.input_pos = input_pos;
  p.pos_ptr = pos_ptr;
  p.head_group = 8;
  p.scale_log2 = qk_scale * 1.4426950408889634f;
  const long long ctas = 2ll * p.num_q_pairs * p.bh_total;
  if (ctas > 0x7fffffffLL) return b200h::set_error(B200_ERR_INVALID, "fmha: grid too large");
  kern<<<(unsigned)ctas, FA_THREADS, L::TOTAL, stream>>>(tmQ, tmK, tmV, tmO, p, di->status);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

}  // namespace b200

// dtype: 0 = bf16, 1 = f16; head_dim 128 only.  Same argument meaning as b200_fmha_fwd_dispatch.
int b200_fmha_fwd_pair_dispatch(int dtype, const void* q, const void* k, const void* v, void* o, int batch, int heads,
                                int heads_kv, int q_len, int kv_len, const int64_t* qs, const int64_t* ks,
                                const int64_t* vs, const int64_t* os, float qk_scale, int causal, int input_pos,
                                const uint32_t* pos_ptr, cudaStream_t stream) {
  using namespace b200;
  return dtype ? launch_fmha_pair<true>(q, k, v, o, batch, heads, heads_kv, q_len, kv_len, qs, ks, vs, os, qk_scale,
                                        causal, input_pos, pos_ptr, stream)
               : launch_fmha_pair<false>(q, k, v, o, batch, heads, heads_kv, q_len, kv_len, qs, ks, vs, os, qk_scale,
                                         causal, input_pos, pos_ptr, stream);
}


#ifdef B200TILE_TRACE
int b200_trace_read_fmha_pair(long long* out) {
  return cudaMemcpyFromSymbol(out, b200::g_trace_fmha_pair, 20 * sizeof(long long)) != cudaSuccess;
}
#endif
