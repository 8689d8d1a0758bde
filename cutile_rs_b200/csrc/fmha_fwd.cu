// Fused multi-head attention forward for sm_100a:  O = softmax(scale * Q K^T + mask) V.
//
// Replaces the machine code the reference obtains by JIT-compiling its FMHA DSL bodies
// (cutile-kernels/src/attention.rs:232-392 `fmha_prefill_causal`; cutile-benchmarks/benches/
// fmha.rs:20-146 and fmha_causal.rs:20-136; cutile-examples/examples/flash_attention*.rs).
// Numerics follow the f32-statistics kernel: log2-domain online softmax (`qk*scale*log2e - m`,
// exp2; attention.rs:286-294,356-366), running max `m`, running sum `l` and the output
// accumulator in fp32, probabilities rounded to 16 bit before P.V (attention.rs:378-380), final
// division by `l` (attention.rs:385-390), causal rule "key position <= query position +
// input_pos" including the diagonal (attention.rs:348), key tiles past the causal frontier skipped
// (attention.rs:303-311).
//
// One CTA owns TWO 128-row query tiles of one (batch, head) problem and walks the key/value tiles
// once for both, so that the tensor core always has the other tile's MMAs to run while one tile is
// in its softmax:
//   warp 0        TMA loads: both Q tiles once, then K and V tiles through two 2-deep rings
//   warp 1        MMA issuer: S_t = Q_t K^T (operands in shared memory) and O_t += P_t V with the
//                 P operand read straight from Tensor Memory -- P never touches shared or global
//   warps 4..7    softmax of tile 0;  warps 8..11  softmax of tile 1 (one query row per thread):
//                 tcgen05.ld S -> max -> exp2 -> sum -> 16-bit P -> tcgen05.st over S's columns
// The O accumulators stay in TMEM across key tiles.  They are rescaled only when a row's maximum
// grew by more than 2^8 since the last rescale (the stale maximum keeps P <= 256, exact after the
// final division); the rescale is done by the row's own softmax thread.
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [384,384+D).
#include <math_constants.h>

#include "host_common.h"
#include "fmha_common.cuh"
#include "sm100_ptx.cuh"
#include "trace.cuh"

namespace b200 {

#ifdef B200TILE_TRACE
// One CTA: MMA thread [0] K/V waits, [1] P waits, [2] P.V issue, [3] Q.K issue, [4] S commits,
// [5] stage-release commits, [6] key tiles, [7] total cycles; [8] the same span in ns; softmax lane 0 of tile 0 from [10]:
// S wait, TMEM load, max and rescale, exp2 loop, store wait, hand-off, key tiles, total.
__device__ long long g_trace_fmha[20];
#endif

template <int D>
struct FmhaSmem {
  static constexpr int HALVES = D / 64;                // 128-byte swizzle rows per head vector
  static constexpr int HALF_BYTES = 128 * 128;         // 128 rows x 128 bytes
  static constexpr int TILE_BYTES = HALVES * HALF_BYTES;
  static constexpr int KV_STAGES = (D == 128) ? 2 : 4;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + 2 * TILE_BYTES;
  static constexpr int OFF_V = OFF_K + KV_STAGES * TILE_BYTES;
  static constexpr int OFF_BAR = OFF_V + KV_STAGES * TILE_BYTES;
  // barriers: q_full[2], k_full[S], k_empty[S], v_full[S], v_empty[S], s_full[2], p_full[2], o_done[2]
  static constexpr int NUM_BARS = 2 + 4 * KV_STAGES + 6;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
  static constexpr int TOTAL = OFF_MISC + 16 + 1024;
};

template <int D, bool OUT_F16>
__global__ void __launch_bounds__(FA_THREADS, 1)
fmha_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                const FmhaParams p, uint32_t* status) {
  using L = FmhaSmem<D>;
  constexpr int STAGES = L::KV_STAGES;
  constexpr int HALVES = L::HALVES;
  constexpr uint32_t HALF = L::HALF_BYTES;
  constexpr uint32_t TILE = L::TILE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));

  const uint32_t sQ = base + L::OFF_Q;
  const uint32_t sK = base + L::OFF_K;
  const uint32_t sV = base + L::OFF_V;
  const uint32_t bar_q_full = base + L::OFF_BAR;
  const uint32_t bar_k_full = bar_q_full + 2 * 8;
  const uint32_t bar_k_empty = bar_k_full + STAGES * 8;
  const uint32_t bar_v_full = bar_k_empty + STAGES * 8;
  const uint32_t bar_v_empty = bar_v_full + STAGES * 8;
  const uint32_t bar_s_full = bar_v_empty + STAGES * 8;
  const uint32_t bar_p_full = bar_s_full + 2 * 8;
  const uint32_t bar_o_done = bar_p_full + 2 * 8;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(gen_base + L::OFF_MISC);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  WaitCtx wctx{misc + 1, status};

  // ---- which work item is this CTA's: head-group swizzle, longest causal rows first ----
  int qp, bh;
  {
    const int idx = blockIdx.x;
    const int per_chunk = p.num_q_pairs * p.head_group;
    const int chunk = idx / per_chunk;
    const int r = idx - chunk * per_chunk;
    const int left = p.bh_total - chunk * p.head_group;
    const int gsz = left < p.head_group ? left : p.head_group;
    qp = r / gsz;
    bh = chunk * p.head_group + (r - qp * gsz);
    if (p.causal) qp = p.num_q_pairs - 1 - qp;
  }
  // decode-style callers keep the position of the first query in device memory
  // (cutile-kernels/src/attention.rs:621-625: `position_start: &Tensor<u32, {[1]}>`)
  const int input_pos = p.pos_ptr ? (int)__ldg(p.pos_ptr) : p.input_pos;
  const int kv_bh = (bh / p.heads) * p.heads_kv + (bh % p.heads) / p.group;
  const int n_total = (p.kv_len + FA_BN - 1) / FA_BN;
  int q0[2], n_kv[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    q0[t] = (qp * 2 + t) * FA_BM;
    if (q0[t] >= p.q_len) {
      n_kv[t] = 0;
    } else if (p.causal) {
      const int last = (q0[t] + FA_BM - 1 + input_pos) / FA_BN + 1;
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
      mbar_init(bar_p_full + i * 8, 4);
      mbar_init(bar_o_done + i * 8, 1);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_k_full + s * 8, 1);
      mbar_init(bar_k_empty + s * 8, 1);
      mbar_init(bar_v_full + s * 8, 1);
      mbar_init(bar_v_empty + s * 8, 1);
    }
    misc[1] = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmO);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(misc)), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = misc[0];
  auto S_COL = [](int t) { return (uint32_t)(t * 128); };
  auto O_COL = [](int t) { return (uint32_t)(256 + t * 128); };

  if (warp < 4) reg_dealloc<FA_OTHER_REGS>();
  if (warp == 0) {
    // ------------------------------- TMA loader -------------------------------
    if (lane == 0) {
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (n_kv[t] == 0) continue;
        mbar_expect_tx(bar_q_full + t * 8, TILE);
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
          tma_load_3d(sQ + t * TILE + h * HALF, &tmQ, bar_q_full + t * 8, h * 64, q0[t], bh);
      }
      uint32_t stage = 0, phase = 0;
      for (int j = 0; j < n_max; ++j) {
        if (!mbar_wait(wctx, bar_k_empty + stage * 8, phase ^ 1, 10)) break;
        mbar_expect_tx(bar_k_full + stage * 8, TILE);
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
          tma_load_3d(sK + stage * TILE + h * HALF, &tmK, bar_k_full + stage * 8, h * 64,
                      j * FA_BN, kv_bh);
        if (!mbar_wait(wctx, bar_v_empty + stage * 8, phase ^ 1, 11)) break;
        mbar_expect_tx(bar_v_full + stage * 8, TILE);
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
          tma_load_3d(sV + stage * TILE + h * HALF, &tmV, bar_v_full + stage * 8, h * 64,
                      j * FA_BN, kv_bh);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer --------------------------------
    // The whole warp runs the control flow and the descriptor arithmetic (which then stays in uniform registers);
    // one elected lane issues the tcgen05 instructions.  Under `if (lane == 0)` every MMA and commit costs the
    // issuing thread ~80 cycles, more than the 64 a 128 x 128 x 16 MMA occupies the tensor pipe.
    if (n_max > 0) {
      const bool me = elect_one() != 0;
      constexpr uint32_t fmt = OUT_F16 ? FMT_F16 : FMT_BF16;
      constexpr uint32_t idesc_qk = make_idesc(fmt, fmt, 0, 0, FA_BM, FA_BN);
      constexpr uint32_t idesc_pv = make_idesc(fmt, fmt, 0, 1, FA_BM, D);
      auto issue_qk = [&](int t, uint32_t k_addr) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * HALF + (kk % 4) * 32;
          const uint64_t a = make_smem_desc(sQ + t * TILE + off, 16, 1024, SWZ_128B);
          const uint64_t b = make_smem_desc(k_addr + off, 16, 1024, SWZ_128B);
          if (me) umma_f16_ss(tmem_base + S_COL(t), a, b, idesc_qk, kk != 0);
        }
      };
      auto issue_pv = [&](int t, uint32_t v_addr, bool acc) {
#pragma unroll
        for (int kk = 0; kk < FA_BN / 16; ++kk) {
          // V is the N-major B operand: 16 key rows per step = two 8-row groups of 1024 bytes;
          // the second 64-wide half of the head vector lies HALF bytes further (leading offset).
          const uint64_t b = make_smem_desc(v_addr + kk * 2048, HALF, 1024, SWZ_128B);
          if (me) umma_f16_ts(tmem_base + O_COL(t), tmem_base + S_COL(t) + kk * 8, b, idesc_pv, acc || kk != 0);
        }
      };
      bool ok = true;
      B200_TR_DECL(7);
      // prologue: S_t(0) = Q_t K(0)^T
      ok = __all_sync(0xffffffffu, mbar_wait(wctx, bar_k_full + 0, 0, 20));
#pragma unroll
      for (int t = 0; t < 2 && ok; ++t) {
        if (n_kv[t] == 0) continue;
        if (!__all_sync(0xffffffffu, mbar_wait(wctx, bar_q_full + t * 8, 0, 21))) { ok = false; break; }
        tc_fence_after_sync();
        issue_qk(t, sK);
        if (me) umma_commit(bar_s_full + t * 8);
      }
      if (ok && me) umma_commit(bar_k_empty + 0);
      for (int j = 0; j < n_max && ok; ++j) {
        const uint32_t vs = j % STAGES, vph = (j / STAGES) & 1;
        const uint32_t ks = (j + 1) % STAGES, kph = ((j + 1) / STAGES) & 1;
        const bool have_next = j + 1 < n_max;
        B200_TR_COUNT(6);
        B200_TR_BEGIN();
        if (!__all_sync(0xffffffffu, mbar_wait(wctx, bar_v_full + vs * 8, vph, 22))) { ok = false; break; }
        if (have_next && !__all_sync(0xffffffffu, mbar_wait(wctx, bar_k_full + ks * 8, kph, 23))) { ok = false; break; }
        tc_fence_after_sync();
        B200_TR_END(0);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j < n_kv[t]) {
            B200_TR_BEGIN();
            if (!__all_sync(0xffffffffu, mbar_wait(wctx, bar_p_full + t * 8, j & 1, 24))) { ok = false; break; }
            tc_fence_after_sync();
            B200_TR_END(1);
            B200_TR_BEGIN();
            issue_pv(t, sV + vs * TILE, j > 0);
            B200_TR_END(2);
            if (j == n_kv[t] - 1 && me) umma_commit(bar_o_done + t * 8);
          }
          if (j + 1 < n_kv[t]) {
            B200_TR_BEGIN();
            issue_qk(t, sK + ks * TILE);
            B200_TR_END(3);
            B200_TR_BEGIN();
            if (me) umma_commit(bar_s_full + t * 8);
            B200_TR_END(4);
          }
        }
        if (!ok) break;
        B200_TR_BEGIN();
        if (me) umma_commit(bar_v_empty + vs * 8);
        if (have_next && me) umma_commit(bar_k_empty + ks * 8);
        B200_TR_END(5);
      }
      B200_TR_FLUSH(g_trace_fmha, 7, blockIdx.x == 7 && lane == 0);
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
      if (lane == 0) mbar_arrive(bar_p_full + t * 8);
      B200_TR_END(5);
    }
    B200_TR_FLUSH(g_trace_fmha + 10, 7, blockIdx.x == 7 && warp == 4 && lane == 0);
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
        if (lane == 0) {
#pragma unroll
          for (int h = 0; h < HALVES; ++h)
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
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int D, bool OUT_F16>
static int launch_fmha(const void* q, const void* k, const void* v, void* o, int batch, int heads,
                       int heads_kv, int q_len, int kv_len, const int64_t* qs, const int64_t* ks,
                       const int64_t* vs, const int64_t* os, float qk_scale, int causal,
                       int input_pos, const uint32_t* pos_ptr, cudaStream_t stream) {
  using L = FmhaSmem<D>;
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  const CUtensorMapDataType dt =
      OUT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  // strides arrays: {stride of (batch*head) index, stride of sequence index}, in elements
  CUtensorMap tmQ, tmK, tmV, tmO;
  int rc;
  const uint64_t bh = (uint64_t)batch * heads, bhkv = (uint64_t)batch * heads_kv;
  if ((rc = b200h::encode_tmap_3d(&tmQ, dt, 2, q, D, q_len, bh, qs[1] * 2, qs[0] * 2, 64, FA_BM, 1,
                                  CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  if ((rc = b200h::encode_tmap_3d(&tmK, dt, 2, k, D, kv_len, bhkv, ks[1] * 2, ks[0] * 2, 64, FA_BN,
                                  1, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  if ((rc = b200h::encode_tmap_3d(&tmV, dt, 2, v, D, kv_len, bhkv, vs[1] * 2, vs[0] * 2, 64, FA_BN,
                                  1, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  if ((rc = b200h::encode_tmap_3d(&tmO, dt, 2, o, D, q_len, bh, os[1] * 2, os[0] * 2, 64, 32, 1,
                                  CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  auto kern = fmha_fwd_kernel<D, OUT_F16>;
  static b200h::DeviceOnce attr_done;
  if (!attr_done.test(di->ordinal)) {
    B200_CUDA_CHECK(
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    attr_done.set(di->ordinal);
  }
  FmhaParams p;
  p.q_len = q_len;
  p.kv_len = kv_len;
  p.num_q_pairs = (q_len + 2 * FA_BM - 1) / (2 * FA_BM);
  p.bh_total = (int)bh;
  p.heads = heads;
  p.heads_kv = heads_kv;
  p.group = heads / heads_kv;
  p.causal = causal;
  p.input_pos = input_pos;
  p.pos_ptr = pos_ptr;
  p.head_group = 8;
  p.scale_log2 = qk_scale * 1.4426950408889634f;
  const long long ctas = (long long)p.num_q_pairs * p.bh_total;
  if (ctas > 0x7fffffffLL) return b200h::set_error(B200_ERR_INVALID, "fmha: grid too large");
  kern<<<(unsigned)ctas, FA_THREADS, L::TOTAL, stream>>>(tmQ, tmK, tmV, tmO, p, di->status);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

}  // namespace b200

// dtype: 0 = bf16, 1 = f16.  Strides are {per (batch*head) index, per sequence position} in
// elements; the head vector is contiguous.
int b200_fmha_fwd_dispatch(int dtype, int head_dim, const void* q, const void* k, const void* v,
                           void* o, int batch, int heads, int heads_kv, int q_len, int kv_len,
                           const int64_t* qs, const int64_t* ks, const int64_t* vs,
                           const int64_t* os, float qk_scale, int causal, int input_pos,
                           const uint32_t* pos_ptr, cudaStream_t stream) {
  using namespace b200;
#define B200_FA_CASE(D_, F16_)                                                                 \
  return launch_fmha<D_, F16_>(q, k, v, o, batch, heads, heads_kv, q_len, kv_len, qs, ks, vs, \
                               os, qk_scale, causal, input_pos, pos_ptr, stream)
  if (head_dim == 128 && dtype == 0) B200_FA_CASE(128, false);
  if (head_dim == 128 && dtype == 1) B200_FA_CASE(128, true);
  if (head_dim == 64 && dtype == 0) B200_FA_CASE(64, false);
  if (head_dim == 64 && dtype == 1) B200_FA_CASE(64, true);
#undef B200_FA_CASE
  return b200h::set_error(B200_ERR_UNSUPPORTED,
                          "fmha: no kernel for head_dim %d (64 and 128 are provided)", head_dim);
}

#ifdef B200TILE_TRACE
int b200_trace_read_fmha(long long* out) {
  return cudaMemcpyFromSymbol(out, b200::g_trace_fmha, 20 * sizeof(long long)) != cudaSuccess;
}
#endif
