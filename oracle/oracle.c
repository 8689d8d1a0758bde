/* TEST INFRASTRUCTURE -- not part of the product.
 *
 * CPU restatement, in plain C, of the host-side reference computations the reference project
 * uses to check its own dense-contraction kernels, plus the element codecs and block quantisers
 * of the low-precision GEMM configurations.  Only tests, the smoke check and the CPU-baseline /
 * reference arms of the benchmark may call into this file; the product path never does.
 *
 * Parity status: pinned against the reference's own known-answer cases (ones x ones GEMM == K,
 * the patterned 64x64x32 GEMM, FP4/FP8 bit constants, nibble order) -- see tests/.  Random-data
 * bf16/fp8/NVFP4 GEMM and 16-bit attention have no golden vectors in the reference
 * ("parity unpinned" for those; the stated tolerances against this fp32 restatement apply).
 *
 * Floating-point contraction must be OFF when compiling this file (-ffp-contract=off): the Rust
 * originals round every product and every sum separately.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

#define ORACLE_API __attribute__((visibility("default")))

/* Minimal static-schedule parallel-for over [0, count) on POSIX threads. */
typedef void (*oracle_range_fn)(void* ctx, int64_t begin, int64_t end);
typedef struct { oracle_range_fn fn; void* ctx; int64_t begin, end; } oracle_task;
static void* oracle_task_main(void* p) {
  oracle_task* t = (oracle_task*)p;
  t->fn(t->ctx, t->begin, t->end);
  return NULL;
}
ORACLE_API int oracle_max_threads(void) {
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n < 1 ? 1 : (n > 256 ? 256 : (int)n);
}
static int oracle_parallel_for(oracle_range_fn fn, void* ctx, int64_t count, int threads) {
  if (threads <= 0) threads = oracle_max_threads();
  if (threads > 256) threads = 256;
  if ((int64_t)threads > count) threads = count > 0 ? (int)count : 1;
  if (threads <= 1) { fn(ctx, 0, count); return 1; }
  pthread_t tid[256];
  oracle_task task[256];
  int started = 0;
  for (int t = 0; t < threads; ++t) {
    task[t].fn = fn; task[t].ctx = ctx;
    task[t].begin = count * t / threads; task[t].end = count * (t + 1) / threads;
    if (t == threads - 1 || pthread_create(&tid[t], NULL, oracle_task_main, &task[t]) != 0) {
      /* last chunk (or a failed create) runs on the calling thread */
      task[t].end = count;
      fn(ctx, task[t].begin, task[t].end);
      break;
    }
    ++started;
  }
  for (int t = 0; t < started; ++t) pthread_join(tid[t], NULL);
  return started + 1;
}

/* ------------------------------------------------------------------------------------------
 * GEMM: cutile-examples/examples/persistent_gemm.rs:140-152 (`cpu_gemm`)
 *   z[row*n+col] = sum over inner (ascending) of x[row*k+inner] * y[inner*n+col], f32.
 * row0/row1 restrict the computation to a slab of output rows (the full function is the slab
 * [0, m)); rows outside the slab are left untouched.
 * ------------------------------------------------------------------------------------------ */
ORACLE_API void oracle_cpu_gemm_rows(const float* x, const float* y, float* z, int64_t m,
                                     int64_t n, int64_t k, int64_t row0, int64_t row1) {
  (void)m;
  for (int64_t row = row0; row < row1; ++row) {
    for (int64_t col = 0; col < n; ++col) {
      float acc = 0.0f;
      for (int64_t inner = 0; inner < k; ++inner) acc += x[row * k + inner] * y[inner * n + col];
      z[row * n + col] = acc;
    }
  }
}

ORACLE_API void oracle_cpu_gemm(const float* x, const float* y, float* z, int64_t m, int64_t n,
                                int64_t k) {
  oracle_cpu_gemm_rows(x, y, z, m, n, k, 0, m);
}

/* Same arithmetic, rows spread over `threads` host threads (each output element is still one
 * sequential ascending-k sum, so results are bit-identical to the single-thread form). */
typedef struct { const float *x, *y; float* z; int64_t m, n, k, row0; float alpha; } gemm_ctx;
static void gemm_range(void* p, int64_t b, int64_t e) {
  gemm_ctx* c = (gemm_ctx*)p;
  oracle_cpu_gemm_rows(c->x, c->y, c->z, c->m, c->n, c->k, c->row0 + b, c->row0 + e);
}
ORACLE_API int oracle_cpu_gemm_rows_mt(const float* x, const float* y, float* z, int64_t m,
                                       int64_t n, int64_t k, int64_t row0, int64_t row1,
                                       int threads) {
  gemm_ctx c = {x, y, z, m, n, k, row0, 1.0f};
  return oracle_parallel_for(gemm_range, &c, row1 - row0, threads);
}

/* "NT" form used by the block-scaled linear kernels (cutile-examples/examples/nvfp4.rs:20-33:
 * z[M,N] = alpha * x[M,K] @ y[N,K]^T): same ascending-k f32 sum, y indexed [col*k+inner]. */
ORACLE_API void oracle_cpu_gemm_nt_rows(const float* x, const float* y, float* z, int64_t m,
                                        int64_t n, int64_t k, float alpha, int64_t row0,
                                        int64_t row1) {
  (void)m;
  for (int64_t row = row0; row < row1; ++row) {
    for (int64_t col = 0; col < n; ++col) {
      float acc = 0.0f;
      for (int64_t inner = 0; inner < k; ++inner) acc += x[row * k + inner] * y[col * k + inner];
      z[row * n + col] = acc * alpha;
    }
  }
}

static void gemm_nt_range(void* p, int64_t b, int64_t e) {
  gemm_ctx* c = (gemm_ctx*)p;
  oracle_cpu_gemm_nt_rows(c->x, c->y, c->z, c->m, c->n, c->k, c->alpha, c->row0 + b, c->row0 + e);
}
ORACLE_API int oracle_cpu_gemm_nt_rows_mt(const float* x, const float* y, float* z, int64_t m,
                                          int64_t n, int64_t k, float alpha, int64_t row0,
                                          int64_t row1, int threads) {
  gemm_ctx c = {x, y, z, m, n, k, row0, alpha};
  return oracle_parallel_for(gemm_nt_range, &c, row1 - row0, threads);
}

/* ------------------------------------------------------------------------------------------
 * Attention: cutile-examples/examples/flash_attention_causal.rs:140-210 (`idx4`, `fmha_ref_cpu`)
 *   layout (b, h, m, d); kv head = h / query_group_size; causal masks j > i + input_pos;
 *   max-subtracted exp; probabilities normalised (score / denom) inside the P.V sum; all f32.
 * (bh0, bh1) and (i0, i1) restrict the work to a slab of (batch*head) problems and query rows.
 * ------------------------------------------------------------------------------------------ */
static inline int64_t idx4(int64_t a, int64_t b, int64_t c, int64_t d, int64_t hsz, int64_t m,
                           int64_t dsz) {
  return (((a * hsz + b) * m + c) * dsz) + d;
}

static void fmha_one_row(const float* q, const float* k, const float* v, float* out, float* scores,
                         int64_t b, int64_t h, int64_t i, int64_t hsz, int64_t hkv, int64_t m,
                         int64_t dsz, float qk_scale, int64_t input_pos, int64_t query_group_size,
                         int causal) {
  const int64_t kv_h = h / query_group_size;
  float max_logit = -INFINITY;
  for (int64_t j = 0; j < m; ++j) {
    if (causal && j > i + input_pos) {
      scores[j] = -INFINITY;
      continue;
    }
    float dot = 0.0f;
    for (int64_t dd = 0; dd < dsz; ++dd)
      dot += q[idx4(b, h, i, dd, hsz, m, dsz)] * k[idx4(b, kv_h, j, dd, hkv, m, dsz)];
    scores[j] = dot * qk_scale;
    max_logit = fmaxf(max_logit, scores[j]);
  }
  float denom = 0.0f;
  for (int64_t j = 0; j < m; ++j) {
    scores[j] = expf(scores[j] - max_logit);
    denom += scores[j];
  }
  for (int64_t dd = 0; dd < dsz; ++dd) {
    float val = 0.0f;
    for (int64_t j = 0; j < m; ++j) {
      const float p = scores[j] / denom;
      val += p * v[idx4(b, kv_h, j, dd, hkv, m, dsz)];
    }
    out[idx4(b, h, i, dd, hsz, m, dsz)] = val;
  }
}

typedef struct {
  const float *q, *k, *v; float* out;
  int64_t hsz, hkv, m, dsz, input_pos, group, bh0, i0, rows; float qk_scale; int causal;
} fmha_ctx;
static void fmha_range(void* p, int64_t b, int64_t e) {
  fmha_ctx* c = (fmha_ctx*)p;
  float* scores = (float*)malloc(sizeof(float) * (size_t)c->m);
  if (!scores) return;
  for (int64_t w = b; w < e; ++w) {
    const int64_t bh = c->bh0 + w / c->rows, i = c->i0 + w % c->rows;
    fmha_one_row(c->q, c->k, c->v, c->out, scores, bh / c->hsz, bh % c->hsz, i, c->hsz, c->hkv,
                 c->m, c->dsz, c->qk_scale, c->input_pos, c->group, c->causal);
  }
  free(scores);
}
ORACLE_API int oracle_fmha_ref_cpu_slab(const float* q, const float* k, const float* v, float* out,
                                        int64_t bsz, int64_t hsz, int64_t hkv, int64_t m,
                                        int64_t dsz, float qk_scale, int64_t input_pos,
                                        int64_t query_group_size, int causal, int64_t bh0,
                                        int64_t bh1, int64_t i0, int64_t i1, int threads) {
  (void)bsz;
  fmha_ctx c = {q, k, v, out, hsz, hkv, m, dsz, input_pos, query_group_size, bh0, i0, i1 - i0,
                qk_scale, causal};
  return oracle_parallel_for(fmha_range, &c, (bh1 - bh0) * (i1 - i0), threads);
}

ORACLE_API void oracle_fmha_ref_cpu(const float* q, const float* k, const float* v, float* out,
                                    int64_t bsz, int64_t hsz, int64_t hkv, int64_t m, int64_t dsz,
                                    float qk_scale, int64_t input_pos, int64_t query_group_size,
                                    int causal) {
  oracle_fmha_ref_cpu_slab(q, k, v, out, bsz, hsz, hkv, m, dsz, qk_scale, input_pos,
                           query_group_size, causal, 0, bsz * hsz, 0, m, 1);
}

/* ------------------------------------------------------------------------------------------
 * Element codecs.  Bit conventions: cuda-core/src/dtype.rs:20-110 (types), :210-229 (1.0 bit
 * patterns: f8e4m3fn 0x38, f8e5m2 0x3C, f8e8m0fnu 0x7F, FP4 1.0 = nibble 0x2).
 * ------------------------------------------------------------------------------------------ */
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* bf16: round to nearest even; NaN stays a quiet NaN. */
ORACLE_API uint16_t oracle_f32_to_bf16(float f) {
  uint32_t u = f32_bits(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
ORACLE_API float oracle_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

ORACLE_API void oracle_f32_to_bf16_array(const float* src, uint16_t* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = oracle_f32_to_bf16(src[i]);
}
ORACLE_API void oracle_bf16_to_f32_array(const uint16_t* src, float* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = oracle_bf16_to_f32(src[i]);
}

/* f8e4m3fn: 1 sign, 4 exponent (bias 7), 3 mantissa; no infinity; 0x7F/0xFF are NaN;
 * largest finite 448 (0x7E). */
ORACLE_API float oracle_e4m3_to_f32(uint8_t b) {
  const int s = b >> 7, e = (b >> 3) & 0xF, mnt = b & 7;
  float v;
  if (e == 0xF && mnt == 7) return NAN;
  if (e == 0) v = ldexpf((float)mnt, -9);            /* subnormal: m/8 * 2^-6 */
  else v = ldexpf(1.0f + (float)mnt / 8.0f, e - 7);
  return s ? -v : v;
}
/* Round-to-nearest-even, saturating to +-448 (the "satfinite" conversion quantisers use). */
ORACLE_API uint8_t oracle_f32_to_e4m3(float f) {
  if (isnan(f)) return 0x7F;
  const uint8_t s = signbit(f) ? 0x80 : 0;
  float a = fabsf(f);
  if (a >= 448.0f) return s | 0x7E;
  if (a < ldexpf(1.0f, -10)) return s;               /* below half the smallest subnormal */
  int e;
  (void)frexpf(a, &e);                                /* a = m * 2^e, m in [0.5,1) */
  int exp = e - 1;                                    /* a = 1.x * 2^exp */
  if (exp < -6) exp = -6;                             /* subnormal range shares exponent -6 */
  const float q = ldexpf(a, 3 - exp);                 /* in units of the mantissa lsb */
  float r = nearbyintf(q);                            /* default rounding mode: nearest even */
  int biased = exp + 7;
  int mant;
  if (exp == -6 && r < 8.0f) { biased = 0; mant = (int)r; }
  else {
    if (r >= 16.0f) { r = 8.0f; biased += 1; }
    mant = (int)r - 8;
  }
  if (biased > 15 || (biased == 15 && mant == 7)) return s | 0x7E;
  return s | (uint8_t)(biased << 3) | (uint8_t)mant;
}

/* f8e5m2 decode only (constant check). */
ORACLE_API float oracle_e5m2_to_f32(uint8_t b) {
  const int s = b >> 7, e = (b >> 2) & 0x1F, mnt = b & 3;
  float v;
  if (e == 0x1F) v = mnt ? NAN : INFINITY;
  else if (e == 0) v = ldexpf((float)mnt, -16);
  else v = ldexpf(1.0f + (float)mnt / 4.0f, e - 15);
  return s ? -v : v;
}

/* f8e8m0fnu: value 2^(b-127); 0xFF is NaN. */
ORACLE_API float oracle_e8m0_to_f32(uint8_t b) { return b == 0xFF ? NAN : ldexpf(1.0f, (int)b - 127); }

/* f4e2m1fn: 1 sign, 2 exponent (bias 1), 1 mantissa: 0, .5, 1, 1.5, 2, 3, 4, 6. */
static const float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
ORACLE_API float oracle_e2m1_to_f32(uint8_t nib) {
  const float v = kE2M1[nib & 7];
  return (nib & 8) ? -v : v;
}
/* Round-to-nearest-even on the e2m1 grid, saturating to +-6. */
ORACLE_API uint8_t oracle_f32_to_e2m1(float f) {
  const uint8_t s = signbit(f) ? 8 : 0;
  const float a = fabsf(f);
  if (isnan(f)) return 7;
  uint8_t code;
  if (a <= 0.25f) code = 0;            /* tie at .25 -> 0 (even mantissa) */
  else if (a < 0.75f) code = 1;
  else if (a <= 1.25f) code = 2;       /* ties .75 -> 1.0, 1.25 -> 1.0 */
  else if (a < 1.75f) code = 3;
  else if (a <= 2.5f) code = 4;        /* ties 1.75 -> 2, 2.5 -> 2 */
  else if (a < 3.5f) code = 5;
  else if (a <= 5.0f) code = 6;        /* ties 3.5 -> 4, 5 -> 4 */
  else code = 7;
  return s | code;
}
/* Packed pair: low nibble = first logical value (cuda-core/src/dtype.rs:60-110, :403-417). */
ORACLE_API uint8_t oracle_pack_e2m1x2(uint8_t low, uint8_t high) {
  return (uint8_t)((low & 0x0F) | ((high & 0x0F) << 4));
}

/* ------------------------------------------------------------------------------------------
 * Block quantisers for the low-precision GEMM configurations.
 * ------------------------------------------------------------------------------------------ */

/* fp8 e4m3 with one fp32 scale per (block_r x block_c) block: scale = blockmax/448 (1 when the
 * block is all zero), q = e4m3_rne_sat(x / scale).  Activations use 1x128, weights 128x128. */
ORACLE_API void oracle_quant_fp8_block(const float* x, int64_t rows, int64_t cols, int64_t block_r,
                                       int64_t block_c, uint8_t* q, float* scales) {
  const int64_t nbr = (rows + block_r - 1) / block_r, nbc = (cols + block_c - 1) / block_c;
  for (int64_t br = 0; br < nbr; ++br)
    for (int64_t bc = 0; bc < nbc; ++bc) {
      const int64_t r1 = (br + 1) * block_r < rows ? (br + 1) * block_r : rows;
      const int64_t c1 = (bc + 1) * block_c < cols ? (bc + 1) * block_c : cols;
      float amax = 0.0f;
      for (int64_t r = br * block_r; r < r1; ++r)
        for (int64_t c = bc * block_c; c < c1; ++c) amax = fmaxf(amax, fabsf(x[r * cols + c]));
      const float scale = amax > 0.0f ? amax / 448.0f : 1.0f;
      scales[br * nbc + bc] = scale;
      for (int64_t r = br * block_r; r < r1; ++r)
        for (int64_t c = bc * block_c; c < c1; ++c)
          q[r * cols + c] = oracle_f32_to_e4m3(x[r * cols + c] / scale);
    }
}

ORACLE_API void oracle_dequant_fp8_block(const uint8_t* q, const float* scales, int64_t rows,
                                         int64_t cols, int64_t block_r, int64_t block_c,
                                         float* out) {
  const int64_t nbc = (cols + block_c - 1) / block_c;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c)
      out[r * cols + c] = oracle_e4m3_to_f32(q[r * cols + c]) * scales[(r / block_r) * nbc + c / block_c];
}

/* NVFP4: global fp32 scale g = amax/(6*448); per 16 contiguous K elements an e4m3 scale
 * s = e4m3(blockmax/(6*g)); q = e2m1_rne(x/(s*g)); two values per byte, low nibble first;
 * scales row-major [rows, cols/16] (cutile-examples/examples/nvfp4.rs:24-33).  Returns g. */
ORACLE_API float oracle_quant_nvfp4(const float* x, int64_t rows, int64_t cols, uint8_t* packed,
                                    uint8_t* scales) {
  float amax = 0.0f;
  for (int64_t i = 0; i < rows * cols; ++i) amax = fmaxf(amax, fabsf(x[i]));
  const float g = amax > 0.0f ? amax / (6.0f * 448.0f) : 1.0f;
  const int64_t nb = cols / 16;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t b = 0; b < nb; ++b) {
      const float* xb = x + r * cols + b * 16;
      float bmax = 0.0f;
      for (int i = 0; i < 16; ++i) bmax = fmaxf(bmax, fabsf(xb[i]));
      const uint8_t sb = oracle_f32_to_e4m3(bmax / (6.0f * g));
      scales[r * nb + b] = sb;
      const float s = oracle_e4m3_to_f32(sb) * g;
      for (int i = 0; i < 16; i += 2) {
        const uint8_t lo = s > 0.0f ? oracle_f32_to_e2m1(xb[i] / s) : 0;
        const uint8_t hi = s > 0.0f ? oracle_f32_to_e2m1(xb[i + 1] / s) : 0;
        packed[(r * cols + b * 16 + i) / 2] = oracle_pack_e2m1x2(lo, hi);
      }
    }
  return g;
}

/* Dequantises WITHOUT the global scale (that one is folded into `alpha`, as the tutorial does:
 * cutile-book/tutorials/11-nvfp4-inference.md:147-148): out = e2m1 * e4m3_scale. */
ORACLE_API void oracle_dequant_nvfp4(const uint8_t* packed, const uint8_t* scales, int64_t rows,
                                     int64_t cols, float* out) {
  const int64_t nb = cols / 16;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c) {
      const uint8_t byte = packed[(r * cols + c) / 2];
      const uint8_t nib = (c & 1) ? (byte >> 4) : (byte & 0x0F);
      out[r * cols + c] = oracle_e2m1_to_f32(nib) * oracle_e4m3_to_f32(scales[r * nb + c / 16]);
    }
}

/* MXFP8 (cutile-examples/examples/mxfp8.rs:25-33): e4m3 values with one f8e8m0fnu scale per 32
 * contiguous K elements, scales row-major [rows, cols/32].  The scale is the smallest power of two
 * with blockmax/scale <= 448 (exponent byte 127 = 1.0 for an all-zero block); q = e4m3_rne(x/scale). */
ORACLE_API void oracle_quant_mxfp8(const float* x, int64_t rows, int64_t cols, uint8_t* q, uint8_t* scales) {
  const int64_t nb = cols / 32;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t b = 0; b < nb; ++b) {
      const float* xb = x + r * cols + b * 32;
      float amax = 0.0f;
      for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(xb[i]));
      int e = 0;
      if (amax > 0.0f) {
        int fe;
        const float fm = frexpf(amax / 448.0f, &fe);   /* amax/448 = fm * 2^fe, fm in [0.5, 1) */
        e = (fm == 0.5f) ? fe - 1 : fe;                /* ceil(log2(amax/448)) */
        if (e < -127) e = -127;
        if (e > 127) e = 127;
      }
      scales[r * nb + b] = (uint8_t)(e + 127);
      const float s = ldexpf(1.0f, e);
      for (int i = 0; i < 32; ++i) q[r * cols + b * 32 + i] = oracle_f32_to_e4m3(xb[i] / s);
    }
}

ORACLE_API void oracle_dequant_mxfp8(const uint8_t* q, const uint8_t* scales, int64_t rows, int64_t cols,
                                     float* out) {
  const int64_t nb = cols / 32;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c)
      out[r * cols + c] = oracle_e4m3_to_f32(q[r * cols + c]) * oracle_e8m0_to_f32(scales[r * nb + c / 32]);
}

/* mmaf_scaled semantics (cutile-book/tutorials/11-nvfp4-inference.md:58-82), NT layout:
 *   z[i,j] = alpha * sum_k  x[i,k]*xs[i,k/V] * y[j,k]*ys[j,k/V]
 * computed here from already-dequantised operands via oracle_cpu_gemm_nt_rows. */

/* Persistent-grid formula: cutile-benchmarks/paper/sec5_exp1_safety_overhead/rust/gemm/src/
 * main.rs:796-811 (`persistent_num_programs`). */
ORACLE_API uint32_t oracle_persistent_num_programs(int64_t m, int64_t n, int bm, int bn, int num_sms,
                                                   int num_cta_in_cga, int occupancy) {
  const int64_t tiles_m = (m + bm - 1) / bm, tiles_n = (n + bn - 1) / bn;
  int64_t total = tiles_m * tiles_n;
  if (total < 1) total = 1;
  int cta = num_cta_in_cga > 1 ? num_cta_in_cga : 1;
  int64_t sm_programs = num_sms / cta;
  if (sm_programs < 1) sm_programs = 1;
  int64_t programs = (sm_programs < total ? sm_programs : total) * (occupancy > 1 ? occupancy : 1);
  return (uint32_t)(programs < 1 ? 1 : programs);
}

/* Grouped-M tile order: main.rs:53-66 (`swizzled_bid`). */
ORACLE_API void oracle_swizzled_bid(int tile_id, int num_bid_m, int num_bid_n, int group_size_m,
                                    int* bid_m, int* bid_n) {
  const int num_bid_in_group = group_size_m * num_bid_n;
  const int group_id = tile_id / num_bid_in_group;
  const int first_bid_m = group_id * group_size_m;
  const int remaining_m = num_bid_m - first_bid_m;
  const int actual = remaining_m < group_size_m ? remaining_m : group_size_m;
  *bid_m = first_bid_m + (tile_id % actual);
  *bid_n = (tile_id % num_bid_in_group) / actual;
}

/* ------------------------------------------------------------------------------------------
 * Split-KV GQA decode attention: cutile-kernels/src/attention.rs:727-901 (`fmha_decode_gqa_split`)
 * and :907-1015 (`splitk_reduce_merge`), restated tile by tile.  Inputs are floats that already
 * hold 16-bit-representable values; `is_f16` selects how P and the outputs are rounded.
 *   q [kv_heads, group, D]; k, v [kv_heads, kv_cap, D]; att [kv_heads, splits*group, D];
 *   lse [kv_heads, splits*group]; s_kv = position_start + 1.
 * ------------------------------------------------------------------------------------------ */
static float round16(float x, int is_f16) {
  if (is_f16) return (float)(_Float16)x;
  return oracle_bf16_to_f32(oracle_f32_to_bf16(x));
}

ORACLE_API void oracle_fmha_decode_gqa_split(const float* q, const float* k, const float* v, float* att,
                                             float* lse, int64_t kv_heads, int64_t group, int64_t D,
                                             int64_t kv_cap, int64_t s_kv, int64_t bn, int64_t splits,
                                             float qk_scale, int is_f16) {
  const float scale_log2 = qk_scale / logf(2.0f);               /* :760-764 */
  const int64_t tiles = (s_kv + bn - 1) / bn;                    /* :767 */
  const int64_t tps = (tiles + splits - 1) / splits;             /* :768 */
  float* qk = (float*)malloc(sizeof(float) * (size_t)(bn * group));
  float* l_i = (float*)malloc(sizeof(float) * (size_t)(bn * group));
  float* acc = (float*)malloc(sizeof(float) * (size_t)(D * group));
  float* m_i = (float*)malloc(sizeof(float) * (size_t)group);
  for (int64_t h = 0; h < kv_heads; ++h)
    for (int64_t sp = 0; sp < splits; ++sp) {
      const int64_t start = sp * tps;
      int64_t end = start + tps;
      if (end > tiles) end = tiles;                              /* :769-771 */
      for (int64_t g = 0; g < group; ++g) m_i[g] = -1.0e30f;     /* :786-789 */
      for (int64_t i = 0; i < bn * group; ++i) l_i[i] = 1.0f;    /* :790 */
      for (int64_t i = 0; i < D * group; ++i) acc[i] = 0.0f;     /* :791 */
      for (int64_t j = start; j < end; ++j) {
        for (int64_t n = 0; n < bn; ++n)
          for (int64_t g = 0; g < group; ++g) {
            const int64_t key = j * bn + n;
            float dot = 0.0f;
            if (key < kv_cap)                                    /* out-of-range tile rows load as zero */
              for (int64_t d = 0; d < D; ++d)
                dot += k[(h * kv_cap + key) * D + d] * q[(h * group + g) * D + d];
            if (j == tiles - 1 && key >= s_kv) dot += -1.0e30f;  /* :832-838 */
            qk[n * group + g] = dot * scale_log2;                /* :843 */
          }
        for (int64_t g = 0; g < group; ++g) {
          float mx = -INFINITY;
          for (int64_t n = 0; n < bn; ++n) mx = fmaxf(mx, qk[n * group + g]);
          const float m_ij = fmaxf(m_i[g], mx);                  /* :847 */
          const float alpha = exp2f(m_i[g] - m_ij);              /* :854 */
          for (int64_t n = 0; n < bn; ++n) {
            const float p = exp2f(qk[n * group + g] - m_ij);     /* :848-850 */
            l_i[n * group + g] = l_i[n * group + g] * alpha + p; /* :857 */
            qk[n * group + g] = round16(p, is_f16);              /* :878 */
          }
          for (int64_t d = 0; d < D; ++d) acc[d * group + g] *= alpha;   /* :859 */
          m_i[g] = m_ij;
        }
        for (int64_t d = 0; d < D; ++d)                          /* :879 acc += v^T p */
          for (int64_t g = 0; g < group; ++g) {
            float a = acc[d * group + g];
            for (int64_t n = 0; n < bn; ++n) {
              const int64_t key = j * bn + n;
              if (key < kv_cap) a += v[(h * kv_cap + key) * D + d] * qk[n * group + g];
            }
            acc[d * group + g] = a;
          }
      }
      for (int64_t g = 0; g < group; ++g) {
        float l_sum = 0.0f;
        for (int64_t n = 0; n < bn; ++n) l_sum += l_i[n * group + g];    /* :888-889 */
        const float l_safe = fmaxf(l_sum, 1.0e-8f);                      /* :891-892 */
        for (int64_t d = 0; d < D; ++d)
          att[((h * splits + sp) * group + g) * D + d] = round16(acc[d * group + g] / l_safe, is_f16);
        lse[(h * splits + sp) * group + g] = m_i[g] + log2f(l_safe);     /* :905 */
      }
    }
  free(qk); free(l_i); free(acc); free(m_i);
}

ORACLE_API void oracle_splitk_reduce_merge(const float* att, const float* lse, float* out, int64_t kv_heads,
                                           int64_t group, int64_t D, int64_t splits, int is_f16) {
  for (int64_t h = 0; h < kv_heads; ++h)
    for (int64_t g = 0; g < group; ++g) {
      float mx = -INFINITY;
      for (int64_t s = 0; s < splits; ++s) mx = fmaxf(mx, lse[(h * splits + s) * group + g]);   /* :975 */
      float sum = 0.0f;
      for (int64_t s = 0; s < splits; ++s) sum += exp2f(lse[(h * splits + s) * group + g] - mx);
      const float safe = fmaxf(sum, 1.0e-8f);                                                    /* :983-984 */
      for (int64_t d = 0; d < D; ++d) {
        float o = 0.0f;
        for (int64_t s = 0; s < splits; ++s)
          o += att[((h * splits + s) * group + g) * D + d] *
               (exp2f(lse[(h * splits + s) * group + g] - mx) / safe);                           /* :985-1009 */
        out[(h * group + g) * D + d] = round16(o, is_f16);
      }
    }
}
