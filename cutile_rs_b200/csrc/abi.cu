// The exported C ABI (include/b200tile.h): argument validation, configuration selection and
// forwarding to the per-kernel launchers.  Nothing here allocates, frees or synchronises on a
// launch path, so launches can be captured into CUDA graphs.
#include "../../include/b200tile.h"

#include <stdlib.h>
#include <string.h>
#include <cuda_fp16.h>

#include <mutex>
#include <vector>

#include "host_common.h"

// per-kernel launchers (defined next to their kernels)
int b200_gemm_tc_dispatch(int dtype, int b_kmajor, int config, const void* A, const void* B,
                          void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                          int group_m, int max_ctas, cudaStream_t stream);
#ifdef B200TILE_TEST_HOOKS
int b200_test_set_skip_stage(int on);
#endif
int b200_gemm_pair_reset_scratch(cudaStream_t stream);
int b200_gemm_pair_dispatch(int dtype, int b_kmajor, int wide, const void* A, const void* B, void* C, int M,
                            int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int group_m,
                            int max_ctas, cudaStream_t stream);
int b200_gemm_f32_dispatch(const float* A, const float* B, float* C, int batch, int M, int N,
                           int K, int64_t lda, int64_t ldb, int64_t ldc, int64_t sa, int64_t sb,
                           int64_t sc, int accumulate, cudaStream_t stream);

int b200_fmha_fwd_dispatch(int dtype, int head_dim, const void* q, const void* k, const void* v,
                           void* o, int batch, int heads, int heads_kv, int q_len, int kv_len,
                           const int64_t* qs, const int64_t* ks, const int64_t* vs,
                           const int64_t* os, float qk_scale, int causal, int input_pos,
                           const uint32_t* pos_ptr, cudaStream_t stream);

int b200_rms_norm_dispatch(int dtype, const void* residual, const void* x, const void* w, void* out,
                           void* residual_out, int rows, int n, long long ld_res, long long ld_x, long long ld_out,
                           long long ld_res_out, float eps, cudaStream_t stream);
int b200_rope_seq_dispatch(int dtype, const void* x, const float* inv_freq, void* out, int seq, int heads,
                           int head_dim, long long xs_seq, long long xs_head, long long os_seq, long long os_head,
                           int position_start, const uint32_t* pos_ptr, cudaStream_t stream);
int b200_qk_norm_rope_kv_dispatch(int dtype, const void* q, const void* k, const void* v, const void* q_weight,
                                  const void* k_weight, const float* inv_freq, void* q_out, void* k_cache,
                                  void* v_cache, float eps, int position_start, const uint32_t* pos_ptr, int seq,
                                  int q_heads, int kv_heads, int head_dim, int max_seq, long long q_ss,
                                  long long k_ss, long long v_ss, long long qo_ss, cudaStream_t stream);
int b200_argmax_blocks_dispatch(int dtype, const void* logits, float* block_max, uint32_t* block_idx, int len,
                                int block_size, cudaStream_t stream);
int b200_lm_head_argmax_blocks_dispatch(int dtype, const void* weights, const void* hidden, float* block_max,
                                        uint32_t* block_idx, int vocab, int k, long long ldw, cudaStream_t stream);
int b200_argmax_reduce_blocks_dispatch(const float* block_max, const uint32_t* block_idx, uint32_t* out,
                                       int num_blocks, cudaStream_t stream);
int b200_pointwise_dispatch(int dtype, int op, void* out, const void* a, const void* b, int rows, int cols,
                            long long ld_out, long long ld_a, long long ld_b, cudaStream_t stream);
int b200_fmha_fwd_alt_dispatch(int dtype, const void* q, const void* k, const void* v, void* o, int batch, int heads,
                               int heads_kv, int q_len, int kv_len, const int64_t* qs, const int64_t* ks,
                               const int64_t* vs, const int64_t* os, float qk_scale, int causal, int input_pos,
                               const uint32_t* pos_ptr, cudaStream_t stream);

#ifdef B200TILE_TRACE
int b200_trace_read_fmha_alt(long long* out);
int b200_trace_read_fmha_alt_t(long long* out);
int b200_trace_read_gemm_pair(long long* out);
int b200_trace_read_fmha(long long* out);
int b200_trace_read_fp4(long long* out);
int b200_trace_read_fp4_pair(long long* out);
int b200_trace_read_fp4_pair_tl(long long* out);
int b200_trace_read_grouped(long long* out);
#endif

int b200_gemm_fp8_blk_dispatch(int out_f32, const void* x, const void* y, const float* xs,
                               const float* ys, void* z, int M, int N, int K, int64_t ldx, int64_t ldy,
                               int64_t ldz, int ld_xs, int ld_ys, float alpha, cudaStream_t stream);

size_t b200_nvfp4_scratch_bytes(int M, int N, int K, int bn);
int b200_gemm_nvfp4_dispatch(int bn, int out_f32, const void* x, const void* y, const void* xs, const void* ys,
                             void* z, int M, int N, int K, int64_t ldx, int64_t ldy, int64_t ldz, int64_t ld_xs,
                             int64_t ld_ys, float alpha, void* scratch, cudaStream_t stream, int b_scales_prepared);
int b200_nvfp4_prepare_b_scales(const void* ys, int N, int K, int64_t ld_ys, int bn, void* out, cudaStream_t stream);

size_t b200_mxfp8_scratch_bytes(int M, int N, int K);
int b200_gemm_mxfp8_dispatch(int out_f32, const void* x, const void* y, const void* xs, const void* ys, void* z,
                             int M, int N, int K, int64_t ldx, int64_t ldy, int64_t ldz, int64_t ld_xs,
                             int64_t ld_ys, float alpha, void* scratch, cudaStream_t stream);
size_t b200_mxf4_scratch_bytes(int M, int N, int K);
// CTA-pair kernels of the block-scaled formats (fmt 1 = NVFP4, 2 = MXFP4, 0 = MXFP8)
size_t b200_blockscaled_pair_scratch_bytes(int fmt, int M, int N, int K);
int b200_gemm_blockscaled_pair_dispatch(int fmt, int out_f32, const void* x, const void* y, const void* xs,
                                        const void* ys, void* z, int M, int N, int K, int64_t ldx, int64_t ldy,
                                        int64_t ldz, int64_t ld_xs, int64_t ld_ys, float alpha, void* scratch,
                                        cudaStream_t stream);
// from this many rows on the CTA-pair kernels are ahead of the single-CTA ones (measured)
static const int kPairMinRows = 512;
int b200_gemm_mxf4_dispatch(int out_f32, const void* x, const void* y, const void* xs, const void* ys, void* z,
                            int M, int N, int K, int64_t ldx, int64_t ldy, int64_t ldz, int64_t ld_xs,
                            int64_t ld_ys, float alpha, void* scratch, cudaStream_t stream);

int b200_fmha_f32_dispatch(int head_dim, const void* q, const void* k, const void* v, void* out, int batch, int heads,
                           int heads_kv, int q_len, int kv_len, const int64_t* qs, const int64_t* ks,
                           const int64_t* vs, const int64_t* os, float qk_scale, int causal, int input_pos,
                           const uint32_t* pos_ptr, cudaStream_t stream);
int b200_fmha_decode_dispatch(int dtype, int head_dim, const void* q, const void* k, const void* v, void* att,
                              float* lse, void* out, const uint32_t* pos, int kv_heads, int group, int kv_cap,
                              int bn, int splits, float qk_scale, const int64_t* strides, cudaStream_t stream);
int b200_gemm_epilogue_dispatch(int dtype, const void* X, const void* W, const void* bias, const void* residual,
                                void* O, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ld_res, int64_t ldo,
                                cudaStream_t stream);
int b200_gemm_swiglu_dispatch(int dtype, const void* X, const void* W, void* O, int M, int I, int K, int64_t ldx,
                              int64_t ldw, int64_t ldo, cudaStream_t stream);
size_t b200_grouped_workspace_bytes(int groups);
int b200_gemm_grouped_dispatch(int dtype, int bn, const int64_t* a_ptrs, const int64_t* b_ptrs, const int64_t* c_ptrs,
                               const int32_t* a_metas, const int32_t* b_metas, const int32_t* c_metas, int groups,
                               void* workspace, cudaStream_t stream);
int b200_splitk_merge_dispatch(int dtype, int head_dim, const void* att, const float* lse, void* out, int kv_heads,
                               int group, int splits, const int64_t* strides, cudaStream_t stream);

using b200h::set_error;

static_assert(B200TILE_ERR_INVALID == B200_ERR_INVALID && B200TILE_ERR_ALIGN == B200_ERR_ALIGN &&
                  B200TILE_ERR_UNSUPPORTED == B200_ERR_UNSUPPORTED &&
                  B200TILE_ERR_CUDA == B200_ERR_CUDA && B200TILE_ERR_DEVICE == B200_ERR_DEVICE,
              "public and internal status codes must agree");

extern "C" {

int b200tile_abi_version(void) { return B200TILE_ABI_VERSION; }

const char* b200tile_last_error(void) { return b200h::last_error(); }

int b200tile_init(int device_ordinal) {
  B200_CUDA_CHECK(cudaSetDevice(device_ordinal));
  B200_CUDA_CHECK(cudaFree(0));  // materialise the primary context on this thread
  return b200h::device_info() ? B200TILE_OK : B200TILE_ERR_CUDA;
}

int b200tile_num_sms(void) {
  const b200h::DeviceInfo* di = b200h::device_info();
  return di ? di->sm_count : -1;
}

int b200tile_status(void* cu_stream, b200tile_status_t* out) {
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200TILE_ERR_CUDA;
  if (!out) return set_error(B200TILE_ERR_INVALID, "status: out is null");
  cudaStream_t s = static_cast<cudaStream_t>(cu_stream);
  uint32_t w[4] = {0, 0, 0, 0};
  B200_CUDA_CHECK(cudaMemcpyAsync(w, di->status, sizeof(w), cudaMemcpyDeviceToHost, s));
  B200_CUDA_CHECK(cudaStreamSynchronize(s));
  out->code = w[0];
  out->block = w[1];
  out->site = w[2];
  out->aux = w[3];
  if (w[0] != 0)
    return set_error(B200TILE_ERR_DEVICE,
                     "device status %u recorded by block %u at wait site %u (aux %u)", w[0], w[1],
                     w[2], w[3]);
  return B200TILE_OK;
}

int b200tile_status_reset(void* cu_stream) {
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200TILE_ERR_CUDA;
  B200_CUDA_CHECK(
      cudaMemsetAsync(di->status, 0, 4 * sizeof(uint32_t), static_cast<cudaStream_t>(cu_stream)));
  // a launch that gave up may have left stream-K hand-off flags raised
  return b200_gemm_pair_reset_scratch(static_cast<cudaStream_t>(cu_stream));
}

// ---------------------------------------------------------------------------
// Configuration tables
// ---------------------------------------------------------------------------
static const b200tile_config kGemmTcConfigs[] = {
    /* id  bm   bn   bk stages cga occ */
    {0, 128, 256, 64, 4, 1, 1},
    {1, 128, 128, 64, 6, 1, 1},
    {2, 256, 256, 64, 6, 2, 1},
    {3, 256, 512, 64, 4, 2, 1},
};
// f16 adds id 4: the 256 x 512 pair tile with f16 accumulators, the accumulator type of the reference's
// benchmark kernel (cutile-benchmarks/benches/gemm.rs:20-41: `mma(x, y, z)` with z a Tile<T>)
static const b200tile_config kGemmTcConfigsF16[] = {
    {0, 128, 256, 64, 4, 1, 1}, {1, 128, 128, 64, 6, 1, 1}, {2, 256, 256, 64, 6, 2, 1},
    {3, 256, 512, 64, 4, 2, 1}, {4, 256, 512, 64, 4, 2, 1},
};
static const b200tile_config kGemmF32Configs[] = {
    {0, 64, 64, 16, 1, 1, 1},
};

static bool is_gemm_name(const char* k) {
  return !strcmp(k, "gemm") || !strcmp(k, "gemm_acc") || !strcmp(k, "gemm_persistent") ||
         !strcmp(k, "batch_matmul") || !strcmp(k, "gemm_static");
}

int b200tile_query_configs(const char* kernel, const char* dtype, b200tile_config* out, int cap) {
  if (!kernel || !dtype) return 0;
  const b200tile_config* tab = nullptr;
  int n = 0;
  if (is_gemm_name(kernel)) {
    if (!strcmp(dtype, "f32")) {
      tab = kGemmF32Configs;
      n = (int)(sizeof(kGemmF32Configs) / sizeof(kGemmF32Configs[0]));
    } else if (!strcmp(dtype, "bf16")) {
      tab = kGemmTcConfigs;
      n = (int)(sizeof(kGemmTcConfigs) / sizeof(kGemmTcConfigs[0]));
    } else if (!strcmp(dtype, "f16")) {
      tab = kGemmTcConfigsF16;
      n = (int)(sizeof(kGemmTcConfigsF16) / sizeof(kGemmTcConfigsF16[0]));
    }
  }
  static const b200tile_config kFmhaConfigs[] = {{0, 128, 128, 0, 2, 1, 1}, {1, 128, 128, 0, 4, 2, 1}};
  if ((!strcmp(kernel, "fmha") || !strcmp(kernel, "fmha_prefill_causal") ||
       !strcmp(kernel, "fmha_prefill_gqa") || !strcmp(kernel, "fmha_causal")) &&
      (!strcmp(dtype, "bf16") || !strcmp(dtype, "f16"))) {
    tab = kFmhaConfigs;
    n = 2;
  }
  static const b200tile_config kFp8Configs[] = {{0, 128, 256, 128, 4, 1, 1}};
  if (!strcmp(kernel, "linear_tile_fp8_blk128")) {
    tab = kFp8Configs;
    n = 1;
  }
  // `linear_tile`: dtype names the OPERAND type, which is what separates the two reference kernels of that
  // name (f4e2m1fnx2 = NVFP4, e4m3 scale per 16; f8e4m3fn = MXFP8, e8m0 scale per 32).  The launcher's tile
  // generics only shape the launch grid; the kernel's own tile is the configuration listed here.
  static const b200tile_config kNvfp4Configs[] = {{0, 128, 128, 256, 5, 1, 1}, {1, 128, 192, 256, 4, 1, 1},
                                                  {2, 128, 256, 256, 3, 1, 1}, {3, 256, 256, 256, 5, 2, 1}};
  static const b200tile_config kMxfp8Configs[] = {{0, 128, 224, 128, 4, 1, 1}};
  if (!strcmp(kernel, "linear_tile")) {
    if (!strcmp(dtype, "f4e2m1fnx2")) {
      tab = kNvfp4Configs;
      n = 4;
    } else if (!strcmp(dtype, "f8e4m3fn")) {
      tab = kMxfp8Configs;
      n = 1;
    }
  }
  for (int i = 0; i < n && i < cap && out; ++i) out[i] = tab[i];
  return n;
}

// Default configuration: the one with the least (waves x per-SM tile work / relative speed).
// Relative speeds are the measured ratios of the kernels at 8192^3 (the 256 x 512 pair tile moves three quarters
// of the 256 x 256 tile's bytes per FLOP and is 3.6 % ahead there).  The pair kernels split a partial last wave
// along K (stream-K) when K is deep enough, so their wave count is fractional above one wave.
static int default_gemm_config(int m, int n, int k) {
  const b200h::DeviceInfo* di = b200h::device_info();
  const int64_t sms = di ? di->sm_count : 148;
  auto cdiv = [](int64_t a, int64_t b) { return (a + b - 1) / b; };
  auto pair_waves = [&](int64_t tiles, int bk) {
    const int64_t pairs = sms / 2;
    if (tiles <= pairs) return 1.0;
    if (cdiv(k, bk) >= 4) return 1.03 * (double)tiles / (double)pairs;
    return (double)cdiv(tiles, pairs);
  };
  const double cost0 = (double)cdiv(cdiv(m, 128) * cdiv(n, 256), sms) * 1.0 / 0.92;
  const double cost1 = (double)cdiv(cdiv(m, 128) * cdiv(n, 128), sms) * 0.5 / 0.72;
  const double cost2 = pair_waves(cdiv(m, 256) * cdiv(n, 256), 128) * 1.0 / 1.0;
  // the 512-wide tile is only taken in whole waves: its K-split fix-up (256 KiB of partials per CTA) costs more
  // than it recovers (8192 x 1024 x 8192: 1182 TFLOP/s against 1369 for the 256-wide tile with its K split)
  const double cost3 = (double)cdiv(cdiv(m, 256) * cdiv(n, 512), sms / 2) * 2.0 / 1.036;
  if (cost3 <= cost2 && cost3 <= cost0 && cost3 <= cost1) return 3;
  if (cost2 <= cost0 && cost2 <= cost1) return 2;
  return cost0 <= cost1 ? 0 : 1;
}

// ---------------------------------------------------------------------------
// Typed GEMM entry point
// ---------------------------------------------------------------------------
int b200tile_gemm(const char* dtype, int b_layout, const void* a, const void* b, void* c,
                  int batch, int m, int n, int k, int64_t lda, int64_t ldb, int64_t ldc,
                  int64_t stride_a, int64_t stride_b, int64_t stride_c, int accumulate, int config,
                  int group_size_m, int num_programs, void* cu_stream) {
  if (!dtype) return set_error(B200TILE_ERR_INVALID, "gemm: dtype is null");
  if (!a || !b || !c) return set_error(B200TILE_ERR_INVALID, "gemm: null tensor pointer");
  if (m <= 0 || n <= 0 || k <= 0 || batch <= 0)
    return set_error(B200TILE_ERR_INVALID,
                     "gemm: Shape dimensions must be positive (batch %d, m %d, n %d, k %d)", batch,
                     m, n, k);
  const int64_t b_cols = b_layout ? k : n;
  if (lda < k || ldb < b_cols || ldc < n)
    return set_error(B200TILE_ERR_INVALID, "gemm: leading dimension smaller than the row length");
  cudaStream_t stream = static_cast<cudaStream_t>(cu_stream);
  if (group_size_m <= 0) group_size_m = 8;

  if (!strcmp(dtype, "f32")) {
    if (b_layout != 0)
      return set_error(B200TILE_ERR_UNSUPPORTED, "gemm(f32): only B[K,N] is provided");
    if (config > 0)
      return set_error(B200TILE_ERR_UNSUPPORTED, "gemm(f32): unknown config %d", config);
    return b200_gemm_f32_dispatch(static_cast<const float*>(a), static_cast<const float*>(b),
                                  static_cast<float*>(c), batch, m, n, k, lda, ldb, ldc, stride_a,
                                  stride_b, stride_c, accumulate, stream);
  }
  int dt;
  if (!strcmp(dtype, "bf16"))
    dt = 0;
  else if (!strcmp(dtype, "f16"))
    dt = 1;
  else
    return set_error(B200TILE_ERR_UNSUPPORTED, "gemm: unsupported element type '%s'", dtype);
  if (accumulate)
    return set_error(B200TILE_ERR_UNSUPPORTED,
                     "gemm(%s): accumulate-into-C is only provided for f32", dtype);
  if (config < 0) config = default_gemm_config(m, n, k);
  if (config > 4 || (config == 4 && dt != 1))
    return set_error(B200TILE_ERR_UNSUPPORTED, "gemm(%s): unknown config %d", dtype, config);
  for (int bi = 0; bi < batch; ++bi) {
    const char* ab = static_cast<const char*>(a) + (int64_t)bi * stride_a * 2;
    const char* bb = static_cast<const char*>(b) + (int64_t)bi * stride_b * 2;
    char* cb = static_cast<char*>(c) + (int64_t)bi * stride_c * 2;
    int rc = config >= 2
                 ? b200_gemm_pair_dispatch(dt, b_layout ? 1 : 0, config - 2, ab, bb, cb, m, n, k, lda, ldb,
                                           ldc, group_size_m, num_programs, stream)
                 : b200_gemm_tc_dispatch(dt, b_layout ? 1 : 0, config, ab, bb, cb, m, n, k, lda,
                                         ldb, ldc, group_size_m, num_programs, stream);
    if (rc) return rc;
  }
  return B200TILE_OK;
}


// ---------------------------------------------------------------------------
// Typed attention entry point
// ---------------------------------------------------------------------------
static int fmha_fwd_common(const char* dtype, const void* q, const void* k, const void* v, void* out,
                           int batch, int heads, int heads_kv, int q_len, int kv_len, int head_dim,
                           const int64_t q_strides[2], const int64_t k_strides[2],
                           const int64_t v_strides[2], const int64_t o_strides[2], float qk_scale,
                           int causal, int input_pos, const uint32_t* pos_ptr, void* cu_stream,
                           int cluster = 0) {
  if (!dtype) return set_error(B200TILE_ERR_INVALID, "fmha: dtype is null");
  if (!q || !k || !v || !out) return set_error(B200TILE_ERR_INVALID, "fmha: null tensor pointer");
  if (!q_strides || !k_strides || !v_strides || !o_strides)
    return set_error(B200TILE_ERR_INVALID, "fmha: null stride array");
  if (batch <= 0 || heads <= 0 || heads_kv <= 0 || q_len <= 0 || kv_len <= 0)
    return set_error(B200TILE_ERR_INVALID, "fmha: Shape dimensions must be positive");
  if (heads % heads_kv != 0)
    return set_error(B200TILE_ERR_INVALID, "fmha: heads (%d) must be a multiple of heads_kv (%d)",
                     heads, heads_kv);
  if (input_pos < 0) return set_error(B200TILE_ERR_INVALID, "fmha: input_pos must be >= 0");
  if (!strcmp(dtype, "f32"))   // exact fp32 on the CUDA cores: the element type of the reference's asserted examples
    return b200_fmha_f32_dispatch(head_dim, q, k, v, out, batch, heads, heads_kv, q_len, kv_len, q_strides, k_strides,
                                  v_strides, o_strides, qk_scale, causal ? 1 : 0, input_pos, pos_ptr,
                                  static_cast<cudaStream_t>(cu_stream));
  int dt;
  if (!strcmp(dtype, "bf16"))
    dt = 0;
  else if (!strcmp(dtype, "f16"))
    dt = 1;
  else
    return set_error(B200TILE_ERR_UNSUPPORTED, "fmha: unsupported element type '%s'", dtype);
  // Two configurations for head_dim 128: one CTA per 256 query rows with S and P sharing their
  // Tensor Memory columns (default), and persistent CTA pairs with cta_group::2 MMAs, separate S and
  // P buffers and two alternating softmax warpgroups, chosen with CompileOptions::num_cta_in_cga = 2
  // on the generic launch or B200TILE_FMHA_PAIR=1.
  static const bool env_pair = [] {
    const char* e = getenv("B200TILE_FMHA_PAIR");
    return e && e[0] != '0';
  }();
  // Unspecified (cluster == 0): the default kernel, except where its 256-row CTAs would leave the last wave mostly
  // empty -- non-causal problems whose CTA count is a few waves with less than 0.9 of the last one used (the shard
  // of 8 x 32 heads x 4096 on one of eight GPUs: 512 CTAs = 3.46 waves, 1060 TFLOP/s against 1140 for the
  // persistent pair kernel, which deals out 128-row items).
  bool auto_pair = false;
  if (cluster == 0 && !env_pair && head_dim == 128 && !causal && heads == heads_kv && q_len % 256 == 0 && kv_len >= 2048) {
    const b200h::DeviceInfo* di = b200h::device_info();
    const int64_t sms = di ? di->sm_count : 148;
    const int64_t ctas = (int64_t)batch * heads * (q_len / 256);
    const int64_t waves = (ctas + sms - 1) / sms;
    auto_pair = waves >= 2 && waves <= 5 && (double)ctas / (double)(waves * sms) < 0.9;
  }
  if (head_dim == 128 && (cluster == 2 || (cluster == 0 && (env_pair || auto_pair))))
    return b200_fmha_fwd_alt_dispatch(dt, q, k, v, out, batch, heads, heads_kv, q_len, kv_len, q_strides,
                                      k_strides, v_strides, o_strides, qk_scale, causal ? 1 : 0, input_pos,
                                      pos_ptr, static_cast<cudaStream_t>(cu_stream));
  return b200_fmha_fwd_dispatch(dt, head_dim, q, k, v, out, batch, heads, heads_kv, q_len, kv_len,
                                q_strides, k_strides, v_strides, o_strides, qk_scale,
                                causal ? 1 : 0, input_pos, pos_ptr, static_cast<cudaStream_t>(cu_stream));
}

int b200tile_fmha_fwd(const char* dtype, const void* q, const void* k, const void* v, void* out,
                      int batch, int heads, int heads_kv, int q_len, int kv_len, int head_dim,
                      const int64_t q_strides[2], const int64_t k_strides[2],
                      const int64_t v_strides[2], const int64_t o_strides[2], float qk_scale,
                      int causal, int input_pos, void* cu_stream) {
  return fmha_fwd_common(dtype, q, k, v, out, batch, heads, heads_kv, q_len, kv_len, head_dim, q_strides,
                         k_strides, v_strides, o_strides, qk_scale, causal, input_pos, nullptr, cu_stream);
}

int b200tile_fmha_fwd_dynpos(const char* dtype, const void* q, const void* k, const void* v, void* out,
                             int batch, int heads, int heads_kv, int q_len, int kv_len, int head_dim,
                             const int64_t q_strides[2], const int64_t k_strides[2],
                             const int64_t v_strides[2], const int64_t o_strides[2], float qk_scale,
                             int causal, const void* position_start, void* cu_stream) {
  if (!position_start) return set_error(B200TILE_ERR_INVALID, "fmha_dynpos: position_start is null");
  if ((reinterpret_cast<uintptr_t>(position_start) & 3) != 0)
    return set_error(B200TILE_ERR_ALIGN, "fmha_dynpos: position_start must be 4-byte aligned");
  return fmha_fwd_common(dtype, q, k, v, out, batch, heads, heads_kv, q_len, kv_len, head_dim, q_strides,
                         k_strides, v_strides, o_strides, qk_scale, causal, 0,
                         static_cast<const uint32_t*>(position_start), cu_stream);
}

// ---------------------------------------------------------------------------
// Typed decode-attention entry points
// ---------------------------------------------------------------------------
static int decode_dtype(const char* dtype, const char* who, int* dt) {
  if (!dtype) return set_error(B200TILE_ERR_INVALID, "%s: dtype is null", who);
  if (!strcmp(dtype, "bf16")) *dt = 0;
  else if (!strcmp(dtype, "f16")) *dt = 1;
  else return set_error(B200TILE_ERR_UNSUPPORTED, "%s: unsupported element type '%s'", who, dtype);
  return B200TILE_OK;
}

int b200tile_fmha_decode_gqa_split(const char* dtype, const void* q, const void* k, const void* v,
                                   void* att_partial, float* lse_partial, void* out,
                                   const void* position_start, int kv_heads, int group, int head_dim,
                                   int kv_capacity, int bn, int num_kv_splits, float qk_scale,
                                   const int64_t q_strides[2], const int64_t k_strides[2],
                                   const int64_t v_strides[2], const int64_t att_strides[2],
                                   int64_t lse_head_stride, const int64_t out_strides[2], void* cu_stream) {
  int dt;
  if (int rc = decode_dtype(dtype, "fmha_decode_gqa_split", &dt)) return rc;
  if (!q || !k || !v || !att_partial || !lse_partial || !position_start || !q_strides || !k_strides ||
      !v_strides || !att_strides || (out && !out_strides))
    return set_error(B200TILE_ERR_INVALID, "fmha_decode_gqa_split: null argument");
  if (kv_heads <= 0 || group <= 0 || kv_capacity <= 0 || bn <= 0 || num_kv_splits <= 0)
    return set_error(B200TILE_ERR_INVALID, "fmha_decode_gqa_split: Shape dimensions must be positive");
  if (group > 16)
    return set_error(B200TILE_ERR_UNSUPPORTED, "fmha_decode_gqa_split: GROUP=%d exceeds 16", group);
  if (num_kv_splits > 65535)
    return set_error(B200TILE_ERR_INVALID, "fmha_decode_gqa_split: too many splits");
  const uintptr_t al = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                       reinterpret_cast<uintptr_t>(v);
  if ((al & 15) != 0 || (k_strides[0] % 8) || (k_strides[1] % 8) || (v_strides[0] % 8) || (v_strides[1] % 8) ||
      (q_strides[0] % 2) || (q_strides[1] % 2))
    return set_error(B200TILE_ERR_ALIGN, "fmha_decode_gqa_split: q/k/v rows must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(att_partial) & 3) || (att_strides[0] % 2) || (att_strides[1] % 2) ||
      (out && ((reinterpret_cast<uintptr_t>(out) & 3) || (out_strides[0] % 2) || (out_strides[1] % 2))))
    return set_error(B200TILE_ERR_ALIGN, "fmha_decode_gqa_split: att_partial/out rows must be 4-byte aligned");
  const int64_t strides[11] = {q_strides[0], q_strides[1], k_strides[0], k_strides[1], v_strides[0], v_strides[1],
                               att_strides[0], att_strides[1], lse_head_stride, out ? out_strides[0] : 0,
                               out ? out_strides[1] : 0};
  return b200_fmha_decode_dispatch(dt, head_dim, q, k, v, att_partial, lse_partial, out,
                                   static_cast<const uint32_t*>(position_start), kv_heads, group, kv_capacity, bn,
                                   num_kv_splits, qk_scale, strides, static_cast<cudaStream_t>(cu_stream));
}

int b200tile_splitk_reduce_merge(const char* dtype, const void* att_partial, const float* lse_partial, void* out,
                                 int kv_heads, int group, int head_dim, int num_kv_splits,
                                 const int64_t att_strides[2], int64_t lse_head_stride,
                                 const int64_t out_strides[2], void* cu_stream) {
  int dt;
  if (int rc = decode_dtype(dtype, "splitk_reduce_merge", &dt)) return rc;
  if (!att_partial || !lse_partial || !out || !att_strides || !out_strides)
    return set_error(B200TILE_ERR_INVALID, "splitk_reduce_merge: null argument");
  if (kv_heads <= 0 || group <= 0 || head_dim <= 0 || num_kv_splits <= 0)
    return set_error(B200TILE_ERR_INVALID, "splitk_reduce_merge: Shape dimensions must be positive");
  if ((reinterpret_cast<uintptr_t>(att_partial) & 3) || (att_strides[0] % 2) || (att_strides[1] % 2) ||
      (reinterpret_cast<uintptr_t>(out) & 3) || (out_strides[0] % 2) || (out_strides[1] % 2))
    return set_error(B200TILE_ERR_ALIGN, "splitk_reduce_merge: att_partial/out rows must be 4-byte aligned");
  const int64_t strides[5] = {att_strides[0], att_strides[1], lse_head_stride, out_strides[0], out_strides[1]};
  return b200_splitk_merge_dispatch(dt, head_dim, att_partial, lse_partial, out, kv_heads, group, num_kv_splits,
                                    strides, static_cast<cudaStream_t>(cu_stream));
}

// ---------------------------------------------------------------------------
// Linear layer with the SwiGLU pointwise step fused into its epilogue
// ---------------------------------------------------------------------------
int b200tile_linear_swiglu(const char* dtype, const void* x, const void* w_gate_up, void* out, int m, int inter,
                           int k, int64_t ldx, int64_t ldw, int64_t ldo, void* cu_stream) {
  int dt;
  if (int rc = decode_dtype(dtype, "linear_swiglu", &dt)) return rc;
  if (!x || !w_gate_up || !out) return set_error(B200TILE_ERR_INVALID, "linear_swiglu: null tensor pointer");
  if (m <= 0 || inter <= 0 || k <= 0)
    return set_error(B200TILE_ERR_INVALID, "linear_swiglu: Shape dimensions must be positive");
  if (ldx < k || ldw < k || ldo < inter)
    return set_error(B200TILE_ERR_INVALID, "linear_swiglu: a leading dimension is smaller than its row");
  const uintptr_t al = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w_gate_up) |
                       reinterpret_cast<uintptr_t>(out);
  if ((al & 15) != 0 || (ldx % 8) || (ldw % 8) || (ldo % 8))
    return set_error(B200TILE_ERR_ALIGN, "linear_swiglu: base pointers and row pitches must be 16-byte aligned");
  return b200_gemm_swiglu_dispatch(dt, x, w_gate_up, out, m, inter, k, ldx, ldw, ldo,
                                   static_cast<cudaStream_t>(cu_stream));
}

int b200tile_linear_bias_residual(const char* dtype, const void* x, const void* w, const void* bias,
                                  const void* residual, void* out, int m, int n, int k, int64_t ldx, int64_t ldw,
                                  int64_t ld_residual, int64_t ldo, void* cu_stream) {
  int dt;
  if (int rc = decode_dtype(dtype, "linear_bias_residual", &dt)) return rc;
  if (!x || !w || !out) return set_error(B200TILE_ERR_INVALID, "linear_bias_residual: null tensor pointer");
  if (m <= 0 || n <= 0 || k <= 0)
    return set_error(B200TILE_ERR_INVALID, "linear_bias_residual: Shape dimensions must be positive");
  if (ldx < k || ldw < k || ldo < n || (residual && ld_residual < n))
    return set_error(B200TILE_ERR_INVALID, "linear_bias_residual: a leading dimension is smaller than its row");
  const uintptr_t al = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out) |
                       reinterpret_cast<uintptr_t>(bias) | reinterpret_cast<uintptr_t>(residual);
  if ((al & 15) != 0 || (ldx % 8) || (ldw % 8) || (ldo % 8) || (residual && (ld_residual % 8)))
    return set_error(B200TILE_ERR_ALIGN, "linear_bias_residual: base pointers and row pitches must be 16-byte aligned");
  return b200_gemm_epilogue_dispatch(dt, x, w, bias, residual, out, m, n, k, ldx, ldw, ld_residual, ldo,
                                     static_cast<cudaStream_t>(cu_stream));
}

// ---------------------------------------------------------------------------
// Grouped GEMM over device-side pointer / extent tables
// ---------------------------------------------------------------------------
uint64_t b200tile_group_gemm_workspace_bytes(int num_groups) { return b200_grouped_workspace_bytes(num_groups); }

int b200tile_group_gemm(const char* dtype, const int64_t* a_ptrs, const int64_t* b_ptrs, const int64_t* c_ptrs,
                        const int32_t* a_metas, const int32_t* b_metas, const int32_t* c_metas, int num_groups,
                        int bn, void* workspace, uint64_t workspace_bytes, void* cu_stream) {
  int dt;
  if (int rc = decode_dtype(dtype, "group_gemm", &dt)) return rc;
  if (num_groups < 0) return set_error(B200TILE_ERR_INVALID, "group_gemm: num_groups must not be negative");
  if (num_groups == 0) return B200TILE_OK;
  if (!a_ptrs || !b_ptrs || !c_ptrs || !a_metas || !b_metas || !c_metas)
    return set_error(B200TILE_ERR_INVALID, "group_gemm: null table pointer");
  if (bn <= 0) bn = 256;
  cudaStream_t stream = static_cast<cudaStream_t>(cu_stream);
  const size_t need = b200_grouped_workspace_bytes(num_groups);
  if (!workspace) {
    // library-owned workspace, one per (device, stream), grown on demand (never inside a stream capture)
    workspace = b200h::stream_scratch(stream, need, "group_gemm");
    if (!workspace) return B200TILE_ERR_INVALID;
  } else if ((reinterpret_cast<uintptr_t>(workspace) & 127) != 0 || workspace_bytes < need) {
    return set_error(B200TILE_ERR_INVALID, "group_gemm: workspace of %llu bytes (128-byte aligned) required, got %llu",
                     (unsigned long long)need, (unsigned long long)workspace_bytes);
  }
  return b200_gemm_grouped_dispatch(dt, bn, a_ptrs, b_ptrs, c_ptrs, a_metas, b_metas, c_metas, num_groups, workspace,
                                    stream);
}

// ---------------------------------------------------------------------------
// Typed block-scaled fp8 entry point
// ---------------------------------------------------------------------------
int b200tile_linear_fp8_blk128(const void* x, const void* y, const float* x_scales,
                               const float* y_scales, void* z, const char* out_dtype, int m, int n,
                               int k, int64_t ldx, int64_t ldy, int64_t ldz, int64_t ld_xs,
                               int64_t ld_ys, float alpha, void* cu_stream) {
  if (!x || !y || !x_scales || !y_scales || !z || !out_dtype)
    return set_error(B200TILE_ERR_INVALID, "linear_fp8_blk128: null argument");
  if (m <= 0 || n <= 0 || k <= 0)
    return set_error(B200TILE_ERR_INVALID, "linear_fp8_blk128: Shape dimensions must be positive");
  if (k % 128 != 0)
    return set_error(B200TILE_ERR_INVALID,
                     "linear_fp8_blk128: K (%d) must be a multiple of the 128-element scale block", k);
  if (ldx < k || ldy < k || ldz < n || ld_xs < k / 128 || ld_ys < k / 128)
    return set_error(B200TILE_ERR_INVALID, "linear_fp8_blk128: leading dimension too small");
  int out_f32;
  if (!strcmp(out_dtype, "f32")) out_f32 = 1;
  else if (!strcmp(out_dtype, "bf16")) out_f32 = 0;
  else return set_error(B200TILE_ERR_UNSUPPORTED, "linear_fp8_blk128: unsupported output type '%s'", out_dtype);
  if ((reinterpret_cast<uintptr_t>(z) & 15) != 0 || (ldz * (out_f32 ? 4 : 2)) % 16 != 0)
    return set_error(B200TILE_ERR_ALIGN, "linear_fp8_blk128: output must be 16-byte aligned with a 16-byte pitch");
  return b200_gemm_fp8_blk_dispatch(out_f32, x, y, x_scales, y_scales, z, m, n, k, ldx, ldy, ldz,
                                    (int)ld_xs, (int)ld_ys, alpha, static_cast<cudaStream_t>(cu_stream));
}

// ---------------------------------------------------------------------------
// Typed NVFP4 entry point
// ---------------------------------------------------------------------------
static const int kNvfp4Bn[3] = {128, 192, 256};

uint64_t b200tile_linear_nvfp4_workspace_bytes(int m, int n, int k) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  size_t best = 0;
  for (int i = 0; i < 3; ++i) {
    const size_t b = b200_nvfp4_scratch_bytes(m, n, k, kNvfp4Bn[i]);
    if (b > best) best = b;
  }
  const size_t pair = b200_blockscaled_pair_scratch_bytes(1, m, n, k);
  if (pair > best) best = pair;
  return (uint64_t)best;
}

int b200tile_linear_nvfp4(const void* x, const void* y, const void* x_scales, const void* y_scales,
                          void* z, const char* out_dtype, int m, int n, int k, int64_t ldx, int64_t ldy,
                          int64_t ldz, int64_t ld_xs, int64_t ld_ys, float alpha, void* workspace,
                          uint64_t workspace_bytes, int config, void* cu_stream) {
  if (!x || !y || !x_scales || !y_scales || !z || !out_dtype)
    return set_error(B200TILE_ERR_INVALID, "linear_nvfp4: null argument");
  if (m <= 0 || n <= 0 || k <= 0)
    return set_error(B200TILE_ERR_INVALID, "linear_nvfp4: Shape dimensions must be positive");
  if (k % 64 != 0)
    return set_error(B200TILE_ERR_INVALID, "linear_nvfp4: K (%d) must be a multiple of 64", k);
  if (ldx < k / 2 || ldy < k / 2 || ldz < n || ld_xs < k / 16 || ld_ys < k / 16)
    return set_error(B200TILE_ERR_INVALID, "linear_nvfp4: leading dimension too small");
  if (ld_xs % 4 != 0 || ld_ys % 4 != 0 || (reinterpret_cast<uintptr_t>(x_scales) & 3) != 0 ||
      (reinterpret_cast<uintptr_t>(y_scales) & 3) != 0)
    return set_error(B200TILE_ERR_ALIGN, "linear_nvfp4: scale rows must be 4-byte aligned");
  int out_f32;
  if (!strcmp(out_dtype, "f32")) out_f32 = 1;
  else if (!strcmp(out_dtype, "bf16")) out_f32 = 0;
  else return set_error(B200TILE_ERR_UNSUPPORTED, "linear_nvfp4: unsupported output type '%s'", out_dtype);
  if ((reinterpret_cast<uintptr_t>(z) & 15) != 0 || (ldz * (out_f32 ? 4 : 2)) % 16 != 0)
    return set_error(B200TILE_ERR_ALIGN, "linear_nvfp4: output must be 16-byte aligned with a 16-byte pitch");
  if (config < -1 || config > 3)
    return set_error(B200TILE_ERR_UNSUPPORTED, "linear_nvfp4: unknown config %d", config);
  // default: CTA pairs (256 x 256 tiles) from 512 rows on (measured ahead of the single-CTA tiles at every such
  // shape: 8 % at 4096 x 14336 x 4096, 24 % at 8192 x 28672 x 8192); below that 192-row B tiles, and decode-sized M
  // takes 128-row tiles (more CTAs for the weight stream, and the short-A-tile configuration exists for that tile only)
  if (config < 0) config = m <= 32 ? 0 : (m >= kPairMinRows ? 3 : 1);
  if (config == 3) {   // CTA pairs, 256 x 256 tiles
    const size_t need = b200_blockscaled_pair_scratch_bytes(1, m, n, k);
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15) != 0 || workspace_bytes < need)
      return set_error(B200TILE_ERR_INVALID,
                       "linear_nvfp4: workspace of %llu bytes (16-byte aligned) required, got %llu",
                       (unsigned long long)need, (unsigned long long)workspace_bytes);
    if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || (reinterpret_cast<uintptr_t>(y) & 15) != 0 || ldx % 16 != 0 ||
        ldy % 16 != 0)
      return set_error(B200TILE_ERR_ALIGN, "linear_nvfp4: operand rows must be 16-byte aligned");
    return b200_gemm_blockscaled_pair_dispatch(1, out_f32, x, y, x_scales, y_scales, z, m, n, k, ldx, ldy, ldz, ld_xs,
                                               ld_ys, alpha, workspace, static_cast<cudaStream_t>(cu_stream));
  }
  const int bn = kNvfp4Bn[config];
  const size_t need = b200_nvfp4_scratch_bytes(m, n, k, bn);
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15) != 0 || workspace_bytes < need)
    return set_error(B200TILE_ERR_INVALID,
                     "linear_nvfp4: workspace of %llu bytes (16-byte aligned) required, got %llu",
                     (unsigned long long)need, (unsigned long long)workspace_bytes);
  return b200_gemm_nvfp4_dispatch(bn, out_f32, x, y, x_scales, y_scales, z, m, n, k, ldx, ldy, ldz, ld_xs,
                                  ld_ys, alpha, workspace, static_cast<cudaStream_t>(cu_stream), 0);
}

// Weight scales laid out once (inference weights do not change): no per-call pre-pass, no workspace.
uint64_t b200tile_nvfp4_weight_scales_bytes(int n, int k, int config) {
  if (n <= 0 || k <= 0 || config < 0 || config > 2) return 0;
  return (uint64_t)b200_nvfp4_scratch_bytes(1, n, k, kNvfp4Bn[config]);
}

int b200tile_nvfp4_prepare_weight_scales(const void* y_scales, int n, int k, int64_t ld_ys, int config,
                                         void* prepared, uint64_t prepared_bytes, void* cu_stream) {
  if (!y_scales || !prepared) return set_error(B200TILE_ERR_INVALID, "nvfp4_prepare_weight_scales: null argument");
  if (n <= 0 || k <= 0 || k % 64 != 0)
    return set_error(B200TILE_ERR_INVALID, "nvfp4_prepare_weight_scales: n, k must be positive and K a multiple of 64");
  if (config < 0 || config > 2)
    return set_error(B200TILE_ERR_UNSUPPORTED, "nvfp4_prepare_weight_scales: config must be 0, 1 or 2 (got %d)", config);
  if (ld_ys < k / 16 || ld_ys % 4 != 0 || (reinterpret_cast<uintptr_t>(y_scales) & 3) != 0)
    return set_error(B200TILE_ERR_ALIGN, "nvfp4_prepare_weight_scales: scale rows must be 4-byte aligned");
  const uint64_t need = b200tile_nvfp4_weight_scales_bytes(n, k, config);
  if ((reinterpret_cast<uintptr_t>(prepared) & 15) != 0 || prepared_bytes < need)
    return set_error(B200TILE_ERR_INVALID,
                     "nvfp4_prepare_weight_scales: buffer of %llu bytes (16-byte aligned) required, got %llu",
                     (unsigned long long)need, (unsigned long long)prepared_bytes);
  return b200_nvfp4_prepare_b_scales(y_scales, n, k, ld_ys, kNvfp4Bn[config], prepared,
                                     static_cast<cudaStream_t>(cu_stream));
}

int b200tile_linear_nvfp4_prepared(const void* x, const void* y, const void* x_scales,
                                   const void* y_scales_prepared, void* z, const char* out_dtype, int m, int n,
                                   int k, int64_t ldx, int64_t ldy, int64_t ldz, int64_t ld_xs, float alpha,
                                   int config, void* cu_stream) {
  if (!x || !y || !x_scales || !y_scales_prepared || !z || !out_dtype)
    return set_error(B200TILE_ERR_INVALID, "linear_nvfp4_prepared: null argument");
  if (m <= 0 || n <= 0 || k <= 0)
    return set_error(B200TILE_ERR_INVALID, "linear_nvfp4_prepared: Shape dimensions must be positive");
  if (k % 64 != 0)
    return set_error(B200TILE_ERR_INVALID, "linear_nvfp4_prepared: K (%d) must be a multiple of 64", k);
  if (ldx < k / 2 || ldy < k / 2 || ldz < n || ld_xs < k / 16)
    return set_error(B200TILE_ERR_INVALID, "linear_nvfp4_prepared: leading dimension too small");
  if (ld_xs % 4 != 0 || (reinterpret_cast<uintptr_t>(x_scales) & 3) != 0 ||
      (reinterpret_cast<uintptr_t>(y_scales_prepared) & 15) != 0)
    return set_error(B200TILE_ERR_ALIGN, "linear_nvfp4_prepared: scale rows must be 4-byte aligned");
  int out_f32;
  if (!strcmp(out_dtype, "f32")) out_f32 = 1;
  else if (!strcmp(out_dtype, "bf16")) out_f32 = 0;
  else return set_error(B200TILE_ERR_UNSUPPORTED, "linear_nvfp4_prepared: unsupported output type '%s'", out_dtype);
  if ((reinterpret_cast<uintptr_t>(z) & 15) != 0 || (ldz * (out_f32 ? 4 : 2)) % 16 != 0)
    return set_error(B200TILE_ERR_ALIGN, "linear_nvfp4_prepared: output must be 16-byte aligned with a 16-byte pitch");
  if (config < 0 || config > 2)
    return set_error(B200TILE_ERR_UNSUPPORTED,
                     "linear_nvfp4_prepared: config must be the one the scales were prepared for (0, 1 or 2)");
  return b200_gemm_nvfp4_dispatch(kNvfp4Bn[config], out_f32, x, y, x_scales, nullptr, z, m, n, k, ldx, ldy, ldz,
                                  ld_xs, 0, alpha, const_cast<void*>(y_scales_prepared),
                                  static_cast<cudaStream_t>(cu_stream), 1);
}

// Registry of prepared weight scales: the reference's `linear_tile` takes logically row-major scales on every
// call, but inference weights do not change, so a serving loop can lay their scales out once
// (b200tile_nvfp4_prepare_weight_scales) and register the result under the address of the row-major tensor.
// `b200tile_launch("linear_tile", ...)` then finds decode-sized calls on that weight and skips the per-call
// re-layout.  The caller owns both buffers and must unregister before freeing either.
namespace {
struct Nvfp4Registered {
  int device;
  const void* y_scales;
  int n, k;
  int64_t ld_ys;
  const void* prepared;
  int config;
};
std::vector<Nvfp4Registered> g_nvfp4_registry;
std::mutex g_nvfp4_registry_mu;
}  // namespace

bool nvfp4_registry_find(const void* y_scales, int n, int k, int64_t ld_ys, const void** prepared, int* config) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  std::lock_guard<std::mutex> lk(g_nvfp4_registry_mu);
  for (const Nvfp4Registered& e : g_nvfp4_registry)
    if (e.device == dev && e.y_scales == y_scales && e.n == n && e.k == k && e.ld_ys == ld_ys) {
      *prepared = e.prepared;
      *config = e.config;
      return true;
    }
  return false;
}

int b200tile_nvfp4_register_weight_scales(const void* y_scales, int n, int k, int64_t ld_ys, int config,
                                          const void* prepared) {
  if (!y_scales || !prepared || n <= 0 || k <= 0 || config < 0 || config > 2)
    return set_error(B200TILE_ERR_INVALID, "nvfp4_register_weight_scales: bad argument");
  if ((reinterpret_cast<uintptr_t>(prepared) & 15) != 0)
    return set_error(B200TILE_ERR_ALIGN, "nvfp4_register_weight_scales: prepared buffer must be 16-byte aligned");
  int dev = -1;
  B200_CUDA_CHECK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_nvfp4_registry_mu);
  for (Nvfp4Registered& e : g_nvfp4_registry)
    if (e.device == dev && e.y_scales == y_scales) {
      e = Nvfp4Registered{dev, y_scales, n, k, ld_ys, prepared, config};
      return B200TILE_OK;
    }
  g_nvfp4_registry.push_back(Nvfp4Registered{dev, y_scales, n, k, ld_ys, prepared, config});
  return B200TILE_OK;
}

int b200tile_nvfp4_unregister_weight_scales(const void* y_scales) {
  int dev = -1;
  B200_CUDA_CHECK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_nvfp4_registry_mu);
  for (size_t i = 0; i < g_nvfp4_registry.size(); ++i)
    if (g_nvfp4_registry[i].device == dev && g_nvfp4_registry[i].y_scales == y_scales) {
      g_nvfp4_registry.erase(g_nvfp4_registry.begin() + (long)i);
      return B200TILE_OK;
    }
  return set_error(B200TILE_ERR_INVALID, "nvfp4_unregister_weight_scales: %p is not registered on this device", y_scales);
}

// ---------------------------------------------------------------------------
// Typed MXFP8 entry point
// ---------------------------------------------------------------------------
uint64_t b200tile_linear_mxfp8_workspace_bytes(int m, int n, int k) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  const size_t a = b200_mxfp8_scratch_bytes(m, n, k), b = b200_blockscaled_pair_scratch_bytes(0, m, n, k);
  return (uint64_t)(a > b ? a : b);
}

int b200tile_linear_mxfp8(const void* x, const void* y, const void* x_scales, const void* y_scales,
                          void* z, const char* out_dtype, int m, int n, int k, int64_t ldx, int64_t ldy,
                          int64_t ldz, int64_t ld_xs, int64_t ld_ys, float alpha, void* workspace,
                          uint64_t workspace_bytes, void* cu_stream) {
  if (!x || !y || !x_scales || !y_scales || !z || !out_dtype)
    return set_error(B200TILE_ERR_INVALID, "linear_mxfp8: null argument");
  if (m <= 0 || n <= 0 || k <= 0)
    return set_error(B200TILE_ERR_INVALID, "linear_mxfp8: Shape dimensions must be positive");
  if (k % 128 != 0)
    return set_error(B200TILE_ERR_INVALID, "linear_mxfp8: K (%d) must be a multiple of 128", k);
  if (ldx < k || ldy < k || ldz < n || ld_xs < k / 32 || ld_ys < k / 32)
    return set_error(B200TILE_ERR_INVALID, "linear_mxfp8: leading dimension too small");
  if (ld_xs % 4 != 0 || ld_ys % 4 != 0 || (reinterpret_cast<uintptr_t>(x_scales) & 3) != 0 ||
      (reinterpret_cast<uintptr_t>(y_scales) & 3) != 0)
    return set_error(B200TILE_ERR_ALIGN, "linear_mxfp8: scale rows must be 4-byte aligned");
  int out_f32;
  if (!strcmp(out_dtype, "f32")) out_f32 = 1;
  else if (!strcmp(out_dtype, "bf16")) out_f32 = 0;
  else return set_error(B200TILE_ERR_UNSUPPORTED, "linear_mxfp8: unsupported output type '%s'", out_dtype);
  if ((reinterpret_cast<uintptr_t>(z) & 15) != 0 || (ldz * (out_f32 ? 4 : 2)) % 16 != 0)
    return set_error(B200TILE_ERR_ALIGN, "linear_mxfp8: output must be 16-byte aligned with a 16-byte pitch");
  const bool pair = m >= kPairMinRows;   // CTA pairs with 256 x 256 tiles, else single CTAs with 224-row B tiles
  const size_t need = pair ? b200_blockscaled_pair_scratch_bytes(0, m, n, k) : b200_mxfp8_scratch_bytes(m, n, k);
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15) != 0 || workspace_bytes < need)
    return set_error(B200TILE_ERR_INVALID,
                     "linear_mxfp8: workspace of %llu bytes (16-byte aligned) required, got %llu",
                     (unsigned long long)need, (unsigned long long)workspace_bytes);
  if (pair)
    return b200_gemm_blockscaled_pair_dispatch(0, out_f32, x, y, x_scales, y_scales, z, m, n, k, ldx, ldy, ldz, ld_xs,
                                               ld_ys, alpha, workspace, static_cast<cudaStream_t>(cu_stream));
  return b200_gemm_mxfp8_dispatch(out_f32, x, y, x_scales, y_scales, z, m, n, k, ldx, ldy, ldz, ld_xs, ld_ys,
                                  alpha, workspace, static_cast<cudaStream_t>(cu_stream));
}

// ---------------------------------------------------------------------------
// Typed MXFP4 entry point: E2M1 operands (packed, as for NVFP4) with UE8M0 scales per 32 elements
// ---------------------------------------------------------------------------
uint64_t b200tile_linear_mxfp4_workspace_bytes(int m, int n, int k) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  const size_t a = b200_mxf4_scratch_bytes(m, n, k), b = b200_blockscaled_pair_scratch_bytes(2, m, n, k);
  return (uint64_t)(a > b ? a : b);
}

int b200tile_linear_mxfp4(const void* x, const void* y, const void* x_scales, const void* y_scales,
                          void* z, const char* out_dtype, int m, int n, int k, int64_t ldx, int64_t ldy,
                          int64_t ldz, int64_t ld_xs, int64_t ld_ys, float alpha, void* workspace,
                          uint64_t workspace_bytes, void* cu_stream) {
  if (!x || !y || !x_scales || !y_scales || !z || !out_dtype)
    return set_error(B200TILE_ERR_INVALID, "linear_mxfp4: null argument");
  if (m <= 0 || n <= 0 || k <= 0)
    return set_error(B200TILE_ERR_INVALID, "linear_mxfp4: Shape dimensions must be positive");
  if (k % 128 != 0)
    return set_error(B200TILE_ERR_INVALID, "linear_mxfp4: K (%d) must be a multiple of 128", k);
  if (ldx < k / 2 || ldy < k / 2 || ldz < n || ld_xs < k / 32 || ld_ys < k / 32)
    return set_error(B200TILE_ERR_INVALID, "linear_mxfp4: leading dimension too small");
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || (reinterpret_cast<uintptr_t>(y) & 15) != 0 || ldx % 16 != 0 ||
      ldy % 16 != 0)
    return set_error(B200TILE_ERR_ALIGN, "linear_mxfp4: operand rows must be 16-byte aligned");
  if (ld_xs % 4 != 0 || ld_ys % 4 != 0 || (reinterpret_cast<uintptr_t>(x_scales) & 3) != 0 ||
      (reinterpret_cast<uintptr_t>(y_scales) & 3) != 0)
    return set_error(B200TILE_ERR_ALIGN, "linear_mxfp4: scale rows must be 4-byte aligned");
  int out_f32;
  if (!strcmp(out_dtype, "f32")) out_f32 = 1;
  else if (!strcmp(out_dtype, "bf16")) out_f32 = 0;
  else return set_error(B200TILE_ERR_UNSUPPORTED, "linear_mxfp4: unsupported output type '%s'", out_dtype);
  if ((reinterpret_cast<uintptr_t>(z) & 15) != 0 || (ldz * (out_f32 ? 4 : 2)) % 16 != 0)
    return set_error(B200TILE_ERR_ALIGN, "linear_mxfp4: output must be 16-byte aligned with a 16-byte pitch");
  const bool pair = m >= kPairMinRows;   // CTA pairs with 256 x 256 tiles, else single CTAs with 192-row B tiles
  const size_t need = pair ? b200_blockscaled_pair_scratch_bytes(2, m, n, k) : b200_mxf4_scratch_bytes(m, n, k);
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15) != 0 || workspace_bytes < need)
    return set_error(B200TILE_ERR_INVALID,
                     "linear_mxfp4: workspace of %llu bytes (16-byte aligned) required, got %llu",
                     (unsigned long long)need, (unsigned long long)workspace_bytes);
  if (pair)
    return b200_gemm_blockscaled_pair_dispatch(2, out_f32, x, y, x_scales, y_scales, z, m, n, k, ldx, ldy, ldz, ld_xs,
                                               ld_ys, alpha, workspace, static_cast<cudaStream_t>(cu_stream));
  return b200_gemm_mxf4_dispatch(out_f32, x, y, x_scales, y_scales, z, m, n, k, ldx, ldy, ldz, ld_xs, ld_ys,
                                 alpha, workspace, static_cast<cudaStream_t>(cu_stream));
}

// ---------------------------------------------------------------------------
// Typed normalisation entry points
// ---------------------------------------------------------------------------
int b200tile_add_rms_norm(const char* dtype, const void* residual, const void* x, const void* w, void* out,
                          void* residual_out, int rows, int n, int64_t ld_residual, int64_t ldx, int64_t ldo,
                          int64_t ld_residual_out, float eps, void* cu_stream) {
  int dt;
  if (int rc = decode_dtype(dtype, "add_rms_norm", &dt)) return rc;
  if (!residual || !x || !w || !out || !residual_out)
    return set_error(B200TILE_ERR_INVALID, "add_rms_norm: null argument");
  if (rows <= 0 || n <= 0) return set_error(B200TILE_ERR_INVALID, "add_rms_norm: Shape dimensions must be positive");
  if (ld_residual < n || ldx < n || ldo < n || ld_residual_out < n)
    return set_error(B200TILE_ERR_INVALID, "add_rms_norm: row pitch smaller than the row");
  return b200_rms_norm_dispatch(dt, residual, x, w, out, residual_out, rows, n, ld_residual, ldx, ldo,
                                ld_residual_out, eps, static_cast<cudaStream_t>(cu_stream));
}

int b200tile_rms_norm(const char* dtype, const void* x, const void* w, void* out, int rows, int n, int64_t ldx,
                      int64_t ldo, float eps, void* cu_stream) {
  int dt;
  if (int rc = decode_dtype(dtype, "rms_norm", &dt)) return rc;
  if (!x || !w || !out) return set_error(B200TILE_ERR_INVALID, "rms_norm: null argument");
  if (rows <= 0 || n <= 0) return set_error(B200TILE_ERR_INVALID, "rms_norm: Shape dimensions must be positive");
  if (ldx < n || ldo < n) return set_error(B200TILE_ERR_INVALID, "rms_norm: row pitch smaller than the row");
  return b200_rms_norm_dispatch(dt, nullptr, x, w, out, nullptr, rows, n, 0, ldx, ldo, 0, eps,
                                static_cast<cudaStream_t>(cu_stream));
}

int b200tile_rope_seq(const char* dtype, const void* x, const float* inv_freq, void* out, int seq, int heads,
                      int head_dim, const int64_t x_strides[2], const int64_t out_strides[2], int position_start,
                      const void* position_ptr, void* cu_stream) {
  int dt;
  if (int rc = decode_dtype(dtype, "rope_seq", &dt)) return rc;
  if (!x || !inv_freq || !out || !x_strides || !out_strides)
    return set_error(B200TILE_ERR_INVALID, "rope_seq: null argument");
  if (seq <= 0 || heads <= 0 || head_dim <= 0)
    return set_error(B200TILE_ERR_INVALID, "rope_seq: Shape dimensions must be positive");
  if ((reinterpret_cast<uintptr_t>(inv_freq) & 3) || (reinterpret_cast<uintptr_t>(position_ptr) & 3))
    return set_error(B200TILE_ERR_ALIGN, "rope_seq: inv_freq / position must be 4-byte aligned");
  return b200_rope_seq_dispatch(dt, x, inv_freq, out, seq, heads, head_dim, x_strides[0], x_strides[1],
                                out_strides[0], out_strides[1], position_start,
                                static_cast<const uint32_t*>(position_ptr), static_cast<cudaStream_t>(cu_stream));
}

int b200tile_qk_norm_rope_kv(const char* dtype, const void* q, const void* k, const void* v, const void* q_weight,
                             const void* k_weight, const float* inv_freq, void* q_out, void* k_cache, void* v_cache,
                             float eps, int position_start, const void* position_ptr, int seq_len, int num_q_heads,
                             int num_kv_heads, int head_dim, int max_seq, int64_t q_seq_stride, int64_t k_seq_stride,
                             int64_t v_seq_stride, int64_t q_out_seq_stride, void* cu_stream) {
  int dt;
  if (int rc = decode_dtype(dtype, "qk_norm_rope_kv", &dt)) return rc;
  if (!q || !k || !v || !q_weight || !k_weight || !inv_freq || !q_out || !k_cache || !v_cache)
    return set_error(B200TILE_ERR_INVALID, "qk_norm_rope_kv: null argument");
  if (seq_len <= 0 || num_q_heads < 0 || num_kv_heads < 0 || num_q_heads + num_kv_heads <= 0 || head_dim <= 0 ||
      max_seq <= 0)
    return set_error(B200TILE_ERR_INVALID, "qk_norm_rope_kv: Shape dimensions must be positive");
  if (!position_ptr && (position_start < 0 || (int64_t)position_start + seq_len > max_seq))
    return set_error(B200TILE_ERR_INVALID, "qk_norm_rope_kv: positions [%d, %lld) do not fit the cache of %d rows",
                     position_start, (long long)position_start + seq_len, max_seq);
  if ((reinterpret_cast<uintptr_t>(inv_freq) & 3) || (reinterpret_cast<uintptr_t>(position_ptr) & 3))
    return set_error(B200TILE_ERR_ALIGN, "qk_norm_rope_kv: inv_freq / position must be 4-byte aligned");
  return b200_qk_norm_rope_kv_dispatch(dt, q, k, v, q_weight, k_weight, inv_freq, q_out, k_cache, v_cache, eps,
                                       position_start, static_cast<const uint32_t*>(position_ptr), seq_len,
                                       num_q_heads, num_kv_heads, head_dim, max_seq, q_seq_stride, k_seq_stride,
                                       v_seq_stride, q_out_seq_stride, static_cast<cudaStream_t>(cu_stream));
}

int b200tile_argmax_blocks(const char* dtype, const void* logits, float* block_max, uint32_t* block_idx, int len,
                           int block_size, void* cu_stream) {
  int dt;
  if (int rc = decode_dtype(dtype, "argmax_blocks", &dt)) return rc;
  if (!logits || !block_max || !block_idx) return set_error(B200TILE_ERR_INVALID, "argmax_blocks: null argument");
  if (len <= 0 || block_size <= 0)
    return set_error(B200TILE_ERR_INVALID, "argmax_blocks: Shape dimensions must be positive");
  return b200_argmax_blocks_dispatch(dt, logits, block_max, block_idx, len, block_size,
                                     static_cast<cudaStream_t>(cu_stream));
}

int b200tile_lm_head_argmax_blocks(const char* dtype, const void* weights, const void* hidden, float* block_max,
                                   uint32_t* block_idx, int vocab, int k, int64_t ldw, void* cu_stream) {
  int dt;
  if (int rc = decode_dtype(dtype, "lm_head_argmax_blocks", &dt)) return rc;
  if (!weights || !hidden || !block_max || !block_idx)
    return set_error(B200TILE_ERR_INVALID, "lm_head_argmax_blocks: null argument");
  if (vocab <= 0 || k <= 0)
    return set_error(B200TILE_ERR_INVALID, "lm_head_argmax_blocks: Shape dimensions must be positive");
  if (ldw < k) return set_error(B200TILE_ERR_INVALID, "lm_head_argmax_blocks: row pitch smaller than the row");
  return b200_lm_head_argmax_blocks_dispatch(dt, weights, hidden, block_max, block_idx, vocab, k, ldw,
                                             static_cast<cudaStream_t>(cu_stream));
}

int b200tile_argmax_reduce_blocks(const float* block_max, const uint32_t* block_idx, uint32_t* out, int num_blocks,
                                  void* cu_stream) {
  if (!block_max || !block_idx || !out) return set_error(B200TILE_ERR_INVALID, "argmax_reduce_blocks: null argument");
  if (num_blocks <= 0) return set_error(B200TILE_ERR_INVALID, "argmax_reduce_blocks: Shape dimensions must be positive");
  return b200_argmax_reduce_blocks_dispatch(block_max, block_idx, out, num_blocks,
                                            static_cast<cudaStream_t>(cu_stream));
}

static int pointwise_common(const char* who, int op, const char* dtype, void* out, const void* a, const void* b,
                            int rows, int cols, int64_t ld_out, int64_t ld_a, int64_t ld_b, void* cu_stream) {
  int dt;
  if (int rc = decode_dtype(dtype, who, &dt)) return rc;
  if (!out || !a || !b) return set_error(B200TILE_ERR_INVALID, "%s: null argument", who);
  if (rows <= 0 || cols <= 0) return set_error(B200TILE_ERR_INVALID, "%s: Shape dimensions must be positive", who);
  if (ld_out < cols || ld_a < cols || ld_b < cols)
    return set_error(B200TILE_ERR_INVALID, "%s: row pitch smaller than the row", who);
  return b200_pointwise_dispatch(dt, op, out, a, b, rows, cols, ld_out, ld_a, ld_b,
                                 static_cast<cudaStream_t>(cu_stream));
}

int b200tile_add_2d(const char* dtype, void* out, const void* lhs, const void* rhs, int rows, int cols, int64_t ld_out,
                    int64_t ld_lhs, int64_t ld_rhs, void* cu_stream) {
  return pointwise_common("add_2d", 0, dtype, out, lhs, rhs, rows, cols, ld_out, ld_lhs, ld_rhs, cu_stream);
}

int b200tile_silu_mul_2d(const char* dtype, void* out, const void* gate, const void* up, int rows, int cols,
                         int64_t ld_out, int64_t ld_gate, int64_t ld_up, void* cu_stream) {
  return pointwise_common("silu_mul_2d", 1, dtype, out, gate, up, rows, cols, ld_out, ld_gate, ld_up, cu_stream);
}

// ---------------------------------------------------------------------------
// Reference-shaped generic launch
// ---------------------------------------------------------------------------
namespace {

struct ParamReader {
  const void* const* p;
  int n, pos;
  bool ok;
  uint64_t u64() {
    if (pos >= n || !p[pos]) { ok = false; return 0; }
    return *static_cast<const uint64_t*>(p[pos++]);
  }
  int32_t i32() {
    if (pos >= n || !p[pos]) { ok = false; return 0; }
    return *static_cast<const int32_t*>(p[pos++]);
  }
  float f32() {
    if (pos >= n || !p[pos]) { ok = false; return 0; }
    return *static_cast<const float*>(p[pos++]);
  }
  // an f16 scalar parameter (two bytes), widened exactly
  float f16() {
    if (pos >= n || !p[pos]) { ok = false; return 0; }
    __half_raw raw;
    raw.x = *static_cast<const uint16_t*>(p[pos++]);
    return __half2float(__half(raw));
  }
};

struct TensorArg {
  uint64_t ptr;
  int rank;
  int32_t dim[4], stride[4], pdim[4], pstride[4];
};

void read_tensor(ParamReader& r, int rank, bool is_mut, TensorArg& t) {
  t.rank = rank;
  t.ptr = r.u64();
  for (int i = 0; i < rank; ++i) t.dim[i] = r.i32();
  for (int i = 0; i < rank; ++i) t.stride[i] = r.i32();
  if (is_mut) {
    for (int i = 0; i < rank; ++i) t.pdim[i] = r.i32();
    for (int i = 0; i < rank; ++i) t.pstride[i] = r.i32();
  }
}

bool parse_int(const char* s, long* out) {
  if (!s || !*s) return false;
  char* end = nullptr;
  long v = strtol(s, &end, 10);
  if (*end != '\0') return false;
  *out = v;
  return true;
}

// Maps (BM, BN, BK, CompileOptions) onto a precompiled GEMM configuration id.
int select_gemm_config(const char* dtype, long bm, long bn, long bk,
                       const b200tile_compile_options* opts, int* config) {
  const int cga = (opts && opts->num_cta_in_cga > 0) ? opts->num_cta_in_cga : 0;
  if (opts) {
    if (cga > 2)
      return set_error(B200TILE_ERR_UNSUPPORTED,
                       "gemm: num_cta_in_cga=%d has no precompiled configuration", cga);
    if (opts->occupancy > 1)
      return set_error(B200TILE_ERR_UNSUPPORTED,
                       "gemm: occupancy=%d has no precompiled configuration", opts->occupancy);
  }
  if (!strcmp(dtype, "f32")) {
    *config = 0;  // the exact-fp32 kernel produces identical results for every tile shape
    return B200TILE_OK;
  }
  if (bm == 256 && bn == 256 && bk == 64 && cga != 1) { *config = 2; return B200TILE_OK; }
  if (bm == 256 && bn == 512 && bk == 64 && cga != 1) { *config = 3; return B200TILE_OK; }
  if (bm == 128 && bn == 256 && bk == 64 && cga != 2) { *config = 0; return B200TILE_OK; }
  if (bm == 128 && bn == 128 && bk == 64 && cga != 2) { *config = 1; return B200TILE_OK; }
  return set_error(B200TILE_ERR_UNSUPPORTED,
                   "gemm(%s): tile (%ld,%ld,%ld) has no precompiled configuration", dtype, bm, bn,
                   bk);
}

int launch_gemm_generic(const char* kernel, const char* const* generics, int n_generics,
                        const b200tile_compile_options* opts, const void* const* params,
                        int n_params, const unsigned grid[3], void* stream, bool launch) {
  const bool batched = !strcmp(kernel, "batch_matmul");
  const bool persistent = !strcmp(kernel, "gemm_persistent");
  if (n_generics < 4)
    return set_error(B200TILE_ERR_UNSUPPORTED,
                     "%s: expected generics [T, BM, BN, BK, ...], got %d entries", kernel,
                     n_generics);
  const char* dtype = generics[0];
  long bm, bn, bk;
  if (!parse_int(generics[1], &bm) || !parse_int(generics[2], &bn) || !parse_int(generics[3], &bk))
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: tile-size generics must be integers", kernel);
  if (strcmp(dtype, "f32") && strcmp(dtype, "bf16") && strcmp(dtype, "f16"))
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: unsupported element type '%s'", kernel, dtype);
  int config = 0;
  if (int rc = select_gemm_config(dtype, bm, bn, bk, opts, &config)) return rc;
  if (!launch) return b200h::device_info() ? B200TILE_OK : B200TILE_ERR_CUDA;

  const int rank = batched ? 3 : 2;
  ParamReader r{params, n_params, 0, true};
  TensorArg z, x, y;
  read_tensor(r, rank, true, z);
  read_tensor(r, rank, false, x);
  read_tensor(r, rank, false, y);
  if (!r.ok)
    return set_error(B200TILE_ERR_INVALID, "%s: parameter array too short (%d values)", kernel,
                     n_params);
  const int o = batched ? 1 : 0;  // offset of the matrix axes
  const int M = z.dim[o], N = z.dim[o + 1], K = x.dim[o + 1];
  if (x.dim[o] != M || y.dim[o] != K || y.dim[o + 1] != N)
    return set_error(B200TILE_ERR_INVALID,
                     "%s: shapes do not compose: z[%d,%d] x[%d,%d] y[%d,%d]", kernel, M, N,
                     x.dim[o], x.dim[o + 1], y.dim[o], y.dim[o + 1]);
  if (z.stride[o + 1] != 1 || x.stride[o + 1] != 1 || y.stride[o + 1] != 1)
    return set_error(B200TILE_ERR_INVALID, "%s: the last axis of every tensor must be contiguous",
                     kernel);
  if (z.pdim[o] != bm || z.pdim[o + 1] != bn)
    return set_error(B200TILE_ERR_INVALID,
                     "%s: output partition (%d,%d) does not match the tile generics (%ld,%ld)",
                     kernel, z.pdim[o], z.pdim[o + 1], bm, bn);
  const unsigned tiles_m = (unsigned)((M + bm - 1) / bm), tiles_n = (unsigned)((N + bn - 1) / bn);
  int batch = 1;
  int num_programs = 0;
  if (batched) {
    batch = z.dim[0];
    if (x.dim[0] != batch || y.dim[0] != batch)
      return set_error(B200TILE_ERR_INVALID, "batch_matmul: batch extents differ");
    if (grid[0] != (unsigned)batch || grid[1] != tiles_m || grid[2] != tiles_n)
      return set_error(B200TILE_ERR_INVALID,
                       "launch grid (%u, %u, %u) does not match the inferred partition grid "
                       "(%d, %u, %u)",
                       grid[0], grid[1], grid[2], batch, tiles_m, tiles_n);
  } else if (persistent) {
    if (grid[0] == 0 || grid[1] != 1 || grid[2] != 1 || grid[0] > tiles_m * tiles_n)
      return set_error(B200TILE_ERR_INVALID,
                       "mapped partition num_tile_blocks cannot exceed the streamed logical tile "
                       "count. (grid (%u, %u, %u), tiles %u)",
                       grid[0], grid[1], grid[2], tiles_m * tiles_n);
    num_programs = (int)grid[0];
  } else {
    if (grid[0] != tiles_m || grid[1] != tiles_n || grid[2] != 1)
      return set_error(B200TILE_ERR_INVALID,
                       "launch grid (%u, %u, %u) does not match the inferred partition grid "
                       "(%u, %u, 1)",
                       grid[0], grid[1], grid[2], tiles_m, tiles_n);
  }
  // The paper and persistent kernels start each tile from zero (main.rs:85,121).  The example
  // `gemm` loads z as the initial accumulator (cutile-examples/examples/gemm.rs:28); a launcher
  // for that body binds the name "gemm_acc".
  const int accumulate = !strcmp(kernel, "gemm_acc") ? 1 : 0;
  long group_m = 8;
  if (persistent && n_generics >= 6) {
    long map_m;
    if (parse_int(generics[4], &map_m) && map_m > 0) group_m = map_m;
  }
  return b200tile_gemm(dtype, 0, reinterpret_cast<const void*>(x.ptr),
                       reinterpret_cast<const void*>(y.ptr), reinterpret_cast<void*>(z.ptr), batch,
                       M, N, K, x.stride[o], y.stride[o], z.stride[o], batched ? x.stride[0] : 0,
                       batched ? y.stride[0] : 0, batched ? z.stride[0] : 0, accumulate, config,
                       (int)group_m, num_programs, stream);
}

// Splits an optional leading element-type generic from the integer generics.
int split_generics(const char* const* generics, int n, const char* dflt, const char** dtype,
                   long* ints, int max_ints, int* n_ints) {
  int start = 0;
  *dtype = dflt;
  long tmp;
  if (n > 0 && generics[0] && !parse_int(generics[0], &tmp)) {
    *dtype = generics[0];
    start = 1;
  }
  *n_ints = 0;
  for (int i = start; i < n; ++i) {
    if (*n_ints >= max_ints || !parse_int(generics[i], &ints[*n_ints])) return 1;
    ++*n_ints;
  }
  return 0;
}

// "fmha": (out[b*h,m,d] partition [1,BM,D], q, k, v (b,h,m,d), qk_scale f32, input_pos i32,
//          query_group_size i32), generics [T?, BM, BN, D, H, CAUSAL, EVEN_K]
//          (cutile-examples/examples/flash_attention_causal.rs:19-45), grid (b*h, m/BM, 1).
// "fmha_prefill_causal": (q [q_len,heads,D], k, v [kv_heads,kv_len,D], out partition [BM,1,D],
//          qk_scale f32, query_group_size i32, kv_len i32, query_start i32),
//          generics [T?, BM, BN, D, CAUSAL, EVEN_K, LATENCY] (cutile-kernels/src/attention.rs:
//          242-262), grid (q_len/BM, heads, 1).
int launch_fmha_generic(const char* kernel, const char* const* generics, int n_generics,
                        const b200tile_compile_options* opts, const void* const* params,
                        int n_params, const unsigned grid[3], void* stream, bool launch) {
  const int cga = (opts && opts->num_cta_in_cga > 0) ? opts->num_cta_in_cga : 0;
  if (cga > 2)
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: num_cta_in_cga=%d has no precompiled configuration", kernel, cga);
  const bool prefill = !strcmp(kernel, "fmha_prefill_causal");
  const char* dtype;
  long g[8];
  int ng;
  if (split_generics(generics, n_generics, "f16", &dtype, g, 8, &ng) || ng < (prefill ? 4 : 5))
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: malformed generics", kernel);
  const long BM = g[0], BN = g[1], D = g[2];
  const long causal = prefill ? g[3] : g[4];
  const bool f32 = !strcmp(dtype, "f32");
  if (!f32 && strcmp(dtype, "bf16") && strcmp(dtype, "f16"))
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: unsupported element type '%s'", kernel, dtype);
  // f32 (CUDA cores): any tile generics, they only shape the launch grid; 16-bit types: the tensor-core tile
  if (f32 ? (BM <= 0 || BN <= 0 || (D != 32 && D != 64 && D != 128)) : (BM != 128 || BN != 128 || (D != 64 && D != 128)))
    return set_error(B200TILE_ERR_UNSUPPORTED,
                     "%s: tile (BM %ld, BN %ld, D %ld) has no precompiled configuration "
                     "(16-bit types: BM=BN=128, D in {64,128}; f32: D in {32,64,128})",
                     kernel, BM, BN, D);
  if (!launch) return b200h::device_info() ? B200TILE_OK : B200TILE_ERR_CUDA;
  ParamReader r{params, n_params, 0, true};
  TensorArg q, k, v, o;
  if (prefill) {
    read_tensor(r, 3, false, q);
    read_tensor(r, 3, false, k);
    read_tensor(r, 3, false, v);
    read_tensor(r, 3, true, o);
    const float scale = r.f32();
    const int group = r.i32();
    const int kv_len = r.i32();
    const int query_start = r.i32();
    if (!r.ok) return set_error(B200TILE_ERR_INVALID, "%s: parameter array too short", kernel);
    const int q_len = q.dim[0], heads = q.dim[1];
    const int heads_kv = k.dim[0];
    if (q.dim[2] != D || k.dim[2] != D || v.dim[2] != D || o.dim[2] != D || q.stride[2] != 1 ||
        k.stride[2] != 1 || v.stride[2] != 1 || o.stride[2] != 1)
      return set_error(B200TILE_ERR_INVALID, "%s: head dimension must equal D and be contiguous",
                       kernel);
    if (group <= 0 || heads != heads_kv * group || kv_len > k.dim[1] || kv_len <= 0)
      return set_error(B200TILE_ERR_INVALID, "%s: inconsistent heads / kv_len", kernel);
    if (o.pdim[0] != BM || o.pdim[1] != 1 || o.pdim[2] != D)
      return set_error(B200TILE_ERR_INVALID, "%s: output partition must be [BM, 1, D]", kernel);
    if (grid[0] != (unsigned)((q_len + BM - 1) / BM) || grid[1] != (unsigned)heads || grid[2] != 1)
      return set_error(B200TILE_ERR_INVALID,
                       "launch grid (%u, %u, %u) does not match the inferred partition grid "
                       "(%ld, %d, 1)",
                       grid[0], grid[1], grid[2], (long)((q_len + BM - 1) / BM), heads);
    const int64_t qs[2] = {q.stride[1], q.stride[0]}, ks[2] = {k.stride[0], k.stride[1]};
    const int64_t vs[2] = {v.stride[0], v.stride[1]}, os[2] = {o.stride[1], o.stride[0]};
    return fmha_fwd_common(dtype, reinterpret_cast<const void*>(q.ptr),
                           reinterpret_cast<const void*>(k.ptr),
                           reinterpret_cast<const void*>(v.ptr), reinterpret_cast<void*>(o.ptr),
                           1, heads, heads_kv, q_len, kv_len, (int)D, qs, ks, vs, os, scale,
                           causal != 0, query_start, nullptr, stream, cga);
  }
  read_tensor(r, 3, true, o);
  read_tensor(r, 4, false, q);
  read_tensor(r, 4, false, k);
  read_tensor(r, 4, false, v);
  const float scale = r.f32();
  const int input_pos = r.i32();
  const int group = r.i32();
  if (!r.ok) return set_error(B200TILE_ERR_INVALID, "%s: parameter array too short", kernel);
  const int b = q.dim[0], heads = q.dim[1], m = q.dim[2], heads_kv = k.dim[1], kv_len = k.dim[2];
  if (q.dim[3] != D || k.dim[3] != D || v.dim[3] != D || o.dim[2] != D || q.stride[3] != 1 ||
      k.stride[3] != 1 || v.stride[3] != 1 || o.stride[2] != 1)
    return set_error(B200TILE_ERR_INVALID, "%s: head dimension must equal D and be contiguous",
                     kernel);
  if (o.dim[0] != b * heads || o.dim[1] != m || k.dim[0] != b || v.dim[0] != b ||
      v.dim[1] != heads_kv || v.dim[2] != kv_len || group <= 0 || heads != heads_kv * group)
    return set_error(B200TILE_ERR_INVALID, "%s: tensor shapes do not compose", kernel);
  if (ng >= 4 && g[3] != heads)
    return set_error(B200TILE_ERR_INVALID, "%s: generic H=%ld but q has %d heads", kernel, g[3],
                     heads);
  // (batch, head) must collapse to one stride for every tensor
  if ((int64_t)q.stride[0] != (int64_t)q.stride[1] * heads ||
      (int64_t)k.stride[0] != (int64_t)k.stride[1] * heads_kv ||
      (int64_t)v.stride[0] != (int64_t)v.stride[1] * heads_kv)
    return set_error(B200TILE_ERR_INVALID,
                     "%s: batch and head axes must be laid out back to back", kernel);
  if (o.pdim[0] != 1 || o.pdim[1] != BM || o.pdim[2] != D)
    return set_error(B200TILE_ERR_INVALID, "%s: output partition must be [1, BM, D]", kernel);
  if (grid[0] != (unsigned)(b * heads) || grid[1] != (unsigned)((m + BM - 1) / BM) || grid[2] != 1)
    return set_error(B200TILE_ERR_INVALID,
                     "launch grid (%u, %u, %u) does not match the inferred partition grid "
                     "(%d, %ld, 1)",
                     grid[0], grid[1], grid[2], b * heads, (long)((m + BM - 1) / BM));
  const int64_t qs[2] = {q.stride[1], q.stride[2]}, ks[2] = {k.stride[1], k.stride[2]};
  const int64_t vs[2] = {v.stride[1], v.stride[2]}, os[2] = {o.stride[0], o.stride[1]};
  return fmha_fwd_common(dtype, reinterpret_cast<const void*>(q.ptr),
                         reinterpret_cast<const void*>(k.ptr),
                         reinterpret_cast<const void*>(v.ptr), reinterpret_cast<void*>(o.ptr), b,
                         heads, heads_kv, m, kv_len, (int)D, qs, ks, vs, os, scale, causal != 0,
                         input_pos, nullptr, stream, cga);
}

// "linear_tile_fp8_blk128": (z [M,N] partition [BM,BN], x [M,K], y [N,K], x_scales [M,K/128],
//   y_scales [N/128,K/128], alpha f32) -- the parameter list of the reference's scaled
//   `linear_tile` (cutile-examples/examples/mxfp8.rs:34-47); generics [T_out?, BM, BN, BK, ...].
int launch_linear_fp8_generic(const char* kernel, const char* const* generics, int n_generics,
                              const void* const* params, int n_params, const unsigned grid[3],
                              void* stream, bool launch) {
  const char* dtype;
  long g[8];
  int ng;
  if (split_generics(generics, n_generics, "bf16", &dtype, g, 8, &ng) || ng < 3)
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: malformed generics", kernel);
  if (g[0] != 128 || g[1] != 256 || g[2] != 128)
    return set_error(B200TILE_ERR_UNSUPPORTED,
                     "%s: tile (%ld,%ld,%ld) has no precompiled configuration (128,256,128)", kernel,
                     g[0], g[1], g[2]);
  if (!launch) return b200h::device_info() ? B200TILE_OK : B200TILE_ERR_CUDA;
  ParamReader r{params, n_params, 0, true};
  TensorArg z, x, y, xs, ys;
  read_tensor(r, 2, true, z);
  read_tensor(r, 2, false, x);
  read_tensor(r, 2, false, y);
  read_tensor(r, 2, false, xs);
  read_tensor(r, 2, false, ys);
  const float alpha = r.f32();
  if (!r.ok) return set_error(B200TILE_ERR_INVALID, "%s: parameter array too short", kernel);
  const int M = z.dim[0], N = z.dim[1], K = x.dim[1];
  if (x.dim[0] != M || y.dim[0] != N || y.dim[1] != K || xs.dim[0] != M || xs.dim[1] * 128 != K ||
      ys.dim[0] != (N + 127) / 128 || ys.dim[1] * 128 != K)
    return set_error(B200TILE_ERR_INVALID, "%s: tensor shapes do not compose", kernel);
  if (z.stride[1] != 1 || x.stride[1] != 1 || y.stride[1] != 1 || xs.stride[1] != 1 || ys.stride[1] != 1)
    return set_error(B200TILE_ERR_INVALID, "%s: the last axis of every tensor must be contiguous", kernel);
  if (z.pdim[0] != g[0] || z.pdim[1] != g[1])
    return set_error(B200TILE_ERR_INVALID, "%s: output partition does not match the tile generics", kernel);
  if (grid[0] != (unsigned)((M + g[0] - 1) / g[0]) || grid[1] != (unsigned)((N + g[1] - 1) / g[1]) || grid[2] != 1)
    return set_error(B200TILE_ERR_INVALID,
                     "launch grid (%u, %u, %u) does not match the inferred partition grid", grid[0],
                     grid[1], grid[2]);
  return b200tile_linear_fp8_blk128(reinterpret_cast<const void*>(x.ptr), reinterpret_cast<const void*>(y.ptr),
                                    reinterpret_cast<const float*>(xs.ptr), reinterpret_cast<const float*>(ys.ptr),
                                    reinterpret_cast<void*>(z.ptr), dtype, M, N, K, x.stride[0], y.stride[0],
                                    z.stride[0], xs.stride[0], ys.stride[0], alpha, stream);
}

// "linear_tile": the block-scaled linear kernels of the reference, which share one name and one parameter list
//   (z [M,N] f32 partition [BM,BN], x, y, x_scales, y_scales, alpha f32) and differ in the operand types:
//   NVFP4  (cutile-examples/examples/nvfp4.rs:37-76): x [M,K/2], y [N,K/2] f4e2m1fnx2, scales [.,K/16] f8e4m3fn,
//          generics [BM, BN, BK, BK_PACKED = BK/2, BK_SCALES = BK/16]
//   MXFP8  (cutile-examples/examples/mxfp8.rs:34-64): x [M,K], y [N,K] f8e4m3fn, scales [.,K/32] f8e8m0fnu,
//          generics [BM, BN, BK, BK_SCALES = BK/32]
//   MXFP4  (the operand / scale pairing of cutile/tests/tensor_and_matrix_ops.rs:224-244): NVFP4's operands with
//          [.,K/32] f8e8m0fnu scales, generics [BM, BN, BK, BK_PACKED = BK/2, BK_SCALES = BK/32]
//   The element types are not generics in the reference, so the formats are told apart by the generics themselves
//   (five integers with BK = 16 or 32 BK_SCALES, or four with BK = 32 BK_SCALES); an optional leading type name
//   selects a bf16 output instead of the reference's f32.  Any tile generics are accepted: they shape the
//   launch grid, which is validated, and the kernel runs its own tile.  The scale re-layout scratch is a
//   library-owned block per (device, stream).  Weight scales registered with
//   b200tile_nvfp4_register_weight_scales are used in their prepared form for decode-sized M.
int launch_linear_tile_generic(const char* kernel, const char* const* generics, int n_generics,
                               const void* const* params, int n_params, const unsigned grid[3], void* stream,
                               bool launch) {
  const char* dtype;
  long g[8];
  int ng;
  if (split_generics(generics, n_generics, "f32", &dtype, g, 8, &ng) || (ng != 4 && ng != 5))
    return set_error(B200TILE_ERR_UNSUPPORTED,
                     "%s: generics must be [BM, BN, BK, BK_PACKED, BK_SCALES] (NVFP4) or [BM, BN, BK, BK_SCALES] (MXFP8)",
                     kernel);
  const bool fp4 = ng == 5;
  const bool mxf4 = fp4 && g[4] * 32 == g[2];
  const long BM = g[0], BN = g[1], BK = g[2];
  if (BM <= 0 || BN <= 0 || BK <= 0)
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: tile generics must be positive", kernel);
  if (fp4 ? (g[3] * 2 != BK || (g[4] * 16 != BK && !mxf4)) : (g[3] * 32 != BK))
    return set_error(B200TILE_ERR_UNSUPPORTED,
                     "%s: generics do not describe a supported block-scaled format (NVFP4: BK_PACKED = BK/2 and "
                     "BK_SCALES = BK/16, or BK/32 for UE8M0 scales; MXFP8: BK_SCALES = BK/32)", kernel);
  if (strcmp(dtype, "f32") && strcmp(dtype, "bf16"))
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: unsupported output type '%s'", kernel, dtype);
  if (!launch) return b200h::device_info() ? B200TILE_OK : B200TILE_ERR_CUDA;
  ParamReader r{params, n_params, 0, true};
  TensorArg z, x, y, xs, ys;
  read_tensor(r, 2, true, z);
  read_tensor(r, 2, false, x);
  read_tensor(r, 2, false, y);
  read_tensor(r, 2, false, xs);
  read_tensor(r, 2, false, ys);
  const float alpha = r.f32();
  if (!r.ok) return set_error(B200TILE_ERR_INVALID, "%s: parameter array too short", kernel);
  const int M = z.dim[0], N = z.dim[1];
  const int K = fp4 ? x.dim[1] * 2 : x.dim[1];
  const int V = (fp4 && !mxf4) ? 16 : 32;
  if (x.dim[0] != M || y.dim[0] != N || y.dim[1] != x.dim[1] || xs.dim[0] != M || ys.dim[0] != N ||
      xs.dim[1] * V != K || ys.dim[1] * V != K)
    return set_error(B200TILE_ERR_INVALID, "%s: tensor shapes do not compose", kernel);
  if (z.stride[1] != 1 || x.stride[1] != 1 || y.stride[1] != 1 || xs.stride[1] != 1 || ys.stride[1] != 1)
    return set_error(B200TILE_ERR_INVALID, "%s: the last axis of every tensor must be contiguous", kernel);
  if (z.pdim[0] != BM || z.pdim[1] != BN)
    return set_error(B200TILE_ERR_INVALID, "%s: output partition does not match the tile generics", kernel);
  if (grid[0] != (unsigned)((M + BM - 1) / BM) || grid[1] != (unsigned)((N + BN - 1) / BN) || grid[2] != 1)
    return set_error(B200TILE_ERR_INVALID,
                     "launch grid (%u, %u, %u) does not match the inferred partition grid", grid[0],
                     grid[1], grid[2]);
  const void* xp = reinterpret_cast<const void*>(x.ptr);
  const void* yp = reinterpret_cast<const void*>(y.ptr);
  const void* xsp = reinterpret_cast<const void*>(xs.ptr);
  const void* ysp = reinterpret_cast<const void*>(ys.ptr);
  void* zp = reinterpret_cast<void*>(z.ptr);
  if (mxf4) {
    const uint64_t need = b200tile_linear_mxfp4_workspace_bytes(M, N, K);
    void* ws = b200h::stream_scratch(static_cast<cudaStream_t>(stream), need, kernel);
    if (!ws) return B200TILE_ERR_INVALID;
    return b200tile_linear_mxfp4(xp, yp, xsp, ysp, zp, dtype, M, N, K, x.stride[0], y.stride[0], z.stride[0],
                                 xs.stride[0], ys.stride[0], alpha, ws, need, stream);
  }
  if (fp4 && M <= 128) {
    const void* prepared = nullptr;
    int config = 0;
    if (nvfp4_registry_find(ysp, N, K, ys.stride[0], &prepared, &config))
      return b200tile_linear_nvfp4_prepared(xp, yp, xsp, prepared, zp, dtype, M, N, K, x.stride[0], y.stride[0],
                                            z.stride[0], xs.stride[0], alpha, config, stream);
  }
  const uint64_t need = fp4 ? b200tile_linear_nvfp4_workspace_bytes(M, N, K) : b200tile_linear_mxfp8_workspace_bytes(M, N, K);
  void* ws = b200h::stream_scratch(static_cast<cudaStream_t>(stream), need, kernel);
  if (!ws) return B200TILE_ERR_INVALID;
  if (fp4)
    return b200tile_linear_nvfp4(xp, yp, xsp, ysp, zp, dtype, M, N, K, x.stride[0], y.stride[0], z.stride[0],
                                 xs.stride[0], ys.stride[0], alpha, ws, need, -1, stream);
  return b200tile_linear_mxfp8(xp, yp, xsp, ysp, zp, dtype, M, N, K, x.stride[0], y.stride[0], z.stride[0],
                               xs.stride[0], ys.stride[0], alpha, ws, need, stream);
}

// Serving attention kernels of cutile-kernels/src/attention.rs in their own parameter order.
// "fmha_prefill_gqa" (:398-582): (q [q_len,q_heads,D], k, v [kv_heads,kv_len,D], out partition
//    [BM,GROUP,D], qk_scale f32, query_group_size i32, kv_len i32, query_start i32), generics
//    [T?, BM, BN, D, GROUP, M_EFF, CAUSAL, EVEN_K, LATENCY], grid (q_len/BM, q_heads/GROUP, 1).
// "fmha_causal" (:588-721): (q [m,h,D], k, v [hkv,n,D], out partition [BM,1,D], qk_scale f16,
//    query_group_size i32, position_start u32[1]), generics [T?, BM, BN, D, CAUSAL, EVEN_K],
//    grid (m/BM, h, 1).
int launch_fmha_serving_generic(const char* kernel, const char* const* generics, int n_generics,
                                const void* const* params, int n_params, const unsigned grid[3],
                                void* stream, bool launch) {
  const bool gqa = !strcmp(kernel, "fmha_prefill_gqa");
  const char* dtype;
  long g[9];
  int ng;
  if (split_generics(generics, n_generics, "f16", &dtype, g, 9, &ng) || ng < (gqa ? 6 : 4))
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: malformed generics", kernel);
  const long BM = g[0], BN = g[1], D = g[2];
  const long GROUP = gqa ? g[3] : 1;
  const long causal = gqa ? g[5] : g[3];
  if (strcmp(dtype, "bf16") && strcmp(dtype, "f16"))
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: unsupported element type '%s'", kernel, dtype);
  if (BM <= 0 || BN <= 0 || GROUP <= 0 || (D != 64 && D != 128))
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: D=%ld has no precompiled configuration (64, 128)",
                     kernel, D);
  if (gqa && g[4] != BM * GROUP)
    return set_error(B200TILE_ERR_INVALID, "%s: M_EFF=%ld must equal BM*GROUP=%ld", kernel, g[4],
                     BM * GROUP);
  if (!launch) return b200h::device_info() ? B200TILE_OK : B200TILE_ERR_CUDA;
  ParamReader r{params, n_params, 0, true};
  TensorArg q, k, v, o, pos;
  read_tensor(r, 3, false, q);
  read_tensor(r, 3, false, k);
  read_tensor(r, 3, false, v);
  read_tensor(r, 3, true, o);
  const float scale = gqa ? r.f32() : r.f16();
  const int group = r.i32();
  int kv_len = 0, query_start = 0;
  if (gqa) {
    kv_len = r.i32();
    query_start = r.i32();
  } else {
    read_tensor(r, 1, false, pos);
    kv_len = k.dim[1];
  }
  if (!r.ok) return set_error(B200TILE_ERR_INVALID, "%s: parameter array too short", kernel);
  const int q_len = q.dim[0], heads = q.dim[1], heads_kv = k.dim[0];
  if (q.dim[2] != D || k.dim[2] != D || v.dim[2] != D || o.dim[2] != D || q.stride[2] != 1 ||
      k.stride[2] != 1 || v.stride[2] != 1 || o.stride[2] != 1)
    return set_error(B200TILE_ERR_INVALID, "%s: head dimension must equal D and be contiguous", kernel);
  if (group <= 0 || heads != heads_kv * group || kv_len > k.dim[1] || kv_len <= 0 || group % GROUP)
    return set_error(B200TILE_ERR_INVALID, "%s: inconsistent heads / GROUP / kv_len", kernel);
  if (o.pdim[0] != BM || o.pdim[1] != GROUP || o.pdim[2] != D)
    return set_error(B200TILE_ERR_INVALID, "%s: output partition must be [BM, %ld, D]", kernel, GROUP);
  if (grid[0] != (unsigned)((q_len + BM - 1) / BM) || grid[1] != (unsigned)(heads / GROUP) || grid[2] != 1)
    return set_error(B200TILE_ERR_INVALID,
                     "launch grid (%u, %u, %u) does not match the inferred partition grid (%ld, %ld, 1)",
                     grid[0], grid[1], grid[2], (long)((q_len + BM - 1) / BM), (long)(heads / GROUP));
  const int64_t qs[2] = {q.stride[1], q.stride[0]}, ks[2] = {k.stride[0], k.stride[1]};
  const int64_t vs[2] = {v.stride[0], v.stride[1]}, os[2] = {o.stride[1], o.stride[0]};
  if (gqa)
    return b200tile_fmha_fwd(dtype, reinterpret_cast<const void*>(q.ptr), reinterpret_cast<const void*>(k.ptr),
                             reinterpret_cast<const void*>(v.ptr), reinterpret_cast<void*>(o.ptr), 1, heads,
                             heads_kv, q_len, kv_len, (int)D, qs, ks, vs, os, scale, causal != 0, query_start,
                             stream);
  if (pos.dim[0] < 1) return set_error(B200TILE_ERR_INVALID, "%s: position_start must hold one u32", kernel);
  return b200tile_fmha_fwd_dynpos(dtype, reinterpret_cast<const void*>(q.ptr), reinterpret_cast<const void*>(k.ptr),
                                  reinterpret_cast<const void*>(v.ptr), reinterpret_cast<void*>(o.ptr), 1, heads,
                                  heads_kv, q_len, kv_len, (int)D, qs, ks, vs, os, scale, causal != 0,
                                  reinterpret_cast<const void*>(pos.ptr), stream);
}

// "rms_norm_f16" (cutile-kernels/src/norms.rs:22-27): (x [rows,N], w [N], out partition [1,N], eps f32);
// "add_rms_norm_f16" (:77-84): (residual [rows,N], x [rows,N], w [N], out partition [1,N], residual_out
// partition [1,N], eps f32).  Generics [T?, N, BLOCK_SIZE]; grid (rows, 1, 1).  BLOCK_SIZE only shapes the
// reference's loop and is ignored here.
int launch_norm_generic(const char* kernel, const char* const* generics, int n_generics, const void* const* params,
                        int n_params, const unsigned grid[3], void* stream, bool launch) {
  const bool add = !strcmp(kernel, "add_rms_norm_f16");
  const char* dtype;
  long g[4];
  int ng;
  if (split_generics(generics, n_generics, "f16", &dtype, g, 4, &ng) || ng < 2)
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: malformed generics", kernel);
  if (strcmp(dtype, "bf16") && strcmp(dtype, "f16"))
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: unsupported element type '%s'", kernel, dtype);
  const long N = g[0];
  if (N <= 0 || g[1] <= 0) return set_error(B200TILE_ERR_INVALID, "%s: N and BLOCK_SIZE must be positive", kernel);
  if (!launch) return b200h::device_info() ? B200TILE_OK : B200TILE_ERR_CUDA;
  ParamReader r{params, n_params, 0, true};
  TensorArg res, x, w, o, ro;
  if (add) read_tensor(r, 2, false, res);
  read_tensor(r, 2, false, x);
  read_tensor(r, 1, false, w);
  read_tensor(r, 2, true, o);
  if (add) read_tensor(r, 2, true, ro);
  const float eps = r.f32();
  if (!r.ok) return set_error(B200TILE_ERR_INVALID, "%s: parameter array too short", kernel);
  const int rows = o.dim[0];
  if (x.dim[0] != rows || x.dim[1] != N || o.dim[1] != N || w.dim[0] != N || x.stride[1] != 1 ||
      o.stride[1] != 1 || w.stride[0] != 1 ||
      (add && (res.dim[0] != rows || res.dim[1] != N || ro.dim[0] != rows || ro.dim[1] != N ||
               res.stride[1] != 1 || ro.stride[1] != 1)))
    return set_error(B200TILE_ERR_INVALID, "%s: tensor shapes do not compose", kernel);
  if (o.pdim[0] != 1 || o.pdim[1] != N || (add && (ro.pdim[0] != 1 || ro.pdim[1] != N)))
    return set_error(B200TILE_ERR_INVALID, "%s: output partition must be [1, N]", kernel);
  if (grid[0] != (unsigned)rows || grid[1] != 1 || grid[2] != 1)
    return set_error(B200TILE_ERR_INVALID,
                     "launch grid (%u, %u, %u) does not match the inferred partition grid (%d, 1, 1)", grid[0],
                     grid[1], grid[2], rows);
  if (add)
    return b200tile_add_rms_norm(dtype, reinterpret_cast<const void*>(res.ptr), reinterpret_cast<const void*>(x.ptr),
                                 reinterpret_cast<const void*>(w.ptr), reinterpret_cast<void*>(o.ptr),
                                 reinterpret_cast<void*>(ro.ptr), rows, (int)N, res.stride[0], x.stride[0],
                                 o.stride[0], ro.stride[0], eps, stream);
  return b200tile_rms_norm(dtype, reinterpret_cast<const void*>(x.ptr), reinterpret_cast<const void*>(w.ptr),
                           reinterpret_cast<void*>(o.ptr), rows, (int)N, x.stride[0], o.stride[0], eps, stream);
}

// "rope_seq_f16" (cutile-kernels/src/positional.rs:20-25): (x [seq,heads,D], inv_freq f32 [HALF_D], out partition
// [1,1,HALF_D], position_start i32); "rope_seq_dynpos_f16" (:74-79): (x, inv_freq, position_start u32[1], out).
// Generics [T?, D, HALF_D]; grid (seq, heads, 2).
int launch_rope_generic(const char* kernel, const char* const* generics, int n_generics, const void* const* params,
                        int n_params, const unsigned grid[3], void* stream, bool launch) {
  const bool dyn = !strcmp(kernel, "rope_seq_dynpos_f16");
  const char* dtype;
  long g[4];
  int ng;
  if (split_generics(generics, n_generics, "f16", &dtype, g, 4, &ng) || ng < 2)
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: malformed generics", kernel);
  if (strcmp(dtype, "bf16") && strcmp(dtype, "f16"))
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: unsupported element type '%s'", kernel, dtype);
  const long D = g[0], HALF = g[1];
  if (D <= 0 || HALF * 2 != D) return set_error(B200TILE_ERR_INVALID, "%s: HALF_D must be D / 2", kernel);
  if (!launch) return b200h::device_info() ? B200TILE_OK : B200TILE_ERR_CUDA;
  ParamReader r{params, n_params, 0, true};
  TensorArg x, f, pos, o;
  int position_start = 0;
  read_tensor(r, 3, false, x);
  read_tensor(r, 1, false, f);
  if (dyn) read_tensor(r, 1, false, pos);
  read_tensor(r, 3, true, o);
  if (!dyn) position_start = r.i32();
  if (!r.ok) return set_error(B200TILE_ERR_INVALID, "%s: parameter array too short", kernel);
  const int seq = x.dim[0], heads = x.dim[1];
  if (x.dim[2] != D || o.dim[0] != seq || o.dim[1] != heads || o.dim[2] != D || f.dim[0] != HALF ||
      x.stride[2] != 1 || o.stride[2] != 1 || f.stride[0] != 1 || (dyn && pos.dim[0] < 1))
    return set_error(B200TILE_ERR_INVALID, "%s: tensor shapes do not compose", kernel);
  if (o.pdim[0] != 1 || o.pdim[1] != 1 || o.pdim[2] != HALF)
    return set_error(B200TILE_ERR_INVALID, "%s: output partition must be [1, 1, HALF_D]", kernel);
  if (grid[0] != (unsigned)seq || grid[1] != (unsigned)heads || grid[2] != 2)
    return set_error(B200TILE_ERR_INVALID,
                     "launch grid (%u, %u, %u) does not match the inferred partition grid (%d, %d, 2)", grid[0],
                     grid[1], grid[2], seq, heads);
  const int64_t xs[2] = {x.stride[0], x.stride[1]}, os[2] = {o.stride[0], o.stride[1]};
  return b200tile_rope_seq(dtype, reinterpret_cast<const void*>(x.ptr), reinterpret_cast<const float*>(f.ptr),
                           reinterpret_cast<void*>(o.ptr), seq, heads, (int)D, xs, os, position_start,
                           dyn ? reinterpret_cast<const void*>(pos.ptr) : nullptr, stream);
}

// "qk_norm_rope_kv_prefill_raw_f16" (experimental/fused_transformer.rs:22-43): nine raw pointers (q, k, v,
// q_weight, k_weight, inv_freq, q_out, k_cache, v_cache), eps f32, position_start, seq_len, num_q_heads,
// num_kv_heads i32; "qk_norm_rope_kv_decode_raw_f16" (:356-372): seven raw pointers (qkv, q_weight, k_weight,
// inv_freq, q_out, k_cache, v_cache), position_start u32[1], eps f32, num_q_heads, num_kv_heads i32.
// Generics [T?, D, HALF_D, MAX_SEQ]; grid (seq_len, num_q_heads + num_kv_heads, 1).
int launch_qk_rope_generic(const char* kernel, const char* const* generics, int n_generics,
                           const void* const* params, int n_params, const unsigned grid[3], void* stream,
                           bool launch) {
  const bool decode = !strcmp(kernel, "qk_norm_rope_kv_decode_raw_f16");
  const char* dtype;
  long g[4];
  int ng;
  if (split_generics(generics, n_generics, "f16", &dtype, g, 4, &ng) || ng < 3)
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: malformed generics", kernel);
  if (strcmp(dtype, "bf16") && strcmp(dtype, "f16"))
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: unsupported element type '%s'", kernel, dtype);
  const long D = g[0], MAXS = g[2];
  if (D <= 0 || g[1] * 2 != D || MAXS <= 0)
    return set_error(B200TILE_ERR_INVALID, "%s: HALF_D must be D / 2 and MAX_SEQ positive", kernel);
  if (!launch) return b200h::device_info() ? B200TILE_OK : B200TILE_ERR_CUDA;
  ParamReader r{params, n_params, 0, true};
  uint64_t ptr[9];
  TensorArg pos;
  float eps;
  int position_start = 0, seq_len = 1, qh, kvh;
  if (decode) {
    for (int i = 0; i < 7; ++i) ptr[i] = r.u64();
    read_tensor(r, 1, false, pos);
    eps = r.f32();
  } else {
    for (int i = 0; i < 9; ++i) ptr[i] = r.u64();
    eps = r.f32();
    position_start = r.i32();
    seq_len = r.i32();
  }
  qh = r.i32();
  kvh = r.i32();
  if (!r.ok) return set_error(B200TILE_ERR_INVALID, "%s: parameter array too short", kernel);
  if (qh < 0 || kvh < 0 || seq_len <= 0)
    return set_error(B200TILE_ERR_INVALID, "%s: Shape dimensions must be positive", kernel);
  if (grid[0] != (unsigned)seq_len || grid[1] != (unsigned)(qh + kvh) || grid[2] != 1)
    return set_error(B200TILE_ERR_INVALID,
                     "launch grid (%u, %u, %u) does not match the inferred partition grid (%d, %d, 1)", grid[0],
                     grid[1], grid[2], seq_len, qh + kvh);
  auto vp = [](uint64_t a) { return reinterpret_cast<void*>(a); };
  if (decode) {
    // one fused projection row: q heads, then k heads, then v heads
    const char* qkv = reinterpret_cast<const char*>(ptr[0]);
    const int64_t row = (int64_t)(qh + 2 * kvh) * D;
    return b200tile_qk_norm_rope_kv(dtype, qkv, qkv + (int64_t)qh * D * 2, qkv + (int64_t)(qh + kvh) * D * 2,
                                    vp(ptr[1]), vp(ptr[2]), reinterpret_cast<const float*>(ptr[3]), vp(ptr[4]),
                                    vp(ptr[5]), vp(ptr[6]), eps, 0, reinterpret_cast<const void*>(pos.ptr), 1, qh, kvh,
                                    (int)D, (int)MAXS, row, row, row, (int64_t)qh * D, stream);
  }
  return b200tile_qk_norm_rope_kv(dtype, vp(ptr[0]), vp(ptr[1]), vp(ptr[2]), vp(ptr[3]), vp(ptr[4]),
                                  reinterpret_cast<const float*>(ptr[5]), vp(ptr[6]), vp(ptr[7]), vp(ptr[8]), eps,
                                  position_start, nullptr, seq_len, qh, kvh, (int)D, (int)MAXS, (int64_t)qh * D,
                                  (int64_t)kvh * D, (int64_t)kvh * D, (int64_t)qh * D, stream);
}

// "argmax_blocks_f16" (cutile-kernels/src/argmax.rs:20-25): (logits [len], block_max partition [1], block_idx
//    partition [1], len i32), generics [T?, BLOCK_SIZE], grid (blocks, 1, 1).
// "lm_head_argmax_blocks_f16" (:88-94): (weights [vocab, K], hidden [1, K], block_max partition [1], block_idx
//    partition [1], vocab_size i32), generics [T?, K], grid (ceil(vocab / 64), 1, 1).
// "argmax_reduce_blocks_to_u32" (:162-167): (block_max [n], block_idx [n], out partition [1], num_blocks i32),
//    generics [BLOCK_SIZE], grid (1, 1, 1).
int launch_argmax_generic(const char* kernel, const char* const* generics, int n_generics, const void* const* params,
                          int n_params, const unsigned grid[3], void* stream, bool launch) {
  const bool fused = !strcmp(kernel, "lm_head_argmax_blocks_f16");
  const bool reduce = !strcmp(kernel, "argmax_reduce_blocks_to_u32");
  const char* dtype;
  long g[2];
  int ng;
  if (split_generics(generics, n_generics, "f16", &dtype, g, 2, &ng) || ng < 1 || g[0] <= 0)
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: malformed generics", kernel);
  if (strcmp(dtype, "bf16") && strcmp(dtype, "f16"))
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: unsupported element type '%s'", kernel, dtype);
  if (!launch) return b200h::device_info() ? B200TILE_OK : B200TILE_ERR_CUDA;
  ParamReader r{params, n_params, 0, true};
  TensorArg a, b, bm, bi;
  read_tensor(r, fused ? 2 : 1, false, a);
  if (fused) read_tensor(r, 2, false, b);
  if (reduce) read_tensor(r, 1, false, b);
  read_tensor(r, 1, true, bm);
  if (!reduce) read_tensor(r, 1, true, bi);
  const int count = r.i32();
  if (!r.ok) return set_error(B200TILE_ERR_INVALID, "%s: parameter array too short", kernel);
  if (bm.pdim[0] != 1 || bm.stride[0] != 1 || (!reduce && (bi.pdim[0] != 1 || bi.stride[0] != 1)))
    return set_error(B200TILE_ERR_INVALID, "%s: outputs must be contiguous with partition [1]", kernel);
  if (reduce) {
    if (count > a.dim[0] || count > b.dim[0] || a.stride[0] != 1 || b.stride[0] != 1 || count > g[0])
      return set_error(B200TILE_ERR_INVALID, "%s: num_blocks exceeds the inputs or BLOCK_SIZE", kernel);
    if (grid[0] != 1 || grid[1] != 1 || grid[2] != 1)
      return set_error(B200TILE_ERR_INVALID, "launch grid (%u, %u, %u) does not match the inferred partition grid (1, 1, 1)",
                       grid[0], grid[1], grid[2]);
    return b200tile_argmax_reduce_blocks(reinterpret_cast<const float*>(a.ptr), reinterpret_cast<const uint32_t*>(b.ptr),
                                         reinterpret_cast<uint32_t*>(bm.ptr), count, stream);
  }
  const long per_block = fused ? 64 : g[0];
  const long blocks = (count + per_block - 1) / per_block;
  if (bm.dim[0] < blocks || bi.dim[0] < blocks)
    return set_error(B200TILE_ERR_INVALID, "%s: block_max / block_idx hold fewer than %ld entries", kernel, blocks);
  if (grid[0] != (unsigned)blocks || grid[1] != 1 || grid[2] != 1)
    return set_error(B200TILE_ERR_INVALID,
                     "launch grid (%u, %u, %u) does not match the inferred partition grid (%ld, 1, 1)", grid[0],
                     grid[1], grid[2], blocks);
  if (fused) {
    if (a.dim[1] != g[0] || b.dim[1] != g[0] || a.stride[1] != 1 || b.stride[1] != 1 || count > a.dim[0])
      return set_error(B200TILE_ERR_INVALID, "%s: tensor shapes do not compose", kernel);
    return b200tile_lm_head_argmax_blocks(dtype, reinterpret_cast<const void*>(a.ptr),
                                          reinterpret_cast<const void*>(b.ptr), reinterpret_cast<float*>(bm.ptr),
                                          reinterpret_cast<uint32_t*>(bi.ptr), count, (int)g[0], a.stride[0], stream);
  }
  if (a.stride[0] != 1 || count > a.dim[0])
    return set_error(B200TILE_ERR_INVALID, "%s: tensor shapes do not compose", kernel);
  return b200tile_argmax_blocks(dtype, reinterpret_cast<const void*>(a.ptr), reinterpret_cast<float*>(bm.ptr),
                                reinterpret_cast<uint32_t*>(bi.ptr), count, (int)g[0], stream);
}

// "add_2d_f16" / "silu_mul_2d_f16" (cutile-kernels/src/pointwise.rs:20-24, 50-54): (out partition [1, BLOCK_SIZE],
// lhs [rows, cols], rhs [rows, cols]), generics [T?, BLOCK_SIZE], grid (rows, ceil(cols / BLOCK_SIZE), 1).
int launch_pointwise_generic(const char* kernel, const char* const* generics, int n_generics,
                             const void* const* params, int n_params, const unsigned grid[3], void* stream,
                             bool launch) {
  const bool silu = !strcmp(kernel, "silu_mul_2d_f16");
  const char* dtype;
  long g[2];
  int ng;
  if (split_generics(generics, n_generics, "f16", &dtype, g, 2, &ng) || ng < 1 || g[0] <= 0)
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: malformed generics", kernel);
  if (strcmp(dtype, "bf16") && strcmp(dtype, "f16"))
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: unsupported element type '%s'", kernel, dtype);
  if (!launch) return b200h::device_info() ? B200TILE_OK : B200TILE_ERR_CUDA;
  ParamReader r{params, n_params, 0, true};
  TensorArg o, a, b;
  read_tensor(r, 2, true, o);
  read_tensor(r, 2, false, a);
  read_tensor(r, 2, false, b);
  if (!r.ok) return set_error(B200TILE_ERR_INVALID, "%s: parameter array too short", kernel);
  const int rows = o.dim[0], cols = o.dim[1];
  if (a.dim[0] != rows || a.dim[1] != cols || b.dim[0] != rows || b.dim[1] != cols || o.stride[1] != 1 ||
      a.stride[1] != 1 || b.stride[1] != 1)
    return set_error(B200TILE_ERR_INVALID, "%s: tensor shapes do not compose", kernel);
  if (o.pdim[0] != 1 || o.pdim[1] != g[0])
    return set_error(B200TILE_ERR_INVALID, "%s: output partition must be [1, BLOCK_SIZE]", kernel);
  const long cb = (cols + g[0] - 1) / g[0];
  if (grid[0] != (unsigned)rows || grid[1] != (unsigned)cb || grid[2] != 1)
    return set_error(B200TILE_ERR_INVALID,
                     "launch grid (%u, %u, %u) does not match the inferred partition grid (%d, %ld, 1)", grid[0],
                     grid[1], grid[2], rows, cb);
  return pointwise_common(silu ? "silu_mul_2d" : "add_2d", silu ? 1 : 0, dtype, reinterpret_cast<void*>(o.ptr),
                          reinterpret_cast<const void*>(a.ptr), reinterpret_cast<const void*>(b.ptr), rows, cols,
                          o.stride[0], a.stride[0], b.stride[0], stream);
}

// "fmha_decode_gqa_split" (:727-901): (q [kv_heads,GROUP,D], k, v [kv_heads,cap,D], att_out partition
//    [1,GROUP,D] of [kv_heads,NUM_KV_SPLITS*GROUP,D], lse_out partition [1,GROUP] of
//    [kv_heads,NUM_KV_SPLITS*GROUP], qk_scale f16, position_start u32[1]), generics
//    [T?, GROUP, BN, D, NUM_KV_SPLITS, LATENCY], grid (kv_heads, NUM_KV_SPLITS, 1).
// "splitk_reduce_merge" (:907-1015): (att_partial [kv_heads,NS_GROUP,D], lse_partial [kv_heads,NS_GROUP],
//    out partition [1,GROUP,CHUNK_D]), generics [T?, GROUP, D, CHUNK_D, NUM_KV_SPLITS, NS_GROUP, LATENCY],
//    grid (kv_heads, 1, D/CHUNK_D).
int launch_decode_generic(const char* kernel, const char* const* generics, int n_generics,
                          const void* const* params, int n_params, const unsigned grid[3], void* stream,
                          bool launch) {
  const bool merge = !strcmp(kernel, "splitk_reduce_merge");
  const char* dtype;
  long g[8];
  int ng;
  if (split_generics(generics, n_generics, "f16", &dtype, g, 8, &ng) || ng < (merge ? 5 : 4))
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: malformed generics", kernel);
  if (strcmp(dtype, "bf16") && strcmp(dtype, "f16"))
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: unsupported element type '%s'", kernel, dtype);
  const long GROUP = g[0];
  const long D = merge ? g[1] : g[2];
  const long NS = g[3];
  if (D != 64 && D != 128)
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: D=%ld has no precompiled configuration (64, 128)",
                     kernel, D);
  if (GROUP <= 0 || GROUP > 16 || NS <= 0)
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: GROUP must be 1..16 and NUM_KV_SPLITS positive", kernel);
  if (merge && (g[4] != NS * GROUP || g[2] <= 0 || D % g[2]))
    return set_error(B200TILE_ERR_INVALID, "%s: NS_GROUP must equal NUM_KV_SPLITS*GROUP and CHUNK_D divide D",
                     kernel);
  if (!launch) return b200h::device_info() ? B200TILE_OK : B200TILE_ERR_CUDA;
  ParamReader r{params, n_params, 0, true};
  if (merge) {
    TensorArg att, lse, o;
    read_tensor(r, 3, false, att);
    read_tensor(r, 2, false, lse);
    read_tensor(r, 3, true, o);
    if (!r.ok) return set_error(B200TILE_ERR_INVALID, "%s: parameter array too short", kernel);
    const int heads = o.dim[0];
    if (att.dim[0] != heads || att.dim[1] != NS * GROUP || att.dim[2] != D || lse.dim[0] != heads ||
        lse.dim[1] != NS * GROUP || o.dim[1] != GROUP || o.dim[2] != D || att.stride[2] != 1 ||
        lse.stride[1] != 1 || o.stride[2] != 1)
      return set_error(B200TILE_ERR_INVALID, "%s: tensor shapes do not compose", kernel);
    if (o.pdim[0] != 1 || o.pdim[1] != GROUP || o.pdim[2] != g[2])
      return set_error(B200TILE_ERR_INVALID, "%s: output partition must be [1, GROUP, CHUNK_D]", kernel);
    if (grid[0] != (unsigned)heads || grid[1] != 1 || grid[2] != (unsigned)(D / g[2]))
      return set_error(B200TILE_ERR_INVALID,
                       "launch grid (%u, %u, %u) does not match the inferred partition grid (%d, 1, %ld)",
                       grid[0], grid[1], grid[2], heads, (long)(D / g[2]));
    const int64_t as[2] = {att.stride[0], att.stride[1]}, os[2] = {o.stride[0], o.stride[1]};
    return b200tile_splitk_reduce_merge(dtype, reinterpret_cast<const void*>(att.ptr),
                                        reinterpret_cast<const float*>(lse.ptr), reinterpret_cast<void*>(o.ptr),
                                        heads, (int)GROUP, (int)D, (int)NS, as, lse.stride[0], os, stream);
  }
  TensorArg q, k, v, att, lse, pos;
  read_tensor(r, 3, false, q);
  read_tensor(r, 3, false, k);
  read_tensor(r, 3, false, v);
  read_tensor(r, 3, true, att);
  read_tensor(r, 2, true, lse);
  const float scale = r.f16();
  read_tensor(r, 1, false, pos);
  if (!r.ok) return set_error(B200TILE_ERR_INVALID, "%s: parameter array too short", kernel);
  const int heads = q.dim[0];
  if (q.dim[1] != GROUP || q.dim[2] != D || k.dim[0] != heads || v.dim[0] != heads || k.dim[2] != D ||
      v.dim[2] != D || v.dim[1] != k.dim[1] || att.dim[0] != heads || att.dim[1] != NS * GROUP ||
      att.dim[2] != D || lse.dim[0] != heads || lse.dim[1] != NS * GROUP || pos.dim[0] < 1)
    return set_error(B200TILE_ERR_INVALID, "%s: tensor shapes do not compose", kernel);
  if (q.stride[2] != 1 || k.stride[2] != 1 || v.stride[2] != 1 || att.stride[2] != 1 || lse.stride[1] != 1)
    return set_error(B200TILE_ERR_INVALID, "%s: the last axis of every tensor must be contiguous", kernel);
  if (att.pdim[0] != 1 || att.pdim[1] != GROUP || att.pdim[2] != D || lse.pdim[0] != 1 || lse.pdim[1] != GROUP)
    return set_error(B200TILE_ERR_INVALID, "%s: output partitions must be [1, GROUP, D] and [1, GROUP]", kernel);
  if (grid[0] != (unsigned)heads || grid[1] != (unsigned)NS || grid[2] != 1)
    return set_error(B200TILE_ERR_INVALID,
                     "launch grid (%u, %u, %u) does not match the inferred partition grid (%d, %ld, 1)",
                     grid[0], grid[1], grid[2], heads, NS);
  const int64_t qs[2] = {q.stride[0], q.stride[1]}, ks[2] = {k.stride[0], k.stride[1]};
  const int64_t vs[2] = {v.stride[0], v.stride[1]}, as[2] = {att.stride[0], att.stride[1]};
  return b200tile_fmha_decode_gqa_split(dtype, reinterpret_cast<const void*>(q.ptr),
                                        reinterpret_cast<const void*>(k.ptr), reinterpret_cast<const void*>(v.ptr),
                                        reinterpret_cast<void*>(att.ptr), reinterpret_cast<float*>(lse.ptr),
                                        nullptr, reinterpret_cast<const void*>(pos.ptr), heads, (int)GROUP, (int)D,
                                        k.dim[1], (int)g[1], (int)NS, scale, qs, ks, vs, as, lse.stride[0], nullptr,
                                        stream);
}

// "group_gemm_f16_nt_desc" (cutile-kernels/src/experimental/moe.rs:66-85): (a_ptrs, b_ptrs, c_ptrs i64[G],
//    a_metas, b_metas, c_metas i32[G,8], num_groups i32), generics [T?, BM, BN, BK, NUM_SM], grid (NUM_SM,1,1).
int launch_group_gemm_generic(const char* kernel, const char* const* generics, int n_generics,
                              const void* const* params, int n_params, void* stream, bool launch) {
  const char* dtype;
  long g[8];
  int ng;
  if (split_generics(generics, n_generics, "f16", &dtype, g, 8, &ng) || ng < 3)
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: malformed generics", kernel);
  if (g[0] != 128 || (g[1] != 128 && g[1] != 256) || g[2] != 64)
    return set_error(B200TILE_ERR_UNSUPPORTED,
                     "%s: tile (%ld,%ld,%ld) has no precompiled configuration ((128,128,64), (128,256,64))", kernel,
                     g[0], g[1], g[2]);
  if (strcmp(dtype, "bf16") && strcmp(dtype, "f16"))
    return set_error(B200TILE_ERR_UNSUPPORTED, "%s: unsupported element type '%s'", kernel, dtype);
  if (!launch) return b200h::device_info() ? B200TILE_OK : B200TILE_ERR_CUDA;
  ParamReader r{params, n_params, 0, true};
  TensorArg ap, bp, cp, am, bmeta, cm;
  read_tensor(r, 1, false, ap);
  read_tensor(r, 1, false, bp);
  read_tensor(r, 1, false, cp);
  read_tensor(r, 2, false, am);
  read_tensor(r, 2, false, bmeta);
  read_tensor(r, 2, false, cm);
  const int groups = r.i32();
  if (!r.ok) return set_error(B200TILE_ERR_INVALID, "%s: parameter array too short", kernel);
  if (groups < 0 || ap.dim[0] < groups || bp.dim[0] < groups || cp.dim[0] < groups || am.dim[0] < groups ||
      bmeta.dim[0] < groups || cm.dim[0] < groups || am.dim[1] != 8 || bmeta.dim[1] != 8 || cm.dim[1] != 8)
    return set_error(B200TILE_ERR_INVALID, "%s: tables must hold num_groups entries ([G] pointers, [G,8] extents)",
                     kernel);
  if (ap.stride[0] != 1 || bp.stride[0] != 1 || cp.stride[0] != 1 || am.stride[0] != 8 || am.stride[1] != 1 ||
      bmeta.stride[0] != 8 || bmeta.stride[1] != 1 || cm.stride[0] != 8 || cm.stride[1] != 1)
    return set_error(B200TILE_ERR_INVALID, "%s: tables must be dense", kernel);
  return b200tile_group_gemm(dtype, reinterpret_cast<const int64_t*>(ap.ptr), reinterpret_cast<const int64_t*>(bp.ptr),
                             reinterpret_cast<const int64_t*>(cp.ptr), reinterpret_cast<const int32_t*>(am.ptr),
                             reinterpret_cast<const int32_t*>(bmeta.ptr), reinterpret_cast<const int32_t*>(cm.ptr),
                             groups, (int)g[1], nullptr, 0, stream);
}

}  // namespace

int b200tile_launch(const char* kernel, const char* const* generics, int n_generics,
                    const b200tile_compile_options* opts, const void* const* params, int n_params,
                    const unsigned grid[3], void* cu_stream) {
  if (!kernel) return set_error(B200TILE_ERR_INVALID, "launch: kernel name is null");
  if (!params || !grid) return set_error(B200TILE_ERR_INVALID, "launch: null params or grid");
  if (is_gemm_name(kernel))
    return launch_gemm_generic(kernel, generics, n_generics, opts, params, n_params, grid,
                               cu_stream, true);
  if (!strcmp(kernel, "fmha") || !strcmp(kernel, "fmha_prefill_causal"))
    return launch_fmha_generic(kernel, generics, n_generics, opts, params, n_params, grid,
                               cu_stream, true);
  if (!strcmp(kernel, "linear_tile_fp8_blk128"))
    return launch_linear_fp8_generic(kernel, generics, n_generics, params, n_params, grid, cu_stream, true);
  if (!strcmp(kernel, "linear_tile"))
    return launch_linear_tile_generic(kernel, generics, n_generics, params, n_params, grid, cu_stream, true);
  if (!strcmp(kernel, "fmha_prefill_gqa") || !strcmp(kernel, "fmha_causal"))
    return launch_fmha_serving_generic(kernel, generics, n_generics, params, n_params, grid, cu_stream, true);
  if (!strcmp(kernel, "fmha_decode_gqa_split") || !strcmp(kernel, "splitk_reduce_merge"))
    return launch_decode_generic(kernel, generics, n_generics, params, n_params, grid, cu_stream, true);
  if (!strcmp(kernel, "group_gemm_f16_nt_desc"))
    return launch_group_gemm_generic(kernel, generics, n_generics, params, n_params, cu_stream, true);
  if (!strcmp(kernel, "rms_norm_f16") || !strcmp(kernel, "add_rms_norm_f16"))
    return launch_norm_generic(kernel, generics, n_generics, params, n_params, grid, cu_stream, true);
  if (!strcmp(kernel, "rope_seq_f16") || !strcmp(kernel, "rope_seq_dynpos_f16"))
    return launch_rope_generic(kernel, generics, n_generics, params, n_params, grid, cu_stream, true);
  if (!strcmp(kernel, "qk_norm_rope_kv_prefill_raw_f16") || !strcmp(kernel, "qk_norm_rope_kv_decode_raw_f16"))
    return launch_qk_rope_generic(kernel, generics, n_generics, params, n_params, grid, cu_stream, true);
  if (!strcmp(kernel, "argmax_blocks_f16") || !strcmp(kernel, "lm_head_argmax_blocks_f16") ||
      !strcmp(kernel, "argmax_reduce_blocks_to_u32"))
    return launch_argmax_generic(kernel, generics, n_generics, params, n_params, grid, cu_stream, true);
  if (!strcmp(kernel, "add_2d_f16") || !strcmp(kernel, "silu_mul_2d_f16"))
    return launch_pointwise_generic(kernel, generics, n_generics, params, n_params, grid, cu_stream, true);
  return set_error(B200TILE_ERR_UNSUPPORTED, "launch: unknown kernel '%s'", kernel);
}

int b200tile_prepare(const char* kernel, const char* const* generics, int n_generics,
                     const b200tile_compile_options* opts) {
  if (!kernel) return set_error(B200TILE_ERR_INVALID, "prepare: kernel name is null");
  if (is_gemm_name(kernel))
    return launch_gemm_generic(kernel, generics, n_generics, opts, nullptr, 0, nullptr, nullptr,
                               false);
  if (!strcmp(kernel, "fmha") || !strcmp(kernel, "fmha_prefill_causal"))
    return launch_fmha_generic(kernel, generics, n_generics, opts, nullptr, 0, nullptr, nullptr,
                               false);
  if (!strcmp(kernel, "linear_tile_fp8_blk128"))
    return launch_linear_fp8_generic(kernel, generics, n_generics, nullptr, 0, nullptr, nullptr, false);
  if (!strcmp(kernel, "linear_tile"))
    return launch_linear_tile_generic(kernel, generics, n_generics, nullptr, 0, nullptr, nullptr, false);
  if (!strcmp(kernel, "fmha_prefill_gqa") || !strcmp(kernel, "fmha_causal"))
    return launch_fmha_serving_generic(kernel, generics, n_generics, nullptr, 0, nullptr, nullptr, false);
  if (!strcmp(kernel, "fmha_decode_gqa_split") || !strcmp(kernel, "splitk_reduce_merge"))
    return launch_decode_generic(kernel, generics, n_generics, nullptr, 0, nullptr, nullptr, false);
  if (!strcmp(kernel, "group_gemm_f16_nt_desc"))
    return launch_group_gemm_generic(kernel, generics, n_generics, nullptr, 0, nullptr, false);
  if (!strcmp(kernel, "rms_norm_f16") || !strcmp(kernel, "add_rms_norm_f16"))
    return launch_norm_generic(kernel, generics, n_generics, nullptr, 0, nullptr, nullptr, false);
  if (!strcmp(kernel, "rope_seq_f16") || !strcmp(kernel, "rope_seq_dynpos_f16"))
    return launch_rope_generic(kernel, generics, n_generics, nullptr, 0, nullptr, nullptr, false);
  if (!strcmp(kernel, "qk_norm_rope_kv_prefill_raw_f16") || !strcmp(kernel, "qk_norm_rope_kv_decode_raw_f16"))
    return launch_qk_rope_generic(kernel, generics, n_generics, nullptr, 0, nullptr, nullptr, false);
  if (!strcmp(kernel, "argmax_blocks_f16") || !strcmp(kernel, "lm_head_argmax_blocks_f16") ||
      !strcmp(kernel, "argmax_reduce_blocks_to_u32"))
    return launch_argmax_generic(kernel, generics, n_generics, nullptr, 0, nullptr, nullptr, false);
  if (!strcmp(kernel, "add_2d_f16") || !strcmp(kernel, "silu_mul_2d_f16"))
    return launch_pointwise_generic(kernel, generics, n_generics, nullptr, 0, nullptr, nullptr, false);
  return set_error(B200TILE_ERR_UNSUPPORTED, "prepare: unknown kernel '%s'", kernel);
}

#ifdef B200TILE_TRACE
// Diagnostic builds only: copies the cycle counters of one traced kernel ("gemm_pair", "fmha",
// "fmha_alt", "fmha_alt_t", "block_scaled", "block_scaled_pair") into out[20]
// ("block_scaled_pair_timeline": out[40]); see csrc/trace.cuh.
B200TILE_API int b200tile_trace_read(const char* which, long long* out) {
  if (!which || !out) return B200TILE_ERR_INVALID;
  for (int i = 0; i < 20; ++i) out[i] = 0;
  if (!strcmp(which, "gemm_pair")) return b200_trace_read_gemm_pair(out) ? B200TILE_ERR_CUDA : B200TILE_OK;
  if (!strcmp(which, "fmha")) return b200_trace_read_fmha(out) ? B200TILE_ERR_CUDA : B200TILE_OK;
  if (!strcmp(which, "fmha_alt_t")) return b200_trace_read_fmha_alt_t(out) ? B200TILE_ERR_CUDA : B200TILE_OK;
  if (!strcmp(which, "fmha_alt")) return b200_trace_read_fmha_alt(out) ? B200TILE_ERR_CUDA : B200TILE_OK;
  if (!strcmp(which, "block_scaled")) return b200_trace_read_fp4(out) ? B200TILE_ERR_CUDA : B200TILE_OK;
  if (!strcmp(which, "block_scaled_pair")) return b200_trace_read_fp4_pair(out) ? B200TILE_ERR_CUDA : B200TILE_OK;
  if (!strcmp(which, "grouped")) return b200_trace_read_grouped(out) ? B200TILE_ERR_CUDA : B200TILE_OK;
  if (!strcmp(which, "block_scaled_pair_timeline"))
    return b200_trace_read_fp4_pair_tl(out) ? B200TILE_ERR_CUDA : B200TILE_OK;
  return B200TILE_ERR_UNSUPPORTED;
}
#endif

#ifdef B200TILE_TEST_HOOKS
// Test builds only: arms / disarms the producer hook of gemm_tc.cu that leaves one stage unloaded.
B200TILE_API int b200tile_test_set_skip_stage(int on) {
  return b200_test_set_skip_stage(on) ? B200TILE_ERR_CUDA : B200TILE_OK;
}
#endif

}  // extern "C"
