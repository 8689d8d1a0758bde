/* b200tile -- C ABI of the sm_100a dense-contraction kernels.
 *
 * This is the boundary a cuTile-Rust launcher binds instead of JIT-compiling the kernel body
 * and calling cuLaunchKernel itself.  Every entry point takes plain pointers and sizes, never
 * allocates or synchronises inside a launch call (so launches may be recorded into a CUDA graph,
 * the contract of `GraphNode`, cuda-async/src/cuda_graph.rs:303-324), borrows device memory only
 * for the duration of the stream-ordered work, returns 0 on success and a small positive code
 * otherwise, and never throws or aborts.  All functions may be called from many threads.
 *
 * The library contains machine code for sm_100a only; there is no CPU or other-GPU fallback.
 */
#ifndef B200TILE_H_
#define B200TILE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200TILE_ABI_VERSION 1

#if defined(__GNUC__)
#define B200TILE_API __attribute__((visibility("default")))
#else
#define B200TILE_API
#endif

/* Return codes. */
#define B200TILE_OK 0
#define B200TILE_ERR_INVALID 1     /* argument violates a kernel precondition            */
#define B200TILE_ERR_UNSUPPORTED 2 /* unknown kernel / generics / config combination     */
#define B200TILE_ERR_CUDA 3        /* a CUDA call failed                                 */
#define B200TILE_ERR_DEVICE 4      /* the device status record holds an error            */
#define B200TILE_ERR_ALIGN 5       /* pointer or pitch violates TMA's 16-byte rules      */

/* Mirrors `CompileOptions` (cutile-compiler/src/hints.rs:94-126).  A field of -1 means
 * "not set".  The options select among the fixed, precompiled kernel configurations. */
typedef struct b200tile_compile_options {
  int occupancy;
  int num_cta_in_cga;
  int max_divisibility;
  int num_worker_warps_per_cta;
} b200tile_compile_options;

/* One precompiled configuration, as enumerated for the autotuner (replaces the open-ended
 * tile-size generics of the JIT, cutile/src/tune.rs:53-121). */
typedef struct b200tile_config {
  int id;
  int bm, bn, bk;
  int stages;
  int num_cta_in_cga;
  int occupancy;
} b200tile_config;

/* Device status record written by bounded waits inside the kernels. */
typedef struct b200tile_status_t {
  uint32_t code;  /* 0 = ok, 1 = a wait gave up, 3 = a grouped-GEMM group broke the 16-byte rule and was skipped */
  uint32_t block; /* blockIdx.x of the CTA that recorded it */
  uint32_t site;  /* which wait (code 1); index of the offending group (code 3) */
  uint32_t aux;
} b200tile_status_t;

/* ---- library management ------------------------------------------------------------------ */

/* Replaces nothing in the reference; lets a binding check it was built against this header. */
B200TILE_API int b200tile_abi_version(void);

/* Binds the device's primary context to the calling thread and resolves per-device state
 * (SM count, status record).  Counterpart of `Device::new` + `bind_to_thread`
 * (cuda-core/src/runtime.rs:126-140,229-237).  Call once per device before capturing graphs. */
B200TILE_API int b200tile_init(int device_ordinal);

/* Text of the last error on the calling thread.  Counterpart of the `Display` text of
 * `Error::KernelLaunch` / `DeviceError` (cutile/src/error.rs:42-55). */
B200TILE_API const char* b200tile_last_error(void);

/* Number of SMs of the current device; what `persistent_num_programs` needs
 * (cutile-benchmarks/paper/sec5_exp1_safety_overhead/rust/gemm/src/main.rs:796-811). */
B200TILE_API int b200tile_num_sms(void);

/* Reads (synchronising `stream`) or clears the device status record. */
B200TILE_API int b200tile_status(void* cu_stream, b200tile_status_t* out);
B200TILE_API int b200tile_status_reset(void* cu_stream);

/* Lists the precompiled configurations of `kernel` for element type `dtype`; returns how many
 * exist (may exceed `cap`).  Feeds `Autotuner::configs` (cutile/src/tune.rs:312-410). */
B200TILE_API int b200tile_query_configs(const char* kernel, const char* dtype, b200tile_config* out, int cap);

/* ---- reference-shaped generic launch ----------------------------------------------------- */

/* Drop-in for the two calls the macro-generated launcher makes per launch: `jit_compile` and
 * `AsyncKernelLaunch::execute` (cutile-macro/src/kernel_launcher_generator.rs:911-923,958-975;
 * cuda-async/src/launch.rs:91-113).
 *   kernel    entry name without the `_entry` suffix: "gemm", "gemm_acc", "gemm_persistent",
 *             "batch_matmul", "fmha", "fmha_prefill_causal", "linear_tile_fp8_blk128"
 *   generics  the launcher's `Vec<String>` (dtype names from cuda-core/src/dtype.rs:147-168,
 *             integers in decimal)
 *   params    the reference's flattened kernel parameter array, one pointer per value, in
 *             signature order: per `&Tensor`: ptr(u64), dims(i32...), strides(i32...); per
 *             `&mut Tensor`: the same plus partition dims and partition strides
 *             (cutile-compiler/src/kernel_entry_generator.rs:176-201; cutile/src/tensor.rs:
 *             1723-1739,2006-2016); scalars by value
 *   grid      the launcher's inferred grid; validated against the output partition
 * An unsupported combination returns B200TILE_ERR_UNSUPPORTED (the autotuner turns that into
 * `TrialState::Invalid`, cutile/src/tune.rs:503-514). */
B200TILE_API int b200tile_launch(const char* kernel, const char* const* generics, int n_generics,
                    const b200tile_compile_options* opts, const void* const* params, int n_params,
                    const unsigned grid[3], void* cu_stream);

/* Warm-up without launching: the `.compile()` path (cutile-macro/src/_module.rs:852-866).
 * Sets function attributes so the first real launch has no lazy cost. */
B200TILE_API int b200tile_prepare(const char* kernel, const char* const* generics, int n_generics,
                     const b200tile_compile_options* opts);

/* ---- typed entry points (what b200tile_launch forwards to) ------------------------------- */

/* C[b] (+)= A[b] * B[b], row-major, leading dimensions and batch strides in ELEMENTS.
 * Replaces the kernels `gemm` (cutile-examples/examples/gemm.rs:20-36, cutile-benchmarks/
 * benches/gemm.rs:20-41), `gemm_persistent` (cutile-benchmarks/paper/sec5_exp1_safety_overhead/
 * rust/gemm/src/main.rs:98-132) and `batch_matmul` (cutile-examples/examples/batch_matmul.rs:
 * 17-43).
 *   dtype       "f32" (exact fp32, bit-identical to the reference's cpu_gemm), "bf16", "f16"
 *               (tensor cores, fp32 accumulation, output rounded to the input type)
 *   b_layout    0: B is [K,N] (reference GEMM), 1: B is [N,K] (reference linear_tile, "NT")
 *   accumulate  0: C = A*B, 1: C = C + A*B (the `load_tile_mut` form; f32 only)
 *   config      id from b200tile_query_configs, or -1 for the default.  Accumulation is fp32 except for
 *               id 4 (f16 only): f16 accumulators, the arithmetic of the reference's benchmark kernel,
 *               whose `mma(x, y, z)` accumulates in a Tile<T> (cutile-benchmarks/benches/gemm.rs:20-41);
 *               never chosen by default
 *   group_size_m  grouped-M tile order (main.rs:53-66); <=0 selects 8
 *   num_programs  persistent grid size; <=0 selects min(SMs, tiles) */
B200TILE_API int b200tile_gemm(const char* dtype, int b_layout, const void* a, const void* b, void* c,
                  int batch, int m, int n, int k, int64_t lda, int64_t ldb, int64_t ldc,
                  int64_t stride_a, int64_t stride_b, int64_t stride_c, int accumulate, int config,
                  int group_size_m, int num_programs, void* cu_stream);

/* C = A*B with all three operands in HOST memory (page-locked for full speed), as one pipeline:
 * B is uploaded first, A follows in slabs of `slab_rows` rows (<= 0 selects 1024; rounded up to a
 * multiple of 256), every slab is multiplied by b200tile_gemm as soon as it has arrived and its
 * rows of C are downloaded while the next slab is still on its way.  Replaces the reference
 * user's serial sequence `copy_host_vec_to_device` x2 (cutile/src/api.rs:422) -> kernel launch ->
 * `copy_device_to_host_vec` (api.rs:371).
 *   a_host [m,k], b_host ([k,n] for b_layout 0, [n,k] for 1), c_host [m,n]: dense row-major
 *   a_dev, b_dev, c_dev: device staging buffers of the same sizes, provided by the caller
 * Ordered after everything already queued on `cu_stream`; when the call returns, the work is
 * queued and `cu_stream` ends after the last download, so synchronising it completes the call.
 * Two internal streams and their events are created on first use per device; not usable inside
 * a stream capture (B200TILE_ERR_UNSUPPORTED). */
B200TILE_API int b200tile_gemm_host(const char* dtype, int b_layout, const void* a_host, const void* b_host,
                                    void* c_host, void* a_dev, void* b_dev, void* c_dev, int m, int n, int k,
                                    int slab_rows, void* cu_stream);

/* out[m, inter] = silu(x . w[0:inter]^T) * (x . w[inter:2*inter]^T): the gate/up projection of a
 * SwiGLU feed-forward block with the pointwise step in the GEMM epilogue.  Replaces the sequence
 * "NT linear layer into [m, 2*inter], then `silu_mul_2d_f16`" (cutile-kernels/src/pointwise.rs:
 * 50-77); gate and up are rounded to the 16-bit type before the pointwise step, as that sequence
 * does, so the result differs from it only by the exp implementation.
 *   dtype      "bf16" or "f16"
 *   x          [m, k], row pitch ldx;  w_gate_up [2*inter, k] (gate rows first), row pitch ldw
 *   out        [m, inter], row pitch ldo.  Pitches in elements, multiples of 8; pointers 16-byte aligned. */
B200TILE_API int b200tile_linear_swiglu(const char* dtype, const void* x, const void* w_gate_up, void* out, int m,
                                        int inter, int k, int64_t ldx, int64_t ldw, int64_t ldo, void* cu_stream);

/* RMSNorm over the last dimension of a [rows, n] 16-bit tensor:
 *     out = round16((x * rsqrt(mean(x^2) + eps)) * w)
 * Replaces `rms_norm_f16` (cutile-kernels/src/norms.rs:22-60; also its per-head use `qk_norm_f16`,
 * :152 ff., when the heads are passed as rows).  Each row is read once (the reference reads it twice).
 *   dtype   "f16" (the reference's type) or "bf16";  w [n];  pitches ldx / ldo in elements.
 *   16-byte aligned bases with pitches that are multiples of 8 take the vector path; anything else
 *   is accepted and runs with scalar accesses. */
B200TILE_API int b200tile_rms_norm(const char* dtype, const void* x, const void* w, void* out, int rows, int n,
                                   int64_t ldx, int64_t ldo, float eps, void* cu_stream);

/* Residual add fused with RMSNorm, also writing the updated residual:
 *     combined = residual + x (fp32);  residual_out = round16(combined);
 *     out = round16((combined * rsqrt(mean(combined^2) + eps)) * w)
 * Replaces `add_rms_norm_f16` (cutile-kernels/src/norms.rs:77-137).  `residual_out` may alias
 * `residual`, and `out` may alias `x` (every element is read before its row is written). */
B200TILE_API int b200tile_add_rms_norm(const char* dtype, const void* residual, const void* x, const void* w,
                                       void* out, void* residual_out, int rows, int n, int64_t ld_residual,
                                       int64_t ldx, int64_t ldo, int64_t ld_residual_out, float eps,
                                       void* cu_stream);

/* Rotary position embedding, chunked (GPT-NeoX) layout, over x [seq, heads, head_dim]:
 *     theta = float(position + s) * inv_freq[i],  i in [0, head_dim/2)
 *     out[s,h,i] = x[s,h,i] cos - x[s,h,i+D/2] sin;   out[s,h,i+D/2] = x[s,h,i+D/2] cos + x[s,h,i] sin
 * Replaces `rope_seq_f16` and, with a non-null `position_ptr` (device u32[1], read by the kernel, so
 * that a captured graph can be replayed with a new position), `rope_seq_dynpos_f16`
 * (cutile-kernels/src/positional.rs:20-62, 74-120).  The angles are evaluated once per position, not
 * once per (position, head, half).
 *   dtype "f16" or "bf16"; inv_freq [head_dim/2] f32; strides {seq, head} in elements (innermost 1);
 *   `out` may alias `x`. */
B200TILE_API int b200tile_rope_seq(const char* dtype, const void* x, const float* inv_freq, void* out, int seq,
                                   int heads, int head_dim, const int64_t x_strides[2],
                                   const int64_t out_strides[2], int position_start, const void* position_ptr,
                                   void* cu_stream);

/* Per-head RMSNorm of Q and K, rotary embedding and the KV-cache write in one pass over a token block:
 * for every position s and head,  n = (x * rsqrt(mean(x^2) + eps)) * w  (fp32),  then the rotation of
 * b200tile_rope_seq at position + s.  Q heads are written to q_out [seq, q_heads, D]; K heads to
 * k_cache [kv_heads, max_seq, D] at row position + s; V heads are copied to v_cache at the same row.
 * Replaces `qk_norm_rope_kv_prefill_raw_f16` and, with seq_len = 1, q / k / v pointing into one fused
 * projection row and a device-side position, `qk_norm_rope_kv_decode_raw_f16`
 * (cutile-kernels/src/experimental/fused_transformer.rs:22-344, 356 ff.).
 *   q [seq, q_heads, D], k and v [seq, kv_heads, D]: heads D apart, rows *_seq_stride elements apart
 *   q_weight, k_weight [D]; inv_freq [D/2] f32; D in {16, 32, 64, 128, 256, 512}
 *   position_ptr: device u32[1] or null (then position_start is used).  Rows that would fall outside
 *   [0, max_seq) are not written to the caches.  All tensors 16-byte aligned. */
B200TILE_API int b200tile_qk_norm_rope_kv(const char* dtype, const void* q, const void* k, const void* v,
                                          const void* q_weight, const void* k_weight, const float* inv_freq,
                                          void* q_out, void* k_cache, void* v_cache, float eps, int position_start,
                                          const void* position_ptr, int seq_len, int num_q_heads, int num_kv_heads,
                                          int head_dim, int max_seq, int64_t q_seq_stride, int64_t k_seq_stride,
                                          int64_t v_seq_stride, int64_t q_out_seq_stride, void* cu_stream);

/* Greedy-decode token selection (cutile-kernels/src/argmax.rs).  Ties go to the lowest index.
 * b200tile_argmax_blocks: per block of `block_size` logits the maximum (as f32) and its index;
 *   replaces `argmax_blocks_f16` (:20-69).  block_max / block_idx hold ceil(len / block_size) entries.
 * b200tile_lm_head_argmax_blocks: the same over logits = weights [vocab, k] . hidden [k] that are never
 *   written, 64 vocabulary rows per block; replaces `lm_head_argmax_blocks_f16` (:81-143).  fp32
 *   products and sums; k <= 16384.  block_max / block_idx hold ceil(vocab / 64) entries.
 * b200tile_argmax_reduce_blocks: the winning index over the blocks into out[0]; replaces
 *   `argmax_reduce_blocks_to_u32` (:155-199), for any number of blocks.
 * dtype "f16" or "bf16"; all pointers are device pointers; ldw is the weights' row pitch in elements. */
B200TILE_API int b200tile_argmax_blocks(const char* dtype, const void* logits, float* block_max, uint32_t* block_idx,
                                        int len, int block_size, void* cu_stream);
B200TILE_API int b200tile_lm_head_argmax_blocks(const char* dtype, const void* weights, const void* hidden,
                                                float* block_max, uint32_t* block_idx, int vocab, int k,
                                                int64_t ldw, void* cu_stream);
B200TILE_API int b200tile_argmax_reduce_blocks(const float* block_max, const uint32_t* block_idx, uint32_t* out,
                                               int num_blocks, void* cu_stream);

/* out[m, n] = x . w^T (+ bias[n]) (+ residual[m, n]): the NT linear layer with its additive epilogue.  `bias` and
 * `residual` may each be NULL.  The bias is added to the fp32 accumulator before the 16-bit rounding; the residual is
 * added as `add_2d_f16` (cutile-kernels/src/pointwise.rs:20-36) adds two 16-bit tensors, so with a NULL bias the call
 * replaces the sequence "NT linear layer, then add_2d_f16" (an attention or MLP output projection followed by the
 * residual add) bit for bit, without the [m, n] intermediate going to memory and back.  `out` may alias `residual`.
 *   dtype "bf16" or "f16"; x [m, k], w [n, k], residual / out [m, n]; pitches in elements, multiples of 8; pointers
 *   16-byte aligned. */
B200TILE_API int b200tile_linear_bias_residual(const char* dtype, const void* x, const void* w, const void* bias,
                                               const void* residual, void* out, int m, int n, int k, int64_t ldx,
                                               int64_t ldw, int64_t ld_residual, int64_t ldo, void* cu_stream);

/* Element-wise kernels over [rows, cols] 16-bit tensors (pitches in elements; `out` may alias an input):
 * b200tile_add_2d:      out = lhs + rhs in the 16-bit type; replaces `add_2d_f16`
 *                       (cutile-kernels/src/pointwise.rs:20-36).
 * b200tile_silu_mul_2d: out = round16((gate / (1 + exp(-gate))) * up) through fp32; replaces
 *                       `silu_mul_2d_f16` (:50-77).  (b200tile_linear_swiglu fuses this step into the
 *                       gate/up projection.)
 * 16-byte aligned tensors take the vector path; anything else is accepted and runs with scalar accesses. */
B200TILE_API int b200tile_add_2d(const char* dtype, void* out, const void* lhs, const void* rhs, int rows, int cols,
                                 int64_t ld_out, int64_t ld_lhs, int64_t ld_rhs, void* cu_stream);
B200TILE_API int b200tile_silu_mul_2d(const char* dtype, void* out, const void* gate, const void* up, int rows,
                                      int cols, int64_t ld_out, int64_t ld_gate, int64_t ld_up, void* cu_stream);

/* Persistent grouped GEMM over device-side tables (MoE expert batches): for g in [0, num_groups)
 * C_g [m_g, n_g] = A_g [m_g, k_g] * B_g [k_g, n_g], row-major 16-bit operands, fp32 accumulation.
 * Replaces `group_gemm_f16_nt_desc` (cutile-kernels/src/experimental/moe.rs:66-128).
 *   a_ptrs, b_ptrs, c_ptrs   DEVICE arrays of num_groups i64 addresses (16-byte aligned tensors)
 *   a_metas, b_metas, c_metas DEVICE tables [num_groups, 8] of i32: {rows, cols, row stride in
 *                            elements (a multiple of 8), 5 unused}, moe.rs:27-63; m_g and k_g are
 *                            taken from a_metas, n_g from b_metas, the row stride of C from c_metas
 *   bn          B tile width: 128 or 256 (<= 0 selects 256); BM = 128, BK = 64
 *   workspace   DEVICE scratch of b200tile_group_gemm_workspace_bytes(num_groups) bytes, 128-byte
 *               aligned (the groups' extents and tile prefix sums); NULL lets
 *               the library keep one such block per device (allocated on first use, never inside a
 *               stream capture; calls that overlap on one device must then bring their own)
 * Groups with m, n = 0 are skipped; k = 0 stores zeros.  Nothing is read back to the host, so a group
 * whose addresses or row strides are not multiples of 16 bytes (or whose stride is shorter than its
 * row) cannot be refused by the call: the kernel skips it, stores nothing for it and records status
 * code 3 with the group's index (b200tile_status).  The operands are fetched with bounds-checked
 * 16-byte copies computed from the table entries; no tensor-map descriptor is built on the device. */
B200TILE_API uint64_t b200tile_group_gemm_workspace_bytes(int num_groups);
B200TILE_API int b200tile_group_gemm(const char* dtype, const int64_t* a_ptrs, const int64_t* b_ptrs,
                                     const int64_t* c_ptrs, const int32_t* a_metas, const int32_t* b_metas,
                                     const int32_t* c_metas, int num_groups, int bn, void* workspace,
                                     uint64_t workspace_bytes, void* cu_stream);

/* out = softmax(qk_scale * Q K^T + mask) V, one query tile per tile-block, online softmax with
 * fp32 statistics, probabilities rounded to the 16-bit input type before P.V.
 * Replaces `fmha_prefill_causal` (cutile-kernels/src/attention.rs:232-392), the benchmark kernels
 * `fmha` (cutile-benchmarks/benches/fmha.rs:20-146, fmha_causal.rs:20-136) and the example
 * kernels (cutile-examples/examples/flash_attention.rs:20-136, flash_attention_causal.rs:19-134).
 *   dtype      "bf16" or "f16" (tensor cores; head_dim 64 or 128), or "f32": every product and sum in IEEE
 *              fp32 on the CUDA cores, head_dim 32, 64 or 128 -- the element type of the reference's two
 *              asserted examples (flash_attention.rs:199-264, flash_attention_causal.rs:216-285); like the
 *              exact fp32 GEMM a correctness configuration, with fp32 probabilities
 *   q          query tensor; element (b, h, i, d) at q + (b*heads + h)*q_strides[0] +
 *              i*q_strides[1] + d  -- covers both (b,h,s,d) and [q_len, heads, D] layouts
 *   k, v       same addressing with heads_kv; kv head = h / (heads / heads_kv) (GQA)
 *   out        same addressing as q
 *   causal     0/1; key j is visible to query i iff j <= i + input_pos (the diagonal included,
 *              attention.rs:348; flash_attention_causal.rs:176)
 * Strides are in ELEMENTS; the head vector is contiguous. */
B200TILE_API int b200tile_fmha_fwd(const char* dtype, const void* q, const void* k, const void* v,
                                   void* out, int batch, int heads, int heads_kv, int q_len,
                                   int kv_len, int head_dim, const int64_t q_strides[2],
                                   const int64_t k_strides[2], const int64_t v_strides[2],
                                   const int64_t o_strides[2], float qk_scale, int causal,
                                   int input_pos, void* cu_stream);

/* b200tile_fmha_fwd with the causal offset read from DEVICE memory at kernel time, so that a
 * captured graph can be replayed while the decode position advances.  Replaces the
 * dynamic-position kernels `fmha_causal` and `flash_attn_causal_seq_dynpos_f16`
 * (cutile-kernels/src/attention.rs:588-721, 118-226: `position_start: &Tensor<u32, {[1]}>`).
 * `position_start` points to one u32 = position of query row 0; key j is visible to query i iff
 * j <= i + *position_start and j < kv_len. */
B200TILE_API int b200tile_fmha_fwd_dynpos(const char* dtype, const void* q, const void* k, const void* v,
                                          void* out, int batch, int heads, int heads_kv, int q_len,
                                          int kv_len, int head_dim, const int64_t q_strides[2],
                                          const int64_t k_strides[2], const int64_t v_strides[2],
                                          const int64_t o_strides[2], float qk_scale, int causal,
                                          const void* position_start, void* cu_stream);

/* Split-KV grouped-query decode attention (one query token per head) and its merge.
 * Replaces `fmha_decode_gqa_split` and `splitk_reduce_merge`
 * (cutile-kernels/src/attention.rs:727-901, 907-1015).
 *   q            [kv_heads, group, D]                 one token, `group` query heads per K/V head
 *   k, v         [kv_heads, kv_capacity, D]           the KV cache
 *   att_partial  [kv_heads, num_kv_splits*group, D]   scratch, same element type (split-major)
 *   lse_partial  [kv_heads, num_kv_splits*group]      scratch, fp32, log2 domain (m + log2 l)
 *   out          [kv_heads, group, D], or NULL to run the split pass only
 *   position_start  DEVICE pointer to one u32: keys [0, *position_start + 1) are attended
 *   bn           key-tile size that defines the split boundaries: split s covers tiles
 *                [s*ceil(T/S), min((s+1)*ceil(T/S), T)) of T = ceil(s_kv/bn) tiles (attention.rs:774-780)
 * Strides in ELEMENTS: {head stride, row stride} per tensor; head vectors contiguous; group <= 16;
 * D in {64, 128}; dtype "bf16" or "f16".  An empty split yields att = 0, lse = -1e30. */
B200TILE_API int b200tile_fmha_decode_gqa_split(const char* dtype, const void* q, const void* k, const void* v,
                                                void* att_partial, float* lse_partial, void* out,
                                                const void* position_start, int kv_heads, int group,
                                                int head_dim, int kv_capacity, int bn, int num_kv_splits,
                                                float qk_scale, const int64_t q_strides[2],
                                                const int64_t k_strides[2], const int64_t v_strides[2],
                                                const int64_t att_strides[2], int64_t lse_head_stride,
                                                const int64_t out_strides[2], void* cu_stream);

/* The merge alone (attention.rs:907-1015): out[h,g,:] = sum_s w_s * att_partial[h, s*group+g, :],
 * w_s = exp2(lse_s - max_s lse) / max(sum_s exp2(lse_s - max), 1e-8). */
B200TILE_API int b200tile_splitk_reduce_merge(const char* dtype, const void* att_partial, const float* lse_partial,
                                              void* out, int kv_heads, int group, int head_dim,
                                              int num_kv_splits, const int64_t att_strides[2],
                                              int64_t lse_head_stride, const int64_t out_strides[2],
                                              void* cu_stream);

/* z[M,N] = alpha * sum over 128-deep k-blocks of  xs[m,kb] * ys[n/128,kb] * (x_q[m,kb] . y_q[n,kb]),
 * x_q [M,K] and y_q [N,K] in f8e4m3fn (bit convention cuda-core/src/dtype.rs:25-31,223), one fp32
 * scale per 1x128 block of x (x_scales [M, K/128]) and per 128x128 block of y
 * (y_scales [ceil(N/128), K/128]).  The reference has no kernel for this scale granularity (its
 * fp8 path is MXFP8, cutile-examples/examples/mxfp8.rs:34-64); the operand layout ("NT", both
 * K-major) and the `alpha` epilogue follow that `linear_tile`.
 *   out_dtype  "bf16" or "f32";  K must be a multiple of 128; leading dimensions in ELEMENTS. */
B200TILE_API int b200tile_linear_fp8_blk128(const void* x, const void* y, const float* x_scales,
                                            const float* y_scales, void* z, const char* out_dtype,
                                            int m, int n, int k, int64_t ldx, int64_t ldy, int64_t ldz,
                                            int64_t ld_xs, int64_t ld_ys, float alpha, void* cu_stream);

/* z[M,N] = alpha * sum_k x[m,k]*xs[m,k/16] * y[n,k]*ys[n,k/16]  (NVFP4 block-scaled linear layer).
 * Replaces `linear_tile` of cutile-examples/examples/nvfp4.rs:37-76 (`mmaf_scaled`,
 * cutile/src/_core.rs:2288-2313): x, y packed f4e2m1fnx2 [M,K/2], [N,K/2] (low nibble = first
 * value, cuda-core/src/dtype.rs:60-110); xs, ys f8e4m3fn scales in logical row-major [M,K/16],
 * [N,K/16] as the example keeps them; alpha carries the folded per-tensor global scales
 * (cutile-book/tutorials/11-nvfp4-inference.md:147-148).
 *   out_dtype  "bf16" or "f32";  K must be a multiple of 64; leading dimensions in BYTES of the
 *              packed / scale rows (ldx, ldy >= K/2; ld_xs, ld_ys >= K/16, multiples of 4)
 *   workspace  device scratch of at least b200tile_linear_nvfp4_workspace_bytes(m, n, k) bytes,
 *              16-byte aligned: the scales are re-laid out into it on every call (stream-ordered);
 *              calls that overlap on the device must not share a workspace
 *   config     -1 = default (0 when m <= 32, 3 when m >= 512, else 1), 0/1/2 = single-CTA kernel with B tiles of
 *              128/192/256 rows, 3 = CTA pairs (cta_group::2) with 256 x 256 tiles */
B200TILE_API uint64_t b200tile_linear_nvfp4_workspace_bytes(int m, int n, int k);
B200TILE_API int b200tile_linear_nvfp4(const void* x, const void* y, const void* x_scales,
                                       const void* y_scales, void* z, const char* out_dtype, int m,
                                       int n, int k, int64_t ldx, int64_t ldy, int64_t ldz,
                                       int64_t ld_xs, int64_t ld_ys, float alpha, void* workspace,
                                       uint64_t workspace_bytes, int config, void* cu_stream);

/* z[M,N] = alpha * sum_k x[m,k]*xs[m,k/32] * y[n,k]*ys[n,k/32]  (MXFP8 block-scaled linear layer).
 * Replaces `linear_tile` of cutile-examples/examples/mxfp8.rs:34-64 (`mmaf_scaled` with
 * f8e8m0fnu scales, cutile/tests/tensor_and_matrix_ops.rs:266-283): x [M,K], y [N,K] f8e4m3fn;
 * xs [M,K/32], ys [N,K/32] f8e8m0fnu in logical row-major order.
 *   out_dtype  "bf16" or "f32";  K must be a multiple of 128; leading dimensions in BYTES
 *   workspace  at least b200tile_linear_mxfp8_workspace_bytes(m, n, k) bytes, 16-byte aligned
 *              (scale re-layout, as for b200tile_linear_nvfp4) */
B200TILE_API uint64_t b200tile_linear_mxfp8_workspace_bytes(int m, int n, int k);
B200TILE_API int b200tile_linear_mxfp8(const void* x, const void* y, const void* x_scales,
                                       const void* y_scales, void* z, const char* out_dtype, int m,
                                       int n, int k, int64_t ldx, int64_t ldy, int64_t ldz,
                                       int64_t ld_xs, int64_t ld_ys, float alpha, void* workspace,
                                       uint64_t workspace_bytes, void* cu_stream);

/* z[M,N] = alpha * sum_k x[m,k]*xs[m,k/32] * y[n,k]*ys[n,k/32]  (MXFP4: NVFP4's packed E2M1 operands with
 * power-of-two f8e8m0fnu scales per 32 elements).  The operand / scale pairing of `mmaf_scaled` in
 * cutile/tests/tensor_and_matrix_ops.rs:224-244 (`raw_mmaf_scaled_nvfp4_kernel`): x [M,K/2], y [N,K/2]
 * f4e2m1fnx2 bytes (low nibble first); xs [M,K/32], ys [N,K/32] in logical row-major order.
 *   out_dtype  "bf16" or "f32";  K must be a multiple of 128; leading dimensions in BYTES
 *   workspace  at least b200tile_linear_mxfp4_workspace_bytes(m, n, k) bytes, 16-byte aligned */
B200TILE_API uint64_t b200tile_linear_mxfp4_workspace_bytes(int m, int n, int k);
B200TILE_API int b200tile_linear_mxfp4(const void* x, const void* y, const void* x_scales,
                                       const void* y_scales, void* z, const char* out_dtype, int m,
                                       int n, int k, int64_t ldx, int64_t ldy, int64_t ldz,
                                       int64_t ld_xs, int64_t ld_ys, float alpha, void* workspace,
                                       uint64_t workspace_bytes, void* cu_stream);

/* NVFP4 linear layer with the weight scales laid out ahead of time.  Inference weights do not
 * change, so their scales can be brought into the kernel's tile layout once
 * (b200tile_nvfp4_prepare_weight_scales, for one `config` = B tile of 128 / 192 / 256 rows); every
 * later call then runs a single kernel and needs no workspace (the activation scales are read in
 * place).  Same operands and semantics as b200tile_linear_nvfp4 otherwise; config 0 suits decode
 * (m <= 128: most tile-blocks), config 1 large m.  No reference counterpart: the reference passes
 * logically row-major scales on every call (cutile-examples/examples/nvfp4.rs:37-76).
 * The weights `y` and their prepared scales are treated as CONSTANTS: with m <= 32 the kernel is launched with
 * programmatic stream serialisation and begins to fetch them while the preceding kernel of the stream is still
 * running (it waits for that kernel before it reads x, x_scales or writes z).  Do not use this entry, or
 * registered scales, for weights that earlier work on the same stream is still writing. */
B200TILE_API uint64_t b200tile_nvfp4_weight_scales_bytes(int n, int k, int config);
B200TILE_API int b200tile_nvfp4_prepare_weight_scales(const void* y_scales, int n, int k, int64_t ld_ys,
                                                      int config, void* prepared, uint64_t prepared_bytes,
                                                      void* cu_stream);
B200TILE_API int b200tile_linear_nvfp4_prepared(const void* x, const void* y, const void* x_scales,
                                                const void* y_scales_prepared, void* z, const char* out_dtype,
                                                int m, int n, int k, int64_t ldx, int64_t ldy, int64_t ldz,
                                                int64_t ld_xs, float alpha, int config, void* cu_stream);

/* Registry behind the generic `linear_tile` route.  The reference's kernel takes the weight scales in
 * logical row-major order on every call (cutile-examples/examples/nvfp4.rs:37-76); weights of a served model
 * do not change, so their scales can be laid out once (b200tile_nvfp4_prepare_weight_scales) and registered
 * under the address of the row-major tensor.  b200tile_launch("linear_tile", ...) with M <= 128 on a registered
 * y_scales (same n, k, row pitch, current device) then runs the prepared form: one kernel, no scale pre-pass.
 * The caller keeps both buffers alive and unregisters before freeing either.  No counterpart in the
 * reference, whose JIT re-reads the row-major scales in every launch. */
B200TILE_API int b200tile_nvfp4_register_weight_scales(const void* y_scales, int n, int k, int64_t ld_ys,
                                                       int config, const void* prepared);
B200TILE_API int b200tile_nvfp4_unregister_weight_scales(const void* y_scales);

/* Same computation as b200tile_linear_nvfp4, for callers that cannot provide device memory
 * (no counterpart in the reference, whose launchers always allocate through their own pool):
 * code that runs while a stream is being captured and must stay away from any allocator, plugins
 * that may not draw from their host's memory pool, and start-up code that runs before that pool
 * exists.  The scale scratch is a fixed array inside the library image, so
 *   - every GPU that loads the library gives up B200TILE_NVFP4_STATIC_SCRATCH_BYTES until exit;
 *   - a problem whose re-laid-out scales exceed that size is refused with B200TILE_ERR_INVALID
 *     (the default config needs about (ceil(M/128)*128 + ceil(N/192)*256) * ceil(K/256)*256 / 16
 *     bytes: 5.9 MB for 4096 x 14336 x 4096);
 *   - all calls on one GPU share the array: calls that may overlap on the device (different
 *     streams, parallel graph branches) race on it and must be serialised by the caller;
 *   - the first call on each device looks the array's address up (no allocation, but a runtime
 *     query): make that first call before beginning a stream capture.
 * It performs no cudaMalloc/cudaFree and calls no allocating library routine. */
#define B200TILE_NVFP4_STATIC_SCRATCH_BYTES (8u << 20)
B200TILE_API int b200tile_linear_nvfp4_static(const void* x, const void* y, const void* x_scales,
                                              const void* y_scales, void* z, const char* out_dtype,
                                              int m, int n, int k, int64_t ldx, int64_t ldy,
                                              int64_t ldz, int64_t ld_xs, int64_t ld_ys, float alpha,
                                              int config, void* cu_stream);

#ifdef __cplusplus
}
#endif
#endif /* B200TILE_H_ */
