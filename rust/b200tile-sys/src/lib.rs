//! Raw FFI bindings to `libb200tile.so`, the precompiled sm_100a implementation of cuTile Rust's
//! dense-contraction kernels (GEMM, block-scaled linear layers, attention forward and their neighbours).
//!
//! Every function exported by `include/b200tile.h` is declared here, in the header's order; the
//! header's comments say which reference kernel or call each one replaces.  The `cutile` crate's
//! generated launchers reach the library through [`b200tile_launch`] (see `cutile-launcher.patch`
//! in the parent directory); the typed entry points are for callers that do not go through a generated
//! launcher.  All functions return 0 on success or a `B200TILE_ERR_*` code; the message of the last
//! error of the calling thread is [`b200tile_last_error`].
//!
//! This file is generated from the header by `gen_ffi.py` (same directory); regenerate it instead of
//! editing the `extern` block by hand.
#![allow(non_camel_case_types)]

use std::os::raw::{c_char, c_int, c_uint, c_void};

pub const B200TILE_OK: c_int = 0;
pub const B200TILE_ERR_INVALID: c_int = 1;
pub const B200TILE_ERR_UNSUPPORTED: c_int = 2;
pub const B200TILE_ERR_CUDA: c_int = 3;
pub const B200TILE_ERR_DEVICE: c_int = 4;
pub const B200TILE_ERR_ALIGN: c_int = 5;

/// `CompileOptions` of the launcher (cutile-compiler/src/hints.rs:94-126); -1 = not set.
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct B200CompileOptions {
    pub occupancy: c_int,
    pub num_cta_in_cga: c_int,
    pub max_divisibility: c_int,
    pub num_worker_warps_per_cta: c_int,
}

/// One precompiled configuration, as listed for the autotuner (cutile/src/tune.rs:53-121).
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct B200Config {
    pub id: c_int,
    pub bm: c_int,
    pub bn: c_int,
    pub bk: c_int,
    pub stages: c_int,
    pub num_cta_in_cga: c_int,
    pub occupancy: c_int,
}

/// Device status record: 0 = ok, 1 = a bounded wait gave up, 3 = a grouped-GEMM group was skipped.
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct B200Status {
    pub code: u32,
    pub block: u32,
    pub site: u32,
    pub aux: u32,
}

#[link(name = "b200tile")]
extern "C" {
// --- generated: begin ---
    pub fn b200tile_abi_version() -> c_int;
    pub fn b200tile_init(device_ordinal: c_int) -> c_int;
    pub fn b200tile_last_error() -> *const c_char;
    pub fn b200tile_num_sms() -> c_int;
    pub fn b200tile_status(cu_stream: *mut c_void, out: *mut B200Status) -> c_int;
    pub fn b200tile_status_reset(cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_query_configs(kernel: *const c_char, dtype: *const c_char, out: *mut B200Config,
        cap: c_int) -> c_int;
    pub fn b200tile_launch(kernel: *const c_char, generics: *const *const c_char, n_generics: c_int,
        opts: *const B200CompileOptions, params: *const *const c_void, n_params: c_int,
        grid: *const c_uint, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_prepare(kernel: *const c_char, generics: *const *const c_char, n_generics: c_int,
        opts: *const B200CompileOptions) -> c_int;
    pub fn b200tile_gemm(dtype: *const c_char, b_layout: c_int, a: *const c_void, b: *const c_void,
        c: *mut c_void, batch: c_int, m: c_int, n: c_int, k: c_int, lda: i64, ldb: i64, ldc: i64,
        stride_a: i64, stride_b: i64, stride_c: i64, accumulate: c_int, config: c_int, group_size_m: c_int,
        num_programs: c_int, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_gemm_host(dtype: *const c_char, b_layout: c_int, a_host: *const c_void,
        b_host: *const c_void, c_host: *mut c_void, a_dev: *mut c_void, b_dev: *mut c_void,
        c_dev: *mut c_void, m: c_int, n: c_int, k: c_int, slab_rows: c_int, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_linear_swiglu(dtype: *const c_char, x: *const c_void, w_gate_up: *const c_void,
        out: *mut c_void, m: c_int, inter: c_int, k: c_int, ldx: i64, ldw: i64, ldo: i64,
        cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_rms_norm(dtype: *const c_char, x: *const c_void, w: *const c_void, out: *mut c_void,
        rows: c_int, n: c_int, ldx: i64, ldo: i64, eps: f32, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_add_rms_norm(dtype: *const c_char, residual: *const c_void, x: *const c_void,
        w: *const c_void, out: *mut c_void, residual_out: *mut c_void, rows: c_int, n: c_int,
        ld_residual: i64, ldx: i64, ldo: i64, ld_residual_out: i64, eps: f32, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_rope_seq(dtype: *const c_char, x: *const c_void, inv_freq: *const f32,
        out: *mut c_void, seq: c_int, heads: c_int, head_dim: c_int, x_strides: *const i64,
        out_strides: *const i64, position_start: c_int, position_ptr: *const c_void, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_qk_norm_rope_kv(dtype: *const c_char, q: *const c_void, k: *const c_void,
        v: *const c_void, q_weight: *const c_void, k_weight: *const c_void, inv_freq: *const f32,
        q_out: *mut c_void, k_cache: *mut c_void, v_cache: *mut c_void, eps: f32, position_start: c_int,
        position_ptr: *const c_void, seq_len: c_int, num_q_heads: c_int, num_kv_heads: c_int,
        head_dim: c_int, max_seq: c_int, q_seq_stride: i64, k_seq_stride: i64, v_seq_stride: i64,
        q_out_seq_stride: i64, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_argmax_blocks(dtype: *const c_char, logits: *const c_void, block_max: *mut f32,
        block_idx: *mut u32, len: c_int, block_size: c_int, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_lm_head_argmax_blocks(dtype: *const c_char, weights: *const c_void,
        hidden: *const c_void, block_max: *mut f32, block_idx: *mut u32, vocab: c_int, k: c_int, ldw: i64,
        cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_argmax_reduce_blocks(block_max: *const f32, block_idx: *const u32, out: *mut u32,
        num_blocks: c_int, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_linear_bias_residual(dtype: *const c_char, x: *const c_void, w: *const c_void,
        bias: *const c_void, residual: *const c_void, out: *mut c_void, m: c_int, n: c_int, k: c_int,
        ldx: i64, ldw: i64, ld_residual: i64, ldo: i64, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_add_2d(dtype: *const c_char, out: *mut c_void, lhs: *const c_void, rhs: *const c_void,
        rows: c_int, cols: c_int, ld_out: i64, ld_lhs: i64, ld_rhs: i64, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_silu_mul_2d(dtype: *const c_char, out: *mut c_void, gate: *const c_void,
        up: *const c_void, rows: c_int, cols: c_int, ld_out: i64, ld_gate: i64, ld_up: i64,
        cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_group_gemm_workspace_bytes(num_groups: c_int) -> u64;
    pub fn b200tile_group_gemm(dtype: *const c_char, a_ptrs: *const i64, b_ptrs: *const i64,
        c_ptrs: *const i64, a_metas: *const i32, b_metas: *const i32, c_metas: *const i32,
        num_groups: c_int, bn: c_int, workspace: *mut c_void, workspace_bytes: u64, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_fmha_fwd(dtype: *const c_char, q: *const c_void, k: *const c_void, v: *const c_void,
        out: *mut c_void, batch: c_int, heads: c_int, heads_kv: c_int, q_len: c_int, kv_len: c_int,
        head_dim: c_int, q_strides: *const i64, k_strides: *const i64, v_strides: *const i64,
        o_strides: *const i64, qk_scale: f32, causal: c_int, input_pos: c_int, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_fmha_fwd_dynpos(dtype: *const c_char, q: *const c_void, k: *const c_void,
        v: *const c_void, out: *mut c_void, batch: c_int, heads: c_int, heads_kv: c_int, q_len: c_int,
        kv_len: c_int, head_dim: c_int, q_strides: *const i64, k_strides: *const i64,
        v_strides: *const i64, o_strides: *const i64, qk_scale: f32, causal: c_int,
        position_start: *const c_void, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_fmha_decode_gqa_split(dtype: *const c_char, q: *const c_void, k: *const c_void,
        v: *const c_void, att_partial: *mut c_void, lse_partial: *mut f32, out: *mut c_void,
        position_start: *const c_void, kv_heads: c_int, group: c_int, head_dim: c_int, kv_capacity: c_int,
        bn: c_int, num_kv_splits: c_int, qk_scale: f32, q_strides: *const i64, k_strides: *const i64,
        v_strides: *const i64, att_strides: *const i64, lse_head_stride: i64, out_strides: *const i64,
        cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_splitk_reduce_merge(dtype: *const c_char, att_partial: *const c_void,
        lse_partial: *const f32, out: *mut c_void, kv_heads: c_int, group: c_int, head_dim: c_int,
        num_kv_splits: c_int, att_strides: *const i64, lse_head_stride: i64, out_strides: *const i64,
        cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_linear_fp8_blk128(x: *const c_void, y: *const c_void, x_scales: *const f32,
        y_scales: *const f32, z: *mut c_void, out_dtype: *const c_char, m: c_int, n: c_int, k: c_int,
        ldx: i64, ldy: i64, ldz: i64, ld_xs: i64, ld_ys: i64, alpha: f32, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_linear_nvfp4_workspace_bytes(m: c_int, n: c_int, k: c_int) -> u64;
    pub fn b200tile_linear_nvfp4(x: *const c_void, y: *const c_void, x_scales: *const c_void,
        y_scales: *const c_void, z: *mut c_void, out_dtype: *const c_char, m: c_int, n: c_int, k: c_int,
        ldx: i64, ldy: i64, ldz: i64, ld_xs: i64, ld_ys: i64, alpha: f32, workspace: *mut c_void,
        workspace_bytes: u64, config: c_int, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_linear_mxfp8_workspace_bytes(m: c_int, n: c_int, k: c_int) -> u64;
    pub fn b200tile_linear_mxfp8(x: *const c_void, y: *const c_void, x_scales: *const c_void,
        y_scales: *const c_void, z: *mut c_void, out_dtype: *const c_char, m: c_int, n: c_int, k: c_int,
        ldx: i64, ldy: i64, ldz: i64, ld_xs: i64, ld_ys: i64, alpha: f32, workspace: *mut c_void,
        workspace_bytes: u64, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_linear_mxfp4_workspace_bytes(m: c_int, n: c_int, k: c_int) -> u64;
    pub fn b200tile_linear_mxfp4(x: *const c_void, y: *const c_void, x_scales: *const c_void,
        y_scales: *const c_void, z: *mut c_void, out_dtype: *const c_char, m: c_int, n: c_int, k: c_int,
        ldx: i64, ldy: i64, ldz: i64, ld_xs: i64, ld_ys: i64, alpha: f32, workspace: *mut c_void,
        workspace_bytes: u64, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_nvfp4_weight_scales_bytes(n: c_int, k: c_int, config: c_int) -> u64;
    pub fn b200tile_nvfp4_prepare_weight_scales(y_scales: *const c_void, n: c_int, k: c_int, ld_ys: i64,
        config: c_int, prepared: *mut c_void, prepared_bytes: u64, cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_linear_nvfp4_prepared(x: *const c_void, y: *const c_void, x_scales: *const c_void,
        y_scales_prepared: *const c_void, z: *mut c_void, out_dtype: *const c_char, m: c_int, n: c_int,
        k: c_int, ldx: i64, ldy: i64, ldz: i64, ld_xs: i64, alpha: f32, config: c_int,
        cu_stream: *mut c_void) -> c_int;
    pub fn b200tile_nvfp4_register_weight_scales(y_scales: *const c_void, n: c_int, k: c_int, ld_ys: i64,
        config: c_int, prepared: *const c_void) -> c_int;
    pub fn b200tile_nvfp4_unregister_weight_scales(y_scales: *const c_void) -> c_int;
    pub fn b200tile_linear_nvfp4_static(x: *const c_void, y: *const c_void, x_scales: *const c_void,
        y_scales: *const c_void, z: *mut c_void, out_dtype: *const c_char, m: c_int, n: c_int, k: c_int,
        ldx: i64, ldy: i64, ldz: i64, ld_xs: i64, ld_ys: i64, alpha: f32, config: c_int,
        cu_stream: *mut c_void) -> c_int;
// --- generated: end ---
}
