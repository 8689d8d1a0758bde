"""TEST INFRASTRUCTURE -- ctypes/numpy front end of ``oracle/oracle.c`` (the CPU restatement of
the reference's host-side checks).  Only tests, the smoke check and the benchmark's CPU-baseline /
reference arms may import this module; the product package never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_float, c_int, c_int64, c_uint8, c_uint16, c_uint32, c_void_p

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compiles oracle.c with the committed Makefile (gcc only)."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(src) > os.path.getmtime(LIB_PATH):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        L = ctypes.CDLL(LIB_PATH)
        fp, u8p, u16p = POINTER(c_float), POINTER(c_uint8), POINTER(c_uint16)
        i64 = c_int64
        sig = {
            "oracle_cpu_gemm": (None, [fp, fp, fp, i64, i64, i64]),
            "oracle_cpu_gemm_rows": (None, [fp, fp, fp, i64, i64, i64, i64, i64]),
            "oracle_cpu_gemm_rows_mt": (c_int, [fp, fp, fp, i64, i64, i64, i64, i64, c_int]),
            "oracle_cpu_gemm_nt_rows": (None, [fp, fp, fp, i64, i64, i64, c_float, i64, i64]),
            "oracle_cpu_gemm_nt_rows_mt": (c_int, [fp, fp, fp, i64, i64, i64, c_float, i64, i64, c_int]),
            "oracle_fmha_ref_cpu": (None, [fp, fp, fp, fp, i64, i64, i64, i64, i64, c_float, i64, i64, c_int]),
            "oracle_fmha_ref_cpu_slab": (c_int, [fp, fp, fp, fp, i64, i64, i64, i64, i64, c_float, i64,
                                                 i64, c_int, i64, i64, i64, i64, c_int]),
            "oracle_f32_to_bf16": (c_uint16, [c_float]),
            "oracle_bf16_to_f32": (c_float, [c_uint16]),
            "oracle_f32_to_bf16_array": (None, [fp, u16p, i64]),
            "oracle_bf16_to_f32_array": (None, [u16p, fp, i64]),
            "oracle_e4m3_to_f32": (c_float, [c_uint8]),
            "oracle_f32_to_e4m3": (c_uint8, [c_float]),
            "oracle_e5m2_to_f32": (c_float, [c_uint8]),
            "oracle_e8m0_to_f32": (c_float, [c_uint8]),
            "oracle_e2m1_to_f32": (c_float, [c_uint8]),
            "oracle_f32_to_e2m1": (c_uint8, [c_float]),
            "oracle_pack_e2m1x2": (c_uint8, [c_uint8, c_uint8]),
            "oracle_quant_fp8_block": (None, [fp, i64, i64, i64, i64, u8p, fp]),
            "oracle_dequant_fp8_block": (None, [u8p, fp, i64, i64, i64, i64, fp]),
            "oracle_quant_nvfp4": (c_float, [fp, i64, i64, u8p, u8p]),
            "oracle_dequant_nvfp4": (None, [u8p, u8p, i64, i64, fp]),
            "oracle_quant_mxfp8": (None, [fp, i64, i64, u8p, u8p]),
            "oracle_dequant_mxfp8": (None, [u8p, u8p, i64, i64, fp]),
            "oracle_fmha_decode_gqa_split": (None, [fp, fp, fp, fp, fp, i64, i64, i64, i64, i64, i64, i64, c_float, c_int]),
            "oracle_splitk_reduce_merge": (None, [fp, fp, fp, i64, i64, i64, i64, c_int]),
            "oracle_persistent_num_programs": (c_uint32, [i64, i64, c_int, c_int, c_int, c_int, c_int]),
            "oracle_swizzled_bid": (None, [c_int, c_int, c_int, c_int, POINTER(c_int), POINTER(c_int)]),
            "oracle_max_threads": (c_int, []),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray, ct):
    return a.ctypes.data_as(POINTER(ct))


def max_threads() -> int:
    return int(lib().oracle_max_threads())


# ---- GEMM -------------------------------------------------------------------------------
def cpu_gemm(x, y, rows=None, threads: int = 1) -> np.ndarray:
    """z = x[M,K] . y[K,N]; `rows=(r0,r1)` computes only that slab (other rows stay zero)."""
    x, y = _f32(x), _f32(y)
    m, k = x.shape
    k2, n = y.shape
    assert k == k2
    z = np.zeros((m, n), dtype=np.float32)
    r0, r1 = rows if rows is not None else (0, m)
    lib().oracle_cpu_gemm_rows_mt(_p(x, c_float), _p(y, c_float), _p(z, c_float), m, n, k, r0, r1,
                                  threads)
    return z


def cpu_gemm_nt(x, y, alpha: float = 1.0, rows=None, threads: int = 1) -> np.ndarray:
    """z = alpha * x[M,K] . y[N,K]^T."""
    x, y = _f32(x), _f32(y)
    m, k = x.shape
    n, k2 = y.shape
    assert k == k2
    z = np.zeros((m, n), dtype=np.float32)
    r0, r1 = rows if rows is not None else (0, m)
    lib().oracle_cpu_gemm_nt_rows_mt(_p(x, c_float), _p(y, c_float), _p(z, c_float), m, n, k,
                                     alpha, r0, r1, threads)
    return z


# ---- attention --------------------------------------------------------------------------
def fmha_ref_cpu(q, k, v, qk_scale: float, input_pos: int = 0, query_group_size: int = 1,
                 causal: bool = False, bh=None, rows=None, threads: int = 1) -> np.ndarray:
    """q (b,h,m,d), k/v (b,hkv,m,d) -> out (b,h,m,d); slabs outside (bh, rows) stay zero."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    b, h, m, d = q.shape
    hkv = k.shape[1]
    out = np.zeros_like(q)
    bh0, bh1 = bh if bh is not None else (0, b * h)
    i0, i1 = rows if rows is not None else (0, m)
    lib().oracle_fmha_ref_cpu_slab(_p(q, c_float), _p(k, c_float), _p(v, c_float),
                                   _p(out, c_float), b, h, hkv, m, d, qk_scale, input_pos,
                                   query_group_size, int(causal), bh0, bh1, i0, i1, threads)
    return out


def fmha_decode_gqa_split(q, k, v, s_kv: int, bn: int, splits: int, qk_scale: float, is_f16: bool = False):
    """q [H,G,D], k/v [H,cap,D] -> (att [H, splits*G, D], lse [H, splits*G])."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    h, g, d = q.shape
    cap = k.shape[1]
    att = np.zeros((h, splits * g, d), dtype=np.float32)
    lse = np.zeros((h, splits * g), dtype=np.float32)
    lib().oracle_fmha_decode_gqa_split(_p(q, c_float), _p(k, c_float), _p(v, c_float), _p(att, c_float),
                                       _p(lse, c_float), h, g, d, cap, s_kv, bn, splits, qk_scale, int(is_f16))
    return att, lse


def splitk_reduce_merge(att, lse, group: int, is_f16: bool = False) -> np.ndarray:
    att, lse = _f32(att), _f32(lse)
    h, sg, d = att.shape
    splits = sg // group
    out = np.zeros((h, group, d), dtype=np.float32)
    lib().oracle_splitk_reduce_merge(_p(att, c_float), _p(lse, c_float), _p(out, c_float), h, group, d, splits,
                                     int(is_f16))
    return out


# ---- codecs -----------------------------------------------------------------------------
def f32_to_bf16_bits(a) -> np.ndarray:
    a = _f32(a)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().oracle_f32_to_bf16_array(_p(a, c_float), _p(out, c_uint16), a.size)
    return out


def bf16_bits_to_f32(bits) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, dtype=np.float32)
    lib().oracle_bf16_to_f32_array(_p(bits, c_uint16), _p(out, c_float), bits.size)
    return out


def round_bf16(a) -> np.ndarray:
    return bf16_bits_to_f32(f32_to_bf16_bits(a))


def e4m3_table() -> np.ndarray:
    return np.array([lib().oracle_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)


def e2m1_table() -> np.ndarray:
    return np.array([lib().oracle_e2m1_to_f32(i) for i in range(16)], dtype=np.float32)


def quant_fp8_block(x, block_r: int, block_c: int):
    x = _f32(x)
    r, c = x.shape
    q = np.empty((r, c), dtype=np.uint8)
    s = np.empty((-(-r // block_r), -(-c // block_c)), dtype=np.float32)
    lib().oracle_quant_fp8_block(_p(x, c_float), r, c, block_r, block_c, _p(q, c_uint8),
                                 _p(s, c_float))
    return q, s


def dequant_fp8_block(q, s, block_r: int, block_c: int) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.uint8)
    s = _f32(s)
    r, c = q.shape
    out = np.empty((r, c), dtype=np.float32)
    lib().oracle_dequant_fp8_block(_p(q, c_uint8), _p(s, c_float), r, c, block_r, block_c,
                                   _p(out, c_float))
    return out


def quant_nvfp4(x):
    """-> (packed [R, C/2] u8, scales [R, C/16] u8 (e4m3 bits), global scale g)."""
    x = _f32(x)
    r, c = x.shape
    assert c % 16 == 0
    packed = np.empty((r, c // 2), dtype=np.uint8)
    scales = np.empty((r, c // 16), dtype=np.uint8)
    g = lib().oracle_quant_nvfp4(_p(x, c_float), r, c, _p(packed, c_uint8), _p(scales, c_uint8))
    return packed, scales, float(g)


def dequant_nvfp4(packed, scales) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    r, c2 = packed.shape
    out = np.empty((r, c2 * 2), dtype=np.float32)
    lib().oracle_dequant_nvfp4(_p(packed, c_uint8), _p(scales, c_uint8), r, c2 * 2,
                               _p(out, c_float))
    return out


_E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def dequant_mxfp4(packed, scales) -> np.ndarray:
    """Packed f4e2m1fnx2 bytes (low nibble = even element, cuda-core/src/dtype.rs:60-110) times one f8e8m0fnu
    scale 2^(e - 127) per 32 elements: the operand / scale pairing of `mmaf_scaled` in
    cutile/tests/tensor_and_matrix_ops.rs:224-244.  numpy; every product is exact in fp32."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    r, c2 = packed.shape
    codes = np.empty((r, c2 * 2), dtype=np.uint8)
    codes[:, 0::2] = packed & 0xF
    codes[:, 1::2] = packed >> 4
    vals = _E2M1_VALUES[codes & 7] * np.where(codes & 8, np.float32(-1.0), np.float32(1.0))
    sc = np.ldexp(np.float32(1.0), scales.astype(np.int32) - 127).astype(np.float32)
    return (vals.reshape(r, c2 * 2 // 32, 32) * sc[:, :, None]).reshape(r, c2 * 2).astype(np.float32)


def quant_mxfp8(x):
    """-> (q [R, C] u8 e4m3 bits, scales [R, C/32] u8 e8m0 bits)."""
    x = _f32(x)
    r, c = x.shape
    assert c % 32 == 0
    q = np.empty((r, c), dtype=np.uint8)
    s = np.empty((r, c // 32), dtype=np.uint8)
    lib().oracle_quant_mxfp8(_p(x, c_float), r, c, _p(q, c_uint8), _p(s, c_uint8))
    return q, s


def dequant_mxfp8(q, s) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.uint8)
    s = np.ascontiguousarray(s, dtype=np.uint8)
    r, c = q.shape
    out = np.empty((r, c), dtype=np.float32)
    lib().oracle_dequant_mxfp8(_p(q, c_uint8), _p(s, c_uint8), r, c, _p(out, c_float))
    return out


# ---- scheduling -------------------------------------------------------------------------
def silu_mul(gate, up, is_f16: bool = False) -> np.ndarray:
    """`silu_mul_2d_f16` (cutile-kernels/src/pointwise.rs:63-75): 16-bit inputs widened to f32,
    sigmoid = 1 / (1 + exp(-gate)), y = sigmoid * gate * up, rounded to the 16-bit type."""
    g, u = _f32(gate), _f32(up)
    one = np.float32(1.0)
    sig = one / (one + np.exp(-g, dtype=np.float32))
    y = (sig * g * u).astype(np.float32)
    return y.astype(np.float16).astype(np.float32) if is_f16 else round_bf16(y)


def add_rms_norm(residual, x, w, eps: float, block_size: int = 512, is_f16: bool = True):
    """`add_rms_norm_f16` (cutile-kernels/src/norms.rs:77-137), and with ``residual=None``
    `rms_norm_f16` (:22-60).  16-bit inputs widened to f32; per row the squares are accumulated
    lane-wise over tiles of ``block_size`` columns (:100-108; overhang lanes read as zero), the lanes are
    summed (:109), inv = rsqrt(sum / N + eps) (:112-115), out = combined * inv * w and the updated
    residual = combined, both rounded to the 16-bit type (:126-134).  numpy's pairwise lane sum stands
    in for the tile reduction, whose order the compiler chooses.  Returns (out, residual_out or None)."""
    rnd = (lambda a: a.astype(np.float16).astype(np.float32)) if is_f16 else round_bf16
    xf, wf = _f32(x), _f32(w)
    comb = (_f32(residual) + xf).astype(np.float32) if residual is not None else xf
    rows, n = comb.shape
    tiles = (n + block_size - 1) // block_size
    pad = np.zeros((rows, tiles * block_size), dtype=np.float32)
    pad[:, :n] = comb
    lanes = np.zeros((rows, block_size), dtype=np.float32)
    for j in range(tiles):
        t = pad[:, j * block_size:(j + 1) * block_size]
        lanes = (lanes + t * t).astype(np.float32)
    ssum = lanes.sum(axis=1, dtype=np.float32)
    inv = (np.float32(1.0) / np.sqrt(ssum / np.float32(n) + np.float32(eps), dtype=np.float32)).astype(np.float32)
    out = rnd(((comb * inv[:, None]).astype(np.float32) * wf[None, :]).astype(np.float32))
    return out, (rnd(comb) if residual is not None else None)


def rope_seq(x, inv_freq, position_start: int, is_f16: bool = True) -> np.ndarray:
    """`rope_seq_f16` / `rope_seq_dynpos_f16` (cutile-kernels/src/positional.rs:20-62, 74-120): x
    [seq, heads, D] in the chunked layout, theta = f32(position_start + s) * inv_freq (:41-44), cos and sin
    in f32 (:46-47), y_lo = x_lo cos - x_hi sin, y_hi = x_hi cos + x_lo sin with every product and sum
    rounded to f32 (:49-50), results rounded to the 16-bit type (:51-52).  The angles are formed in f32 as the
    kernel does and their cos / sin taken in double precision and rounded, i.e. correctly rounded values."""
    rnd = (lambda a: a.astype(np.float16).astype(np.float32)) if is_f16 else round_bf16
    xf = _f32(x)
    seq, heads, d = xf.shape
    half = d // 2
    pos = (np.arange(seq, dtype=np.int64) + int(position_start)).astype(np.float32)
    theta = (pos[:, None] * _f32(inv_freq)[None, :]).astype(np.float32)
    cs = np.cos(theta.astype(np.float64)).astype(np.float32)[:, None, :]
    sn = np.sin(theta.astype(np.float64)).astype(np.float32)[:, None, :]
    lo, hi = xf[:, :, :half], xf[:, :, half:]
    y_lo = ((lo * cs).astype(np.float32) - (hi * sn).astype(np.float32)).astype(np.float32)
    y_hi = ((hi * cs).astype(np.float32) + (lo * sn).astype(np.float32)).astype(np.float32)
    return rnd(np.concatenate([y_lo, y_hi], axis=2))


def qk_norm_rope_kv(q, k, v, q_weight, k_weight, inv_freq, k_cache, v_cache, eps: float, position_start: int,
                    is_f16: bool = True):
    """`qk_norm_rope_kv_prefill_raw_f16` (cutile-kernels/src/experimental/fused_transformer.rs:145-344; the decode
    form :356 ff. is the same arithmetic on one row): per (position, head) the squares of the low and the high
    half are added lane-wise and summed (:184-186), inv = rsqrt(sum / D + eps) (:187-191), n = x * inv * w in f32
    (:240-241), then the rotation of `rope_seq` on n (:251-262) and one rounding to the 16-bit type (:263-264).
    Returns q_out; k_cache / v_cache (float arrays [kv_heads, MAX_SEQ, D]) are updated in place at rows
    position_start + s."""
    rnd = (lambda a: a.astype(np.float16).astype(np.float32)) if is_f16 else round_bf16
    seq = q.shape[0]
    half = q.shape[2] // 2
    pos = (np.arange(seq, dtype=np.int64) + int(position_start)).astype(np.float32)
    theta = (pos[:, None] * _f32(inv_freq)[None, :]).astype(np.float32)
    cs = np.cos(theta.astype(np.float64)).astype(np.float32)[:, None, :]
    sn = np.sin(theta.astype(np.float64)).astype(np.float32)[:, None, :]

    def one(x, w):
        xf, wf = _f32(x), _f32(w)
        lo, hi = xf[:, :, :half], xf[:, :, half:]
        ssum = ((lo * lo).astype(np.float32) + (hi * hi).astype(np.float32)).astype(np.float32).sum(axis=2, dtype=np.float32)
        inv = (np.float32(1.0) / np.sqrt(ssum / np.float32(2 * half) + np.float32(eps), dtype=np.float32))[:, :, None]
        nlo = ((lo * inv).astype(np.float32) * wf[None, None, :half]).astype(np.float32)
        nhi = ((hi * inv).astype(np.float32) * wf[None, None, half:]).astype(np.float32)
        ylo = ((nlo * cs).astype(np.float32) - (nhi * sn).astype(np.float32)).astype(np.float32)
        yhi = ((nhi * cs).astype(np.float32) + (nlo * sn).astype(np.float32)).astype(np.float32)
        return rnd(np.concatenate([ylo, yhi], axis=2))

    q_out = one(q, q_weight)
    k_rot = one(k, k_weight)
    for s_ in range(seq):
        k_cache[:, position_start + s_, :] = k_rot[s_]
        v_cache[:, position_start + s_, :] = _f32(v)[s_]
    return q_out


def argmax_blocks(logits, length: int, block_size: int):
    """`argmax_blocks_f16` (cutile-kernels/src/argmax.rs:27-68): per block the maximum of the logits widened to
    f32, positions >= len counting as -1e30 (:41-46), and the lowest index that attains it (:52-58)."""
    x = _f32(logits).reshape(-1)
    blocks = (length + block_size - 1) // block_size
    pad = np.full(blocks * block_size, np.float32(-1.0e30), dtype=np.float32)
    pad[:length] = x[:length]
    pad = pad.reshape(blocks, block_size)
    mx = pad.max(axis=1)
    idx = (pad == mx[:, None]).argmax(axis=1) + np.arange(blocks) * block_size
    return mx.astype(np.float32), idx.astype(np.uint32)


def lm_head_logits(weights, hidden) -> np.ndarray:
    """The logits of `lm_head_argmax_blocks_f16` (cutile-kernels/src/argmax.rs:103-114): per row, for every
    32-wide slice of K in order, the f32 products are summed and the partial sum is added to the accumulator."""
    w, h = _f32(weights), _f32(hidden).reshape(-1)
    acc = np.zeros(w.shape[0], dtype=np.float32)
    for kb in range(0, w.shape[1], 32):
        prod = (w[:, kb:kb + 32] * h[None, kb:kb + 32]).astype(np.float32)
        acc = (acc + prod.sum(axis=1, dtype=np.float32)).astype(np.float32)
    return acc


def argmax_reduce_blocks(block_max, block_idx, num_blocks: int) -> int:
    """`argmax_reduce_blocks_to_u32` (cutile-kernels/src/argmax.rs:169-198): the lowest block_idx among the
    blocks whose maximum equals the overall maximum."""
    bm = np.asarray(block_max, dtype=np.float32)[:num_blocks]
    bi = np.asarray(block_idx).astype(np.int64)[:num_blocks]
    return int(bi[bm == bm.max()].min())


def persistent_num_programs(m, n, bm, bn, num_sms, num_cta_in_cga, occupancy) -> int:
    return int(lib().oracle_persistent_num_programs(m, n, bm, bn, num_sms, num_cta_in_cga, occupancy))


def swizzled_bid(tile_id, num_bid_m, num_bid_n, group_size_m):
    a, b = c_int(), c_int()
    lib().oracle_swizzled_bid(tile_id, num_bid_m, num_bid_n, group_size_m, ctypes.byref(a),
                              ctypes.byref(b))
    return a.value, b.value


# ---- error metrics ----------------------------------------------------------------------
def rel_frobenius(got, ref) -> float:
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))


def max_abs(got, ref) -> float:
    return float(np.max(np.abs(np.asarray(got, dtype=np.float64) - np.asarray(ref, dtype=np.float64))))
