"""ctypes binding of ``libb200tile.so`` (declared in ``include/b200tile.h``).

The library holds sm_100a machine code only.  There is no fallback: when the
shared object is missing or cannot be loaded, importing callers get a
``RuntimeError`` that says how to build it.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, Structure, c_char_p, c_float, c_int, c_int64, c_uint, c_uint32,
                    c_uint64, c_void_p)

_HERE = os.path.dirname(os.path.abspath(__file__))
# B200TILE_LIB selects another build of the same library (the diagnostic trace build)
LIB_PATH = os.environ.get("B200TILE_LIB") or os.path.join(_HERE, "libb200tile.so")

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_DEVICE, ERR_ALIGN = range(6)


class CompileOptionsC(Structure):
    _fields_ = [("occupancy", c_int), ("num_cta_in_cga", c_int), ("max_divisibility", c_int),
                ("num_worker_warps_per_cta", c_int)]


class ConfigC(Structure):
    _fields_ = [("id", c_int), ("bm", c_int), ("bn", c_int), ("bk", c_int), ("stages", c_int),
                ("num_cta_in_cga", c_int), ("occupancy", c_int)]


class StatusC(Structure):
    _fields_ = [("code", c_uint32), ("block", c_uint32), ("site", c_uint32), ("aux", c_uint32)]


# name -> (restype, argtypes); the single source of truth for the Python side of the ABI.
SIGNATURES = {
    "b200tile_abi_version": (c_int, []),
    "b200tile_init": (c_int, [c_int]),
    "b200tile_last_error": (c_char_p, []),
    "b200tile_num_sms": (c_int, []),
    "b200tile_status": (c_int, [c_void_p, POINTER(StatusC)]),
    "b200tile_status_reset": (c_int, [c_void_p]),
    "b200tile_query_configs": (c_int, [c_char_p, c_char_p, POINTER(ConfigC), c_int]),
    "b200tile_launch": (c_int, [c_char_p, POINTER(c_char_p), c_int, POINTER(CompileOptionsC),
                                POINTER(c_void_p), c_int, POINTER(c_uint), c_void_p]),
    "b200tile_prepare": (c_int, [c_char_p, POINTER(c_char_p), c_int, POINTER(CompileOptionsC)]),
    "b200tile_gemm": (c_int, [c_char_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                              c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int,
                              c_int, c_int, c_int, c_void_p]),
    "b200tile_gemm_host": (c_int, [c_char_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_int, c_int, c_int, c_int, c_void_p]),
    "b200tile_linear_swiglu": (c_int, [c_char_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64,
                                       c_int64, c_void_p]),
    "b200tile_rms_norm": (c_int, [c_char_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_float,
                                  c_void_p]),
    "b200tile_add_rms_norm": (c_int, [c_char_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                      c_int64, c_int64, c_int64, c_int64, c_float, c_void_p]),
    "b200tile_rope_seq": (c_int, [c_char_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, POINTER(c_int64),
                                  POINTER(c_int64), c_int, c_void_p, c_void_p]),
    "b200tile_qk_norm_rope_kv": (c_int, [c_char_p] + [c_void_p] * 9 + [c_float, c_int, c_void_p, c_int, c_int, c_int,
                                                                       c_int, c_int, c_int64, c_int64, c_int64,
                                                                       c_int64, c_void_p]),
    "b200tile_argmax_blocks": (c_int, [c_char_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "b200tile_lm_head_argmax_blocks": (c_int, [c_char_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64,
                                               c_void_p]),
    "b200tile_argmax_reduce_blocks": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "b200tile_add_2d": (c_int, [c_char_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64,
                                c_void_p]),
    "b200tile_silu_mul_2d": (c_int, [c_char_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64,
                                     c_void_p]),
    "b200tile_linear_bias_residual": (c_int, [c_char_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                              c_int, c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "b200tile_group_gemm_workspace_bytes": (c_uint64, [c_int]),
    "b200tile_group_gemm": (c_int, [c_char_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                    c_int, c_void_p, c_uint64, c_void_p]),
    "b200tile_fmha_fwd": (c_int, [c_char_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                  c_int, c_int, c_int, c_int, POINTER(c_int64), POINTER(c_int64),
                                  POINTER(c_int64), POINTER(c_int64), c_float, c_int, c_int,
                                  c_void_p]),
    "b200tile_fmha_fwd_dynpos": (c_int, [c_char_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                         c_int, c_int, c_int, c_int, POINTER(c_int64), POINTER(c_int64),
                                         POINTER(c_int64), POINTER(c_int64), c_float, c_int, c_void_p,
                                         c_void_p]),
    "b200tile_fmha_decode_gqa_split": (c_int, [c_char_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                               c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                               c_float, POINTER(c_int64), POINTER(c_int64), POINTER(c_int64),
                                               POINTER(c_int64), c_int64, POINTER(c_int64), c_void_p]),
    "b200tile_splitk_reduce_merge": (c_int, [c_char_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                             POINTER(c_int64), c_int64, POINTER(c_int64), c_void_p]),
    "b200tile_linear_fp8_blk128": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_char_p,
                                           c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int64,
                                           c_int64, c_float, c_void_p]),
    "b200tile_linear_nvfp4_workspace_bytes": (c_uint64, [c_int, c_int, c_int]),
    "b200tile_linear_nvfp4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_char_p, c_int,
                                      c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_float,
                                      c_void_p, c_uint64, c_int, c_void_p]),
    "b200tile_nvfp4_weight_scales_bytes": (c_uint64, [c_int, c_int, c_int]),
    "b200tile_nvfp4_register_weight_scales": (c_int, [c_void_p, c_int, c_int, c_int64, c_int, c_void_p]),
    "b200tile_nvfp4_unregister_weight_scales": (c_int, [c_void_p]),
    "b200tile_nvfp4_prepare_weight_scales": (c_int, [c_void_p, c_int, c_int, c_int64, c_int, c_void_p, c_uint64,
                                                     c_void_p]),
    "b200tile_linear_nvfp4_prepared": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_char_p, c_int,
                                               c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_float, c_int,
                                               c_void_p]),
    "b200tile_linear_mxfp8_workspace_bytes": (c_uint64, [c_int, c_int, c_int]),
    "b200tile_linear_mxfp8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_char_p, c_int,
                                      c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_float,
                                      c_void_p, c_uint64, c_void_p]),
    "b200tile_linear_mxfp4_workspace_bytes": (c_uint64, [c_int, c_int, c_int]),
    "b200tile_linear_mxfp4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_char_p, c_int,
                                      c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_float,
                                      c_void_p, c_uint64, c_void_p]),
    "b200tile_linear_nvfp4_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_char_p,
                                             c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int64,
                                             c_int64, c_float, c_int, c_void_p]),
}

_lib = None


class B200TileError(RuntimeError):
    """A non-zero status from the C ABI; ``code`` is the ``B200TILE_ERR_*`` value."""

    def __init__(self, code: int, message: str):
        super().__init__(f"b200tile error {code}: {message}")
        self.code = code
        self.message = message


def load() -> ctypes.CDLL:
    """Loads the shared library once and attaches the declared signatures."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with cutile_rs_b200/csrc/build.sh "
            "(or `python -c 'import __graft_entry__ as g; g.build()'`). There is no CPU fallback.")
    lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError when the header and the binary disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != OK:
        raise B200TileError(rc, load().b200tile_last_error().decode("utf-8", "replace"))
