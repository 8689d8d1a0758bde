"""The C-ABI library loads and exports every symbol include/b200tile.h declares; host-only
validation paths answer with the documented codes (no GPU, no compute calls)."""
import ctypes
import os
import re

from cutile_rs_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200tile.h")).read()
    return sorted(set(re.findall(r"B200TILE_API\s+[\w\s\*]+?\b(b200tile_\w+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 10
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signatures and header declarations differ"
    lib = _lib.load()
    assert lib.b200tile_abi_version() == 1


def test_host_only_validation_codes():
    lib = _lib.load()
    grid = (ctypes.c_uint * 3)(1, 1, 1)
    params = (ctypes.c_void_p * 1)()
    rc = lib.b200tile_launch(b"no_such_kernel", None, 0, None, params, 0, grid, None)
    assert rc == _lib.ERR_UNSUPPORTED and b"unknown kernel" in lib.b200tile_last_error()
    gens = (ctypes.c_char_p * 4)(b"bf16", b"96", b"96", b"64")
    rc = lib.b200tile_launch(b"gemm", gens, 4, None, params, 0, grid, None)
    assert rc == _lib.ERR_UNSUPPORTED and b"no precompiled configuration" in lib.b200tile_last_error()
    gens = (ctypes.c_char_p * 4)(b"i8", b"128", b"256", b"64")
    assert lib.b200tile_launch(b"gemm", gens, 4, None, params, 0, grid, None) == _lib.ERR_UNSUPPORTED
    opts = _lib.CompileOptionsC(-1, 4, -1, -1)   # clusters of four: not in the fixed table
    gens = (ctypes.c_char_p * 4)(b"bf16", b"128", b"256", b"64")
    rc = lib.b200tile_launch(b"gemm", gens, 4, ctypes.byref(opts), params, 0, grid, None)
    assert rc == _lib.ERR_UNSUPPORTED and b"num_cta_in_cga" in lib.b200tile_last_error()
    rc = lib.b200tile_gemm(b"bf16", 0, 16, 16, 16, 1, 0, 8, 8, 8, 8, 8, 0, 0, 0, 0, -1, 0, 0, None)
    assert rc == _lib.ERR_INVALID and b"positive" in lib.b200tile_last_error()
    rc = lib.b200tile_gemm(b"bf16", 0, None, 16, 16, 1, 8, 8, 8, 8, 8, 8, 0, 0, 0, 0, -1, 0, 0, None)
    assert rc == _lib.ERR_INVALID
    I2 = ctypes.c_int64 * 2
    rc = lib.b200tile_fmha_fwd(b"bf16", 16, 16, 16, 16, 1, 3, 2, 128, 128, 128, I2(1, 1), I2(1, 1), I2(1, 1),
                               I2(1, 1), 1.0, 0, 0, None)
    assert rc == _lib.ERR_INVALID and b"multiple of heads_kv" in lib.b200tile_last_error()


def test_query_configs_lists_the_fixed_table():
    lib = _lib.load()
    arr = (_lib.ConfigC * 8)()
    n = lib.b200tile_query_configs(b"gemm", b"bf16", arr, 8)
    assert n >= 2 and (arr[0].bm, arr[0].bn, arr[0].bk) == (128, 256, 64)
    assert lib.b200tile_query_configs(b"gemm", b"f32", arr, 8) == 1
    assert lib.b200tile_query_configs(b"fmha", b"bf16", arr, 8) == 2   # one CTA per 256 rows; persistent CTA pairs, 256 rows per item
    assert (arr[0].num_cta_in_cga, arr[1].num_cta_in_cga) == (1, 2)
    assert lib.b200tile_query_configs(b"gemm", b"i4", arr, 8) == 0
    assert lib.b200tile_query_configs(b"unknown", b"bf16", arr, 8) == 0


def test_rust_sys_crate_declares_every_header_symbol():
    """rust/b200tile-sys/src/lib.rs is generated from the header: it must be up to date and name every export."""
    import subprocess
    import sys
    gen = os.path.join(ROOT, "rust", "b200tile-sys", "gen_ffi.py")
    assert subprocess.call([sys.executable, gen, "--check"]) == 0, "run rust/b200tile-sys/gen_ffi.py"
    rs = open(os.path.join(ROOT, "rust", "b200tile-sys", "src", "lib.rs")).read()
    assert sorted(set(re.findall(r"pub fn (b200tile_\w+)\(", rs))) == declared_symbols()
    assert lib_query_linear_tile() == (4, 1)   # NVFP4: three single-CTA tiles and the CTA-pair tile


def lib_query_linear_tile():
    lib = _lib.load()
    arr = (_lib.ConfigC * 8)()
    return (lib.b200tile_query_configs(b"linear_tile", b"f4e2m1fnx2", arr, 8),
            lib.b200tile_query_configs(b"linear_tile", b"f8e4m3fn", arr, 8))
