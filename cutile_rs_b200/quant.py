"""Block quantisers for the low-precision GEMM inputs (torch, any device).

These produce the operand formats the block-scaled kernels consume; they are input preparation,
not part of a kernel.  Bit conventions: f8e4m3fn and packed f4e2m1fnx2 (low nibble first) as in
cuda-core/src/dtype.rs:25-31,60-110.
"""
from __future__ import annotations

from typing import Tuple

import torch


def quant_fp8_block(x: torch.Tensor, block_r: int, block_c: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """e4m3 with one fp32 scale per (block_r x block_c) block: scale = blockmax / 448 (1 for an
    all-zero block), q = round-to-nearest-even(x / scale).  Returns (q as uint8 bits, scales)."""
    r, c = x.shape
    assert r % block_r == 0 and c % block_c == 0, "shape must be a multiple of the scale block"
    xb = x.float().reshape(r // block_r, block_r, c // block_c, block_c)
    amax = xb.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    q = (xb / scale[:, None, :, None]).reshape(r, c).to(torch.float8_e4m3fn)
    return q.view(torch.uint8), scale.contiguous()


_E2M1_BOUNDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)   # round-to-nearest-even decision points
_E2M1_TIE_UP = (False, True, False, True, False, True, False)  # at a tie, go up iff the upper code is even


def _to_e2m1_codes(a: torch.Tensor) -> torch.Tensor:
    """|value| -> 3-bit magnitude code on the grid 0, .5, 1, 1.5, 2, 3, 4, 6 (ties to even mantissa)."""
    code = torch.zeros_like(a, dtype=torch.uint8)
    for bound, tie_up in zip(_E2M1_BOUNDS, _E2M1_TIE_UP):
        code += ((a >= bound) if tie_up else (a > bound)).to(torch.uint8)
    return code


def quant_nvfp4(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, float]:
    """NVFP4: global fp32 scale g = amax/(6*448); per 16 contiguous K elements an e4m3 scale
    s = e4m3(blockmax/(6 g)); q = e2m1(x / (s g)).  Returns (packed [R, C/2] uint8, scales [R, C/16]
    uint8 holding e4m3 bits, g)."""
    r, c = x.shape
    assert c % 16 == 0
    xf = x.float()
    amax = xf.abs().max()
    g = float(amax / (6.0 * 448.0)) if float(amax) > 0 else 1.0
    xb = xf.reshape(r, c // 16, 16)
    bmax = xb.abs().amax(dim=2)
    sb = (bmax / (6.0 * g)).to(torch.float8_e4m3fn)
    s = sb.float() * g
    y = torch.where(s[:, :, None] > 0, xb / s[:, :, None], torch.zeros_like(xb))
    code = _to_e2m1_codes(y.abs()) | ((y < 0) | ((y == 0) & torch.signbit(y))).to(torch.uint8) * 8
    code = code.reshape(r, c)
    packed = (code[:, 0::2] & 0xF) | ((code[:, 1::2] & 0xF) << 4)
    return packed.contiguous(), sb.view(torch.uint8).contiguous(), g


def quant_mxfp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """MXFP8: e4m3 values with one e8m0 (power-of-two) scale per 32 contiguous K elements; the scale
    is the smallest power of two with blockmax/scale <= 448.  Returns (q uint8 [R,C], scales uint8
    [R,C/32] holding the biased exponent)."""
    r, c = x.shape
    assert c % 32 == 0
    xb = x.float().reshape(r, c // 32, 32)
    amax = xb.abs().amax(dim=2)
    mant, exp = torch.frexp(amax / 448.0)           # amax/448 = mant * 2^exp, mant in [0.5, 1)
    e = torch.where(mant == 0.5, exp - 1, exp)
    e = torch.where(amax > 0, e, torch.zeros_like(e)).clamp(-127, 127)
    scale = torch.ldexp(torch.ones_like(amax), e)
    q = (xb / scale[:, :, None]).reshape(r, c).to(torch.float8_e4m3fn)
    return q.view(torch.uint8), (e + 127).to(torch.uint8).contiguous()


def quant_mxfp4(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """MXFP4: e2m1 values with one e8m0 (power-of-two) scale per 32 contiguous K elements; the scale is the
    smallest power of two with blockmax/scale <= 6.  Returns (packed [R, C/2] uint8, low nibble first; scales
    uint8 [R, C/32] holding the biased exponent)."""
    r, c = x.shape
    assert c % 32 == 0
    xb = x.float().reshape(r, c // 32, 32)
    amax = xb.abs().amax(dim=2)
    mant, exp = torch.frexp(amax / 6.0)             # amax/6 = mant * 2^exp, mant in [0.5, 1)
    e = torch.where(mant == 0.5, exp - 1, exp)
    e = torch.where(amax > 0, e, torch.zeros_like(e)).clamp(-127, 127)
    scale = torch.ldexp(torch.ones_like(amax), e)
    y = xb / scale[:, :, None]
    code = _to_e2m1_codes(y.abs()) | ((y < 0) | ((y == 0) & torch.signbit(y))).to(torch.uint8) * 8
    code = code.reshape(r, c)
    packed = (code[:, 0::2] & 0xF) | ((code[:, 1::2] & 0xF) << 4)
    return packed.contiguous(), (e + 127).to(torch.uint8).contiguous()
