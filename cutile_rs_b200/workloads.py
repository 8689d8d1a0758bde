"""Seeded synthetic inputs for the benchmark configurations.

The reference has no dataset for this path (its examples draw from cuRAND or use constants), so
inputs are generated on the host from ``torch.Generator(cpu).manual_seed(0xC0FFEE00 + config)``
in fp32, rounded to the storage type on the host, and copied to the device bit-identically --
the kernels and the CPU oracle therefore see the same bits.
"""
from __future__ import annotations

import math
from typing import Tuple

import torch

SEED_BASE = 0xC0FFEE00


def _gen(config_index: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(SEED_BASE + int(config_index))


def gemm_f32_inputs(m: int = 512, n: int = 512, k: int = 512, config_index: int = 0
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Config 0: A, B ~ U[-1, 1] i.i.d. fp32, row-major."""
    g = _gen(config_index)
    a = torch.rand(m, k, generator=g, dtype=torch.float32) * 2.0 - 1.0
    b = torch.rand(k, n, generator=g, dtype=torch.float32) * 2.0 - 1.0
    return a, b


def gemm_bf16_inputs(m: int = 8192, n: int = 8192, k: int = 8192, config_index: int = 1
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Config 1: A[M,K], B[K,N] ~ N(0,1)/sqrt(K), rounded to bf16 (nearest even)."""
    g = _gen(config_index)
    s = 1.0 / math.sqrt(k)
    a = (torch.randn(m, k, generator=g, dtype=torch.float32) * s).to(torch.bfloat16)
    b = (torch.randn(k, n, generator=g, dtype=torch.float32) * s).to(torch.bfloat16)
    return a, b


def fmha_inputs(b: int = 8, h: int = 32, s: int = 4096, d: int = 128, h_kv: int = None,
                config_index: int = 2) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Config 2: Q (b,h,s,d), K and V (b,h_kv,s,d) ~ N(0,1), rounded to bf16."""
    g = _gen(config_index)
    h_kv = h if h_kv is None else h_kv
    q = torch.randn(b, h, s, d, generator=g, dtype=torch.float32).to(torch.bfloat16)
    k = torch.randn(b, h_kv, s, d, generator=g, dtype=torch.float32).to(torch.bfloat16)
    v = torch.randn(b, h_kv, s, d, generator=g, dtype=torch.float32).to(torch.bfloat16)
    return q, k, v


def gemm_normal_inputs(m: int, n: int, k: int, config_index: int
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Configs 3 and 4 before quantisation: A[M,K], B[N,K] (weights, K-major) ~ N(0,1), fp32."""
    g = _gen(config_index)
    a = torch.randn(m, k, generator=g, dtype=torch.float32)
    b = torch.randn(n, k, generator=g, dtype=torch.float32)
    return a, b


def gemm_flops(m: int, n: int, k: int) -> float:
    return 2.0 * m * n * k


def fmha_flops(b: int, h: int, s: int, d: int, causal: bool) -> float:
    """4*S^2*D*H*B, halved for causal (the reference's convention,
    cutile-benchmarks/benches/fmha_causal.rs:180)."""
    f = 4.0 * s * s * d * h * b
    return f / 2.0 if causal else f
