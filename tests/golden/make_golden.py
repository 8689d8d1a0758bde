"""Generates the committed golden fixtures of tests/golden/ (run from the repo root).

The reference cannot be built or run in this environment (no Rust toolchain, no `tileiras`), so
the fixtures restate, in float64 numpy, the inputs and expected outputs of the reference's own
checks:
  * persistent_gemm_64x64x32.npy -- cutile-examples/examples/persistent_gemm.rs:89-94,140-152,
    evaluated with separately rounded float32 products and sums in ascending k.
  * fmha_causal_pos5.npz -- the shape of cutile-examples/examples/flash_attention_causal.rs:216-223
    (2 x 8 x 64 x 32, input_pos = 5) on seeded normal inputs (the example draws from cuRAND, which
    cannot be reproduced), expected output from the softmax definition in float64.
"""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    m, n, k = 64, 64, 32
    x = np.array([[((r % 7) - 3.0) * 0.25 + (c % 5) * 0.125 for c in range(k)] for r in range(m)], np.float32)
    y = np.array([[((r % 3) + 1.0) * 0.2 - (c % 11) * 0.05 for c in range(n)] for r in range(k)], np.float32)
    z = np.zeros((m, n), np.float32)
    for i in range(m):
        for j in range(n):
            acc = np.float32(0.0)
            for t in range(k):
                acc = np.float32(acc + np.float32(x[i, t] * y[t, j]))
            z[i, j] = acc
    np.save(os.path.join(HERE, "persistent_gemm_64x64x32.npy"), z)

    rng = np.random.default_rng(20240605)
    b, h, s, d = 2, 8, 64, 32
    q = rng.normal(size=(b, h, s, d)).astype(np.float32)
    kk = rng.normal(size=(b, h, s, d)).astype(np.float32)
    v = rng.normal(size=(b, h, s, d)).astype(np.float32)
    scale = 1.0 / np.sqrt(d)
    sc = np.einsum("bhid,bhjd->bhij", q.astype(np.float64), kk.astype(np.float64)) * scale
    i, j = np.arange(s)[:, None], np.arange(s)[None, :]
    sc = np.where(j > i + 5, -np.inf, sc)
    p = np.exp(sc - sc.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    out = np.einsum("bhij,bhjd->bhid", p, v.astype(np.float64)).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "fmha_causal_pos5.npz"), q=q, k=kk, v=v, out=out,
                        scale=np.float32(scale))


if __name__ == "__main__":
    main()
