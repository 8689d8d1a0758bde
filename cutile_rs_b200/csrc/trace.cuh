// Optional cycle accounting for the single-thread roles of the kernels (TMA, MMA, one softmax lane).
// A normal build compiles all of this away.  A diagnostic build (-DB200TILE_TRACE, e.g.
// B200_NVCC_EXTRA=-DB200TILE_TRACE csrc/build.sh) accumulates clock64() differences per phase in
// registers and lets one chosen CTA write them to a per-kernel device array, which
// b200tile_trace_read() copies out.  The extra clock reads cost a few percent, so the phase
// SHARES are what the numbers are good for.
#pragma once
#ifdef B200TILE_TRACE
#define B200_TR_DECL(n) long long tr_[n] = {}; long long tr_a_ = 0; const long long tr_t0_ = clock64()
#define B200_TR_BEGIN() tr_a_ = clock64()
#define B200_TR_END(i) tr_[i] += clock64() - tr_a_
#define B200_TR_COUNT(i) tr_[i] += 1
#define B200_TR_FLUSH(dst, n, cond)                       \
  if (cond) {                                             \
    for (int i_ = 0; i_ < (n); ++i_) (dst)[i_] = tr_[i_]; \
    (dst)[n] = clock64() - tr_t0_;                        \
  }
#else
#define B200_TR_DECL(n)
#define B200_TR_BEGIN()
#define B200_TR_END(i)
#define B200_TR_COUNT(i)
#define B200_TR_FLUSH(dst, n, cond)
#endif
