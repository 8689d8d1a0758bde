// Optional cycle accounting for the single-thread roles of the kernels (TMA, MMA, one softmax lane).
// A normal build compiles all of this away.  A diagnostic build (-DB200TILE_TRACE, e.g.
// B200_NVCC_EXTRA=-DB200TILE_TRACE csrc/build.sh) accumulates clock64() differences per phase in
// registers and lets one chosen CTA write them to a per-kernel device array, which
// b200tile_trace_read() copies out.  The extra clock reads cost a few percent, so the phase
// SHARES are what the numbers are good for.  The slot after the total holds the same span in
// nanoseconds of the global timer: cycles / ns is the SM clock the kernel really ran at.
#pragma once
#ifdef B200TILE_TRACE
__device__ __forceinline__ long long b200_globaltimer_ns() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define B200_TR_DECL(n) long long tr_[n] = {}; long long tr_a_ = 0; const long long tr_t0_ = clock64(); \
  const long long tr_ns0_ = b200_globaltimer_ns()
#define B200_TR_BEGIN() tr_a_ = clock64()
#define B200_TR_END(i) tr_[i] += clock64() - tr_a_
#define B200_TR_COUNT(i) tr_[i] += 1
#define B200_TR_FLUSH(dst, n, cond)                       \
  if (cond) {                                             \
    for (int i_ = 0; i_ < (n); ++i_) (dst)[i_] = tr_[i_]; \
    (dst)[n] = clock64() - tr_t0_;                        \
    (dst)[(n) + 1] = b200_globaltimer_ns() - tr_ns0_;     \
  }
#else
#define B200_TR_DECL(n)
#define B200_TR_BEGIN()
#define B200_TR_END(i)
#define B200_TR_COUNT(i)
#define B200_TR_FLUSH(dst, n, cond)
#endif
