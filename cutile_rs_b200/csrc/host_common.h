// Host-side helpers shared by the translation units of libb200tile:
// thread-local error text, CUtensorMap encoding through the driver entry
// point (no link-time libcuda dependency), per-device facts and the device
// status record that bounded waits write into.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

// Status codes returned across the C ABI (see include/b200tile.h).
#define B200_OK 0
#define B200_ERR_INVALID 1      // argument violates a kernel precondition
#define B200_ERR_UNSUPPORTED 2  // unknown kernel / generics / config combination
#define B200_ERR_CUDA 3         // a CUDA runtime/driver call failed
#define B200_ERR_DEVICE 4       // device-side status word reported a problem
#define B200_ERR_ALIGN 5        // pointer/stride not usable by TMA (16-byte rules)

namespace b200h {

int set_error(int code, const char* fmt, ...);
const char* last_error();

// Encodes a rank-2 tiled tensor map.  dims/strides follow TMA convention:
// dim0 is the contiguous (innermost) extent; stride1_bytes is the pitch of dim1.
int encode_tmap_2d(CUtensorMap* out, CUtensorMapDataType dtype, int elem_bytes, const void* base,
                   uint64_t dim0, uint64_t dim1, uint64_t stride1_bytes, uint32_t box0,
                   uint32_t box1, CUtensorMapSwizzle swizzle);
// Rank-3 variant (dim2 outermost, stride2_bytes its pitch).
int encode_tmap_3d(CUtensorMap* out, CUtensorMapDataType dtype, int elem_bytes, const void* base,
                   uint64_t dim0, uint64_t dim1, uint64_t dim2, uint64_t stride1_bytes,
                   uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                   CUtensorMapSwizzle swizzle);

// Per-device first-use flag for idempotent set-up (function attributes).  Threads that race may both do
// the set-up, which is harmless because the calls are idempotent; the flag itself is atomic.
struct DeviceOnce {
  std::atomic<bool> done[64];
  bool test(int dev) const { return done[dev].load(std::memory_order_acquire); }
  void set(int dev) { done[dev].store(true, std::memory_order_release); }
};

// Per-device facts, resolved once per device on first use.
struct DeviceInfo {
  int ordinal;
  int sm_count;
  int cc_major, cc_minor;
  int max_smem_optin;
  uint32_t* status;  // device address of the 4-word status record
};
// Returns nullptr (and sets the error) when the current device is unusable.
const DeviceInfo* device_info();

// Library-owned scratch, one block per (device, stream), grown on demand and kept until process exit.
// Streams are told apart by cudaStreamGetId (never reused within a process); inside a stream capture,
// where that query and every allocation are illegal, a block is found by the stream handle it was
// created under, and a missing or too-small block is an error.  Returns nullptr with the error set.
// Work enqueued on one stream is ordered, so consecutive launches may share the block.
void* stream_scratch(cudaStream_t stream, size_t bytes, const char* who);

#define B200_CUDA_CHECK(expr)                                                              \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess)                                                                 \
      return b200h::set_error(B200_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

}  // namespace b200h
