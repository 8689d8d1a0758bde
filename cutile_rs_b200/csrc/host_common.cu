#include "host_common.h"

#include <cudaTypedefs.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

namespace b200h {

// ---------------------------------------------------------------------------
// Thread-local error text (the C ABI never throws).
// ---------------------------------------------------------------------------
static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
const char* last_error() { return g_err; }

// ---------------------------------------------------------------------------
// cuTensorMapEncodeTiled through the runtime's driver-entry-point lookup.
// ---------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

static int check_tma_rules(const void* base, const uint64_t* strides_bytes, int nstrides) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0)
    return set_error(B200_ERR_ALIGN, "tensor base %p is not 16-byte aligned (TMA requirement)",
                     base);
  for (int i = 0; i < nstrides; ++i)
    if (strides_bytes[i] % 16 != 0)
      return set_error(B200_ERR_ALIGN,
                       "tensor pitch of %llu bytes is not a multiple of 16 (TMA requirement)",
                       (unsigned long long)strides_bytes[i]);
  return B200_OK;
}

int encode_tmap_2d(CUtensorMap* out, CUtensorMapDataType dtype, int elem_bytes, const void* base,
                   uint64_t dim0, uint64_t dim1, uint64_t stride1_bytes, uint32_t box0,
                   uint32_t box1, CUtensorMapSwizzle swizzle) {
  auto fn = get_encode_fn();
  if (!fn) return set_error(B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  uint64_t strides[1] = {stride1_bytes};
  if (int rc = check_tma_rules(base, strides, 1)) return rc;
  (void)elem_bytes;
  cuuint64_t gdim[2] = {dim0, dim1};
  cuuint64_t gstr[1] = {stride1_bytes};
  cuuint32_t box[2] = {box0, box1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dtype, 2, const_cast<void*>(base), gdim, gstr, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(B200_ERR_CUDA,
                     "cuTensorMapEncodeTiled(2d) failed with CUresult %d (dims %llu x %llu, pitch "
                     "%llu, box %u x %u)",
                     (int)r, (unsigned long long)dim0, (unsigned long long)dim1,
                     (unsigned long long)stride1_bytes, box0, box1);
  return B200_OK;
}

int encode_tmap_3d(CUtensorMap* out, CUtensorMapDataType dtype, int elem_bytes, const void* base,
                   uint64_t dim0, uint64_t dim1, uint64_t dim2, uint64_t stride1_bytes,
                   uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                   CUtensorMapSwizzle swizzle) {
  auto fn = get_encode_fn();
  if (!fn) return set_error(B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  uint64_t strides[2] = {stride1_bytes, stride2_bytes};
  if (int rc = check_tma_rules(base, strides, 2)) return rc;
  (void)elem_bytes;
  cuuint64_t gdim[3] = {dim0, dim1, dim2};
  cuuint64_t gstr[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dtype, 3, const_cast<void*>(base), gdim, gstr, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(B200_ERR_CUDA, "cuTensorMapEncodeTiled(3d) failed with CUresult %d", (int)r);
  return B200_OK;
}

// ---------------------------------------------------------------------------
// Device status record + per-device facts.
// ---------------------------------------------------------------------------
__device__ uint32_t g_device_status[4];

static DeviceInfo g_info[64];
static bool g_info_ok[64];
static std::mutex g_info_mu;

const DeviceInfo* device_info() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error(B200_ERR_CUDA, "no usable CUDA device is current");
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_info_mu);
  if (g_info_ok[dev]) return &g_info[dev];
  DeviceInfo& d = g_info[dev];
  d.ordinal = dev;
  cudaError_t e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev);
  if (e == cudaSuccess)
    e = cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  void* sp = nullptr;
  if (e == cudaSuccess) e = cudaGetSymbolAddress(&sp, g_device_status);
  if (e != cudaSuccess) {
    set_error(B200_ERR_CUDA, "device query failed: %s", cudaGetErrorString(e));
    return nullptr;
  }
  if (d.cc_major != 10) {
    set_error(B200_ERR_UNSUPPORTED,
              "device %d is sm_%d%d; this library only contains sm_100a code", dev, d.cc_major,
              d.cc_minor);
    return nullptr;
  }
  d.status = static_cast<uint32_t*>(sp);
  g_info_ok[dev] = true;
  return &d;
}

// ---------------------------------------------------------------------------
// Per-(device, stream) scratch blocks.
// ---------------------------------------------------------------------------
namespace {
struct ScratchBlock {
  unsigned long long stream_id;
  cudaStream_t handle;
  bool handle_live;   // false once another stream has been seen under the same handle
  void* ptr;
  size_t bytes;
  bool used;
};
constexpr int kScratchPerDevice = 16;
ScratchBlock g_scratch[64][kScratchPerDevice];
std::mutex g_scratch_mu;
}  // namespace

void* stream_scratch(cudaStream_t stream, size_t bytes, const char* who) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error(B200_ERR_CUDA, "%s: no usable CUDA device is current", who);
    return nullptr;
  }
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess) {
    cudaGetLastError();
    set_error(B200_ERR_CUDA, "%s: cudaStreamIsCapturing failed", who);
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  ScratchBlock* tab = g_scratch[dev];
  if (cs != cudaStreamCaptureStatusNone) {
    for (int i = 0; i < kScratchPerDevice; ++i)
      if (tab[i].used && tab[i].handle_live && tab[i].handle == stream && tab[i].bytes >= bytes) return tab[i].ptr;
    set_error(B200_ERR_INVALID,
              "%s: needs %llu bytes of library scratch, which cannot be allocated inside a stream capture; run the "
              "call once on this stream before capturing, or use the entry point that takes a workspace",
              who, (unsigned long long)bytes);
    return nullptr;
  }
  unsigned long long id = 0;
  if (cudaStreamGetId(stream, &id) != cudaSuccess) {
    cudaGetLastError();
    set_error(B200_ERR_CUDA, "%s: cudaStreamGetId failed", who);
    return nullptr;
  }
  ScratchBlock* e = nullptr;
  for (int i = 0; i < kScratchPerDevice && !e; ++i)
    if (tab[i].used && tab[i].stream_id == id) e = &tab[i];
  if (e && e->bytes >= bytes) return e->ptr;
  if (!e)
    for (int i = 0; i < kScratchPerDevice && !e; ++i)
      if (!tab[i].used) e = &tab[i];
  if (!e) {
    set_error(B200_ERR_INVALID, "%s: all %d scratch blocks of this device belong to other streams; use the entry "
              "point that takes a workspace", who, kScratchPerDevice);
    return nullptr;
  }
  if (e->used) {
    // grow: earlier launches of this stream may still read the old block
    if (cudaStreamSynchronize(stream) != cudaSuccess || cudaFree(e->ptr) != cudaSuccess) {
      set_error(B200_ERR_CUDA, "%s: could not release the old scratch block", who);
      return nullptr;
    }
    e->used = false;
  }
  const size_t grow = bytes < (size_t(1) << 20) ? (size_t(1) << 20) : bytes + bytes / 2;
  void* p = nullptr;
  if (cudaMalloc(&p, grow) != cudaSuccess) {
    cudaGetLastError();
    set_error(B200_ERR_CUDA, "%s: cudaMalloc of %llu scratch bytes failed", who, (unsigned long long)grow);
    return nullptr;
  }
  e->stream_id = id;
  e->handle = stream;
  e->handle_live = true;
  e->ptr = p;
  e->bytes = grow;
  e->used = true;
  for (int j = 0; j < kScratchPerDevice; ++j)
    if (&tab[j] != e && tab[j].used && tab[j].handle == stream) tab[j].handle_live = false;
  return p;
}

}  // namespace b200h
