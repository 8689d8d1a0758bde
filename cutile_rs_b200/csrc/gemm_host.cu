// GEMM with HOST operands: upload, multiply and download as one software pipeline.
//
// The reference user writes `copy_host_vec_to_device` (cutile/src/api.rs:422) for both operands,
// launches the kernel and reads the result with `copy_device_to_host_vec` (api.rs:371): three
// serial phases on one stream, of which the PCIe transfers take ten times longer than the
// multiplication at 8192^3.  Here the B operand goes up first, A follows in row slabs, every slab
// is multiplied as soon as it has arrived and its C rows travel back while the next slab is
// still coming in: uploads, tensor-core work and downloads overlap on three streams, and the
// elapsed time approaches the larger of (bytes up, bytes down) / link bandwidth.
//
// Nothing is allocated on the device: the caller passes the device staging buffers.  Two
// non-blocking streams and a pool of events are created once per device.
#include "../../include/b200tile.h"
#include <string.h>

#include <mutex>

#include "host_common.h"

namespace {

constexpr int kMaxSlabs = 64;

struct HostPipe {
  bool ready = false;
  cudaStream_t s_in = nullptr, s_out = nullptr;
  cudaEvent_t start = nullptr, b_up = nullptr, done = nullptr;
  cudaEvent_t a_up[kMaxSlabs] = {}, c_ready[kMaxSlabs] = {};
};

HostPipe g_pipes[64];
// One pipe (two side streams, one set of events) per device, shared by every caller: the whole enqueue
// sequence of a call holds the device's lock, so that two host threads cannot interleave their records
// and waits on the same events.  The work itself is asynchronous; the lock is held for microseconds.
std::mutex g_pipe_mu[64];

int get_pipe(int ordinal, HostPipe** out) {
  HostPipe& p = g_pipes[ordinal];
  if (!p.ready) {
    B200_CUDA_CHECK(cudaStreamCreateWithFlags(&p.s_in, cudaStreamNonBlocking));
    B200_CUDA_CHECK(cudaStreamCreateWithFlags(&p.s_out, cudaStreamNonBlocking));
    B200_CUDA_CHECK(cudaEventCreateWithFlags(&p.start, cudaEventDisableTiming));
    B200_CUDA_CHECK(cudaEventCreateWithFlags(&p.b_up, cudaEventDisableTiming));
    B200_CUDA_CHECK(cudaEventCreateWithFlags(&p.done, cudaEventDisableTiming));
    for (int i = 0; i < kMaxSlabs; ++i) {
      B200_CUDA_CHECK(cudaEventCreateWithFlags(&p.a_up[i], cudaEventDisableTiming));
      B200_CUDA_CHECK(cudaEventCreateWithFlags(&p.c_ready[i], cudaEventDisableTiming));
    }
    p.ready = true;
  }
  *out = &p;
  return B200_OK;
}

}  // namespace

extern "C" int b200tile_gemm_host(const char* dtype, int b_layout, const void* a_host, const void* b_host,
                                  void* c_host, void* a_dev, void* b_dev, void* c_dev, int m, int n, int k,
                                  int slab_rows, void* cu_stream) {
  using b200h::set_error;
  if (!dtype || !a_host || !b_host || !c_host || !a_dev || !b_dev || !c_dev)
    return set_error(B200_ERR_INVALID, "gemm_host: null argument");
  if (m <= 0 || n <= 0 || k <= 0) return set_error(B200_ERR_INVALID, "gemm_host: Shape dimensions must be positive");
  size_t es;
  if (!strcmp(dtype, "bf16") || !strcmp(dtype, "f16")) es = 2;
  else if (!strcmp(dtype, "f32")) es = 4;
  else return set_error(B200_ERR_UNSUPPORTED, "gemm_host: unsupported element type '%s'", dtype);
  const b200h::DeviceInfo* di = b200h::device_info();
  if (!di) return B200_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(cu_stream);
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  B200_CUDA_CHECK(cudaStreamIsCapturing(s, &cap));
  if (cap != cudaStreamCaptureStatusNone)
    return set_error(B200_ERR_UNSUPPORTED, "gemm_host: not available inside a stream capture");
  if (slab_rows <= 0) slab_rows = 1024;
  slab_rows = (slab_rows + 255) / 256 * 256;
  int slabs = (m + slab_rows - 1) / slab_rows;
  if (slabs > kMaxSlabs) {
    slab_rows = ((m + kMaxSlabs - 1) / kMaxSlabs + 255) / 256 * 256;
    slabs = (m + slab_rows - 1) / slab_rows;
  }
  std::lock_guard<std::mutex> lk(g_pipe_mu[di->ordinal]);
  HostPipe* p;
  if (int rc = get_pipe(di->ordinal, &p)) return rc;

  // Whatever has been queued on the side streams when this function returns -- normally the whole pipeline,
  // after an error a prefix of it -- is joined to the caller's stream, so that synchronising that stream always
  // covers every copy that still touches the caller's buffers.
  auto join = [&]() {
    if (cudaEventRecord(p->b_up, p->s_in) == cudaSuccess) cudaStreamWaitEvent(s, p->b_up, 0);
    if (cudaEventRecord(p->done, p->s_out) == cudaSuccess) cudaStreamWaitEvent(s, p->done, 0);
  };
  auto enqueue = [&]() -> int {
    // everything queued on the caller's stream so far comes first (it may still use the staging buffers)
    B200_CUDA_CHECK(cudaEventRecord(p->start, s));
    B200_CUDA_CHECK(cudaStreamWaitEvent(p->s_in, p->start, 0));
    B200_CUDA_CHECK(cudaStreamWaitEvent(p->s_out, p->start, 0));
    B200_CUDA_CHECK(cudaMemcpyAsync(b_dev, b_host, (size_t)n * k * es, cudaMemcpyHostToDevice, p->s_in));
    B200_CUDA_CHECK(cudaEventRecord(p->b_up, p->s_in));
    B200_CUDA_CHECK(cudaStreamWaitEvent(s, p->b_up, 0));
    const int64_t ldb = b_layout ? k : n;
    for (int i = 0; i < slabs; ++i) {
      const int r0 = i * slab_rows;
      const int rows = (m - r0) < slab_rows ? (m - r0) : slab_rows;
      const size_t a_off = (size_t)r0 * k * es, c_off = (size_t)r0 * n * es;
      B200_CUDA_CHECK(cudaMemcpyAsync(static_cast<char*>(a_dev) + a_off, static_cast<const char*>(a_host) + a_off,
                                      (size_t)rows * k * es, cudaMemcpyHostToDevice, p->s_in));
      B200_CUDA_CHECK(cudaEventRecord(p->a_up[i], p->s_in));
      B200_CUDA_CHECK(cudaStreamWaitEvent(s, p->a_up[i], 0));
      if (int rc = b200tile_gemm(dtype, b_layout, static_cast<char*>(a_dev) + a_off, b_dev,
                                 static_cast<char*>(c_dev) + c_off, 1, rows, n, k, k, ldb, n, 0, 0, 0, 0, -1, 0, 0, s))
        return rc;
      B200_CUDA_CHECK(cudaEventRecord(p->c_ready[i], s));
      B200_CUDA_CHECK(cudaStreamWaitEvent(p->s_out, p->c_ready[i], 0));
      B200_CUDA_CHECK(cudaMemcpyAsync(static_cast<char*>(c_host) + c_off, static_cast<char*>(c_dev) + c_off,
                                      (size_t)rows * n * es, cudaMemcpyDeviceToHost, p->s_out));
    }
    return B200_OK;
  };
  const int rc = enqueue();
  // the caller's stream ends after the last download: synchronising it covers the whole call
  join();
  return rc;
}
