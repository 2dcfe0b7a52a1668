// rtxb_mxfp8_linear_fwd_noalloc: the quantize + GEMM forward for callers that
// cannot provide scratch memory.
//
// Some hosts of this library are handed nothing but their input and output
// buffers and have no allocator they are allowed to call: a generated wrapper
// that receives `(x, w, out=buf)`, a C plugin living inside another runtime's
// memory pool, or a latency-critical section in which cudaMalloc (which
// synchronises the whole device) is off limits.  For them the quantized
// operands and scale tiles, which every other entry point keeps in a
// caller-owned workspace, live here in one fixed array in device memory that is
// part of the library image.  Every GPU that loads the library carries the
// array until the process exits, so it is kept modest:
// RTXB_NOALLOC_SCRATCH_BYTES (32 MiB).
#include "../../include/rtxb.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

namespace rtxb {
int set_last_error(int code, const char* msg);   // api.cu: text behind rtxb_last_cuda_error()
}

namespace {

// The scratch itself.  In host code this name is only a handle for the runtime's
// symbol table, not a device address; the address each device maps it at is
// obtained with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[RTXB_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_address[kMaxDevices] = {nullptr};

// First call on a device: resolve that device's address of the array, with the
// device current.  Later calls on the same device reuse it.
int scratch_for_current_device(void** out) {
  char msg[192];
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    snprintf(msg, sizeof(msg), "cudaGetDevice: %s", cudaGetErrorString(e));
    return rtxb::set_last_error(RTXB_E_CUDA, msg);
  }
  if (dev < 0 || dev >= kMaxDevices) {
    snprintf(msg, sizeof(msg), "device index %d is outside the %d devices the no-allocation entry point tracks", dev,
             kMaxDevices);
    return rtxb::set_last_error(RTXB_E_UNSUPPORTED, msg);
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_address[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      snprintf(msg, sizeof(msg), "cudaGetSymbolAddress(scratch array) on device %d: %s", dev,
               e != cudaSuccess ? cudaGetErrorString(e) : "null address");
      return rtxb::set_last_error(RTXB_E_CUDA, msg);
    }
    g_scratch_address[dev] = ptr;
  }
  *out = g_scratch_address[dev];
  return RTXB_OK;
}

}  // namespace

extern "C" int rtxb_mxfp8_linear_fwd_noalloc(const void* x_bf16, const void* w_bf16, void* out_bf16, int64_t m,
                                             int64_t n, int64_t k, int rounding, void* stream, int* status) {
  if (!x_bf16 || !w_bf16 || !out_bf16) return rtxb::set_last_error(RTXB_E_INVALID_ARGUMENT, "null operand");
  if (m <= 0 || n <= 0 || k <= 0) return rtxb::set_last_error(RTXB_E_INVALID_ARGUMENT, "m, n, k must be positive");
  // The operands of this shape must fit the fixed array; nothing is launched otherwise.
  const size_t need = rtxb_mxfp8_linear_workspace_bytes(m, n, k);
  if (need > static_cast<size_t>(RTXB_NOALLOC_SCRATCH_BYTES)) {
    char msg[192];
    snprintf(msg, sizeof(msg), "this shape needs %zu bytes of quantized operands, the built-in array holds %d", need,
             RTXB_NOALLOC_SCRATCH_BYTES);
    return rtxb::set_last_error(RTXB_E_SCRATCH_CAPACITY, msg);
  }
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != RTXB_OK) return rc;
  // The array was looked up for the CURRENT device; a stream of another device would make the kernels run
  // there with this device's address.  The legacy and per-thread default streams belong to the current device.
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (s != nullptr && s != cudaStreamLegacy && s != cudaStreamPerThread) {
    int current = -1, of_stream = -1;
    if (cudaGetDevice(&current) == cudaSuccess && cudaStreamGetDevice(s, &of_stream) == cudaSuccess &&
        of_stream != current) {
      char msg[160];
      snprintf(msg, sizeof(msg), "the stream belongs to device %d but device %d is current", of_stream, current);
      return rtxb::set_last_error(RTXB_E_INVALID_ARGUMENT, msg);
    }
  }
  // Same kernels as rtxb_mxfp8_linear_fwd.  They overwrite every byte of the scratch they later
  // read (payload rows and whole scale tiles, padding included), so nothing has to be cleared even
  // though the array still holds the previous call's operands.
  return rtxb_mxfp8_linear_fwd(x_bf16, w_bf16, out_bf16, m, n, k, rounding, scratch,
                               static_cast<size_t>(RTXB_NOALLOC_SCRATCH_BYTES), stream, status);
}
