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

#include <mutex>

namespace {

// The scratch itself.  In host code this name is only a handle for the runtime's
// symbol table, not a device address; the address each device maps it at is
// obtained with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[RTXB_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_address[kMaxDevices] = {nullptr};

thread_local char g_noalloc_error[192] = "";

// First call on a device: resolve that device's address of the array, with the
// device current.  Later calls on the same device reuse it.
int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) return RTXB_E_CUDA;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_address[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) return RTXB_E_CUDA;
    g_scratch_address[dev] = ptr;
  }
  *out = g_scratch_address[dev];
  return RTXB_OK;
}

}  // namespace

extern "C" int rtxb_mxfp8_linear_fwd_noalloc(const void* x_bf16, const void* w_bf16, void* out_bf16, int64_t m,
                                             int64_t n, int64_t k, int rounding, void* stream, int* status) {
  if (!x_bf16 || !w_bf16 || !out_bf16) return RTXB_E_INVALID_ARGUMENT;
  if (m <= 0 || n <= 0 || k <= 0) return RTXB_E_INVALID_ARGUMENT;
  // The operands of this shape must fit the fixed array; nothing is launched otherwise.
  const size_t need = rtxb_mxfp8_linear_workspace_bytes(m, n, k);
  if (need > static_cast<size_t>(RTXB_NOALLOC_SCRATCH_BYTES)) return RTXB_E_SCRATCH_CAPACITY;
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != RTXB_OK) return rc;
  // Same kernels as rtxb_mxfp8_linear_fwd.  They overwrite every byte of the scratch they later
  // read (payload rows and whole scale tiles, padding included), so nothing has to be cleared even
  // though the array still holds the previous call's operands.
  return rtxb_mxfp8_linear_fwd(x_bf16, w_bf16, out_bf16, m, n, k, rounding, scratch,
                               static_cast<size_t>(RTXB_NOALLOC_SCRATCH_BYTES), stream, status);
}
