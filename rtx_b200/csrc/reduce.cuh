// FP32 partial sums -> one BF16 rounding: out[i] = bf16( sum_s parts[s * stride + i] ), serial order s = 0, 1, ...
// The reference's MXFP8WorkspaceReduceKernel (rtx/kernels/mxfp8_reduce.py:20-104, "serial" algorithm) reduces
// the [split, M, N] workspace of its split-K GEMMs this way.  Here the partials are the per-rank dW blocks that
// the data-parallel backward writes into the owner's staging slots over NVLink; the owner sums them once and
// rounds once.  HBM bound: (4 * parts + 2) bytes per element.
#pragma once

#include "common.cuh"

namespace rtxb {

constexpr int kReduceThreads = 256;

__global__ void __launch_bounds__(kReduceThreads) sum_parts_f32_to_bf16_kernel(const float* __restrict__ parts, int n_parts,
                                                                              int64_t stride, int64_t count,
                                                                              __nv_bfloat16* __restrict__ out) {
  // eight elements per thread: two 16-byte loads per part, one 16-byte store
  const int64_t vecs = count / 8;
  for (int64_t v = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; v < vecs;
       v += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
#pragma unroll 4
    for (int s = 0; s < n_parts; ++s) {
      const float4* src = reinterpret_cast<const float4*>(parts + s * stride + v * 8);
      const float4 a = __ldg(src), b = __ldg(src + 1);
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
      w[e] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(out + v * 8) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  // tail (count not a multiple of 8)
  if (blockIdx.x == 0) {
    for (int64_t i = vecs * 8 + threadIdx.x; i < count; i += blockDim.x) {
      float acc = 0.0f;
      for (int s = 0; s < n_parts; ++s) acc += parts[s * stride + i];
      out[i] = __float2bfloat16_rn(acc);
    }
  }
}

// Self-test of the bounded wait every kernel role uses: one warp waits on a barrier that nothing will ever
// complete, with the limit given; when the limit runs out it records kStatusWaitSelfTest in the status word,
// raises the abort flag as the GEMM roles do, and the kernel returns normally.  Nothing traps, nothing spins
// without a bound: this is how a lost arrival shows up to the host instead of as a hung GPU.
__global__ void wait_selftest_kernel(uint64_t limit_ns, int* status, unsigned long long* waited_ns) {
  __shared__ uint64_t never;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&never, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  const uint64_t t0 = global_timer_ns();
  const bool completed = mbar_wait(&never, 0, &abort_flag, limit_ns);
  const uint64_t t1 = global_timer_ns();
  if (!completed && threadIdx.x == 0) {
    if (status) atomicCAS(status, 0, kStatusWaitSelfTest);
    abort_flag = 1;
    if (waited_ns) *waited_ns = t1 - t0;
  }
}

}  // namespace rtxb
