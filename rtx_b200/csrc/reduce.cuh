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

}  // namespace rtxb
