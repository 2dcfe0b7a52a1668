// Decode forward for a handful of token rows (layout: up to 8; dispatched for M <= 4) in ONE kernel: the BF16 activations are quantized
// to NVFP4 inside the GEMM kernel by the warps that otherwise only run the epilogue, while the producer
// warp is already streaming the packed weight.  This is the fused form the reference's NVFP4 path aims at
// (quantizer warps next to the MMA, rtx/kernels/nvfp4_quant.py + nvfp4_gemm.py; frontend
// `nvfp4_linear_dynamic_x_prequant_w`, rtx/fp4.py:1628-1686 with the current-|max| outer scale of
// NVFP4Linear.forward), affordable here because every CTA can re-quantize the few rows itself:
//
//   warp 0      TMA producer: weight tiles B / SFB only (3-D boxes of `ks` K steps), from kernel entry
//   warp 1      MMA issuer: waits until the activations are in place, then as the streaming kernel
//   warps 2..   1. |max| of the whole X (4 quantizer warps for M <= 2, 12 above) (every CTA reads all M x K values from L2 and gets the same bits)
//               2. outer scale by the tensor-scale rule; output scale = that x the weight's outer scale
//               3. quantize X: E2M1 payload written straight into 128-byte-swizzled A tiles (one 1 KB tile of
//                  8 rows per K step, all K steps resident) and E4M3 block scales into 128-row scale tiles
//               4. fence to the async proxy, signal the MMA warp, then run the epilogue
//
// Same arithmetic, in the same order, as amax_bf16_kernel + nvfp4_tensor_scale_kernel +
// quant_nvfp4_rows_kernel followed by the streaming GEMM: outputs are bit-identical to that chain.
// Shared memory: A tiles k_tiles x 1 KB, scale tiles k_tiles x 2 KB (K <= 8192: 96 KB), the rest is the
// weight ring.  Rows M..7 of the A tiles and rows 8..127 of the scale tiles are never written: they only
// reach accumulator rows that are not stored.
#pragma once

#include "gemm_skinny.cuh"
#include "quant.cuh"

namespace rtxb {

constexpr int kFusedMaxRows = 8;
constexpr int kFusedATile = kFusedMaxRows * kBlockKBytes;   // 1 KB per K step
constexpr int kFusedBarBytes = (2 * kSkinnyMaxSlots + 5) * 8 + 16;   // ring + accumulator + a_ready barriers, 3 words

struct FusedXParams {
  const __nv_bfloat16* x;   // [m, k], pitch ldx elements; k % 16 == 0, ldx % 8 == 0, 16-byte aligned
  int64_t ldx;
  int k;                    // values per row
  int mode;                 // tensor-scale rule: 0 exact, 1 power of two
  const float* w_scale;     // outer scale of the packed weight
  float* x_scale_out;       // optional: the activation scale used (written by CTA 0)
};

__host__ __device__ inline int fused_ring_slot_bytes(int ks) {
  return ks * (SkinnyTraits<kKindNvfp4>::kBBytes + SkinnyTraits<kKindNvfp4>::kSfBytes);
}
__host__ __device__ inline int fused_resident_bytes(int k_tiles) {
  return k_tiles * (kFusedATile + SkinnyTraits<kKindNvfp4>::kSfBytes);
}
__host__ __device__ inline int fused_slots_for(int k_tiles, int ks) {
  const int s = (kSkinnySmemBudget - 1024 - kFusedBarBytes - fused_resident_bytes(k_tiles)) / fused_ring_slot_bytes(ks);
  return s > kSkinnyMaxSlots ? kSkinnyMaxSlots : s;
}
__host__ __device__ inline int fused_smem_bytes(int k_tiles, int ks, int slots) {
  return 1024 + fused_resident_bytes(k_tiles) + slots * fused_ring_slot_bytes(ks) + kFusedBarBytes;
}

// Threads: 64 (producer + MMA warps) + 32 per quantizer warp; the first four quantizer warps also run the
// epilogue (one per TMEM lane quadrant), further ones only quantize.
constexpr int kFusedMaxThreads = 64 + 12 * 32;

__global__ void __launch_bounds__(kFusedMaxThreads, 1)
gemm_decode_fused_kernel(const __grid_constant__ CUtensorMap map_b, const GemmParams p, const FusedXParams fx) {
  using T = SkinnyTraits<kKindNvfp4>;
  const int S = p.slots, KS = p.ks;
  const int off_sfa = p.k_tiles * kFusedATile;
  const int off_b = off_sfa + p.k_tiles * T::kSfBytes;
  const int off_sfb = off_b + S * KS * T::kBBytes;
  const int off_bars = off_sfb + S * KS * T::kSfBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + off_bars);
  uint64_t* full_bar = bars;                  // [S] weights of a slot landed
  uint64_t* empty_bar = bars + S;             // [S]
  uint64_t* acc_full_bar = bars + 2 * S;      // [2]
  uint64_t* acc_free_bar = acc_full_bar + 2;  // [2]
  uint64_t* a_ready_bar = acc_free_bar + 2;   // quantized activations in place (one arrival per quantizer warp)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(a_ready_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint32_t* cta_amax = const_cast<uint32_t*>(reinterpret_cast<volatile uint32_t*>(abort_flag + 1));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_tiles = p.n_tiles;
  const int k_groups = (p.k_tiles + KS - 1) / KS;
  const int my_tiles = (total_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                       static_cast<int>(gridDim.x);
  const int total_groups = my_tiles * k_groups;

  griddep_launch_dependents();

  // weights of group `kg` of tile `tile` into ring slot `slot`
  auto load_weights = [&](int slot, int tile, int kg) {
    const int b_row0 = tile * kSkinnyN;
    const int kt0 = kg * KS, live = min(KS, p.k_tiles - kt0);
    mbar_expect_tx(&full_bar[slot], static_cast<uint32_t>(KS * T::kBBytes + live * T::kSfBytes));
    tma_load_3d(smem + off_b + slot * KS * T::kBBytes, &map_b, &full_bar[slot], 0, b_row0, kt0);
    const uint8_t* sfb_src =
        p.sfb + (static_cast<size_t>(b_row0 >> 7) * p.sf_k_chunks + static_cast<size_t>(kt0) * T::kSfChunks) * 512;
    bulk_load_1d(smem + off_sfb + slot * KS * T::kSfBytes, sfb_src, live * T::kSfBytes, &full_bar[slot]);
  };

  const int first_pass = total_groups < S ? total_groups : S;
  if (warp == 0) {
    // one lane per ring slot initialises its two barriers (S <= 24), so the first load is not behind 2 S serial inits
    if (lane == 0) prefetch_tensormap(&map_b);
    if (lane < S) {
      mbar_init(&full_bar[lane], 1);
      mbar_init(&empty_bar[lane], 1);
    }
    fence_barrier_init();
    __syncwarp();
    if (lane == 0) {
      int tile = blockIdx.x, kg = 0;
      for (int i = 0; i < first_pass; ++i) {   // the weights never depend on the grid before this one
        load_weights(i, tile, kg);
        if (++kg == k_groups) { kg = 0; tile += gridDim.x; }
      }
    }
    __syncwarp();
  } else if (threadIdx.x == 32) {
    for (int w = 0; w < 2; ++w) {
      mbar_init(&acc_full_bar[w], 1);
      mbar_init(&acc_free_bar[w], 4);
    }
    mbar_init(a_ready_bar, (blockDim.x - 64) >> 5);   // one arrival per quantizer warp
    *abort_flag = 0;
    *cta_amax = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(tmem_slot, T::kTmemColsS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (weights) ------------------------------
    const bool leader = elect_one_sync();
    int slot = first_pass == S ? 0 : first_pass;
    uint32_t phase = first_pass == S ? 1 : 0;
    int tile = static_cast<int>(blockIdx.x) + (first_pass / k_groups) * static_cast<int>(gridDim.x);
    int kg = first_pass % k_groups;
    for (int g = first_pass; g < total_groups; ++g) {
      if (!mbar_wait(&empty_bar[slot], phase ^ 1, abort_flag)) {
        if (p.status && leader) atomicCAS(p.status, 0, kStatusWaitProducer);
        *abort_flag = 1;
        break;
      }
      if (leader) load_weights(slot, tile, kg);
      __syncwarp();
      if (++slot == S) { slot = 0; phase ^= 1; }
      if (++kg == k_groups) { kg = 0; tile += gridDim.x; }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    const bool leader = elect_one_sync();
    const uint32_t smem_base = smem_u32(smem);
    bool ok = mbar_wait(a_ready_bar, 0, abort_flag);   // activations quantized (generic writes fenced by the writers)
    if (!ok) {
      if (p.status && leader) atomicCAS(p.status, 0, kStatusWaitQuant);
      *abort_flag = 1;
    }
    tc_fence_after_sync();
    int slot = 0;
    uint32_t phase = 0, local_tile = 0, step = 0;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local_tile) {
      const int win = local_tile & 1;
      const uint32_t sfb_shift = 2 * (tile & 1);
      if (local_tile >= 2) {
        if (!mbar_wait(&acc_free_bar[win], ((local_tile >> 1) - 1) & 1, abort_flag)) {
          if (p.status && leader) atomicCAS(p.status, 0, kStatusWaitMma);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
      }
      for (int kg = 0; kg < k_groups; ++kg) {
        if (!mbar_wait(&full_bar[slot], phase, abort_flag)) {
          if (p.status && leader) atomicCAS(p.status, 0, kStatusWaitMma);
          *abort_flag = 1;
          ok = false;
          break;
        }
        if (leader) {
          const int live = min(KS, p.k_tiles - kg * KS);
          for (int sub = 0; sub < live; ++sub, ++step) {
            const int kt = kg * KS + sub;
            const int set = step & 1;
            const uint32_t ta = tmem_base + T::kSfBase + set * T::kSfSetCols;
            const uint32_t tb = ta + 4 * T::kSfChunks;
            const uint32_t ssfa = smem_base + off_sfa + kt * T::kSfBytes;
            const uint32_t ssfb = smem_base + off_sfb + (slot * KS + sub) * T::kSfBytes;
#pragma unroll
            for (int c = 0; c < T::kSfChunks; ++c) {
              tc_cp_32x128b_warpx4(ta + 4 * c, umma_desc_sf(ssfa + 512 * c));
              tc_cp_32x128b_warpx4(tb + 4 * c, umma_desc_sf(ssfb + 512 * c));
            }
            const uint64_t da = umma_desc_sw128(smem_base + kt * kFusedATile);
            const uint64_t db = umma_desc_sw128(smem_base + off_b + (slot * KS + sub) * T::kBBytes);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t acc = (kg > 0 || sub > 0 || j > 0) ? 1u : 0u;
              tc_mma_mxf4nvf4(tmem_base + win * kSkinnyN, da + 2 * j, db + 2 * j, T::kIdesc, ta + 4 * j,
                              tb + 4 * j + sfb_shift, acc);
            }
          }
          tc_commit(&empty_bar[slot]);
        }
        __syncwarp();
        if (++slot == S) { slot = 0; phase ^= 1; }
      }
      if (!ok) break;
      if (leader) tc_commit(&acc_full_bar[win]);
      __syncwarp();
    }
    __syncwarp();
  } else {
    // ------------------------------ quantizer, then epilogue ------------------------------
    griddep_wait();   // X may be the output of the grid launched just before this one
    const int qt = threadIdx.x - 64;        // index among the quantizer threads
    const int nq = blockDim.x - 64;         // quantizer threads (a multiple of 32, at least 128)
    const uint16_t* xs = reinterpret_cast<const uint16_t*>(fx.x);
    // 1. |max| of X as bits (NaN patterns order above infinity), eight 16-byte loads in flight per thread
    {
      const int vec_per_row = fx.k / 8;
      const int total = p.m * vec_per_row;
      uint32_t m = 0;
      for (int i0 = qt; i0 < total; i0 += 8 * nq) {
        uint4 raw[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int i = i0 + nq * j;
          raw[j] = i < total ? __ldg(reinterpret_cast<const uint4*>(xs + static_cast<int64_t>(i / vec_per_row) * fx.ldx) +
                                     i % vec_per_row)
                             : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t w[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            m = max(m, (w[e] << 16) & 0x7FFFFFFFu);
            m = max(m, w[e] & 0x7FFF0000u);
          }
        }
      }
      m = __reduce_max_sync(0xffffffffu, m);
      if (lane == 0 && m != 0) atomicMax(cta_amax, m);
      asm volatile("bar.sync 1, %0;" ::"r"(nq) : "memory");   // the quantizer warps only
    }
    // 2. outer scale (the same bits in every CTA) and the GEMM's output scale
    const float st = nvfp4_scale_from_amax_bits(*cta_amax, fx.mode);
    const float out_scale = st * __ldg(fx.w_scale);
    if (fx.x_scale_out && blockIdx.x == 0 && qt == 0) *fx.x_scale_out = st;
    // 3. quantize: unit = (row, block of 16 values) -> 8 payload bytes + 1 scale byte, written where the MMA
    //    expects them (128-byte swizzle: 16-byte chunk index XOR row % 8)
    {
      const float six_st = 6.0f * st;
      const float inv_st = __fdiv_rn(1.0f, st);
      const int nb_row = p.k_tiles * 16;            // blocks per row up to the end of the last K step
      const int nb_live = fx.k / 16;                // blocks holding values
      const int units = p.m * nb_row;
      for (int u0 = qt; u0 < units; u0 += 4 * nq) {
        // four units per pass so that eight 16-byte loads are in flight before the first is used
        uint4 raw[4][2];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int u = u0 + nq * j;
          const int row = u / nb_row, blk = u - row * nb_row;
          raw[j][0] = raw[j][1] = make_uint4(0, 0, 0, 0);
          if (u < units && blk < nb_live) {
            const uint4* src = reinterpret_cast<const uint4*>(xs + static_cast<int64_t>(row) * fx.ldx + blk * 16);
            raw[j][0] = __ldg(src);
            raw[j][1] = __ldg(src + 1);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int u = u0 + nq * j;
          if (u >= units) break;
          const int row = u / nb_row, blk = u - row * nb_row;
          float v[16];
          unpack8(raw[j][0], *reinterpret_cast<float(*)[8]>(&v[0]));
          unpack8(raw[j][1], *reinterpret_cast<float(*)[8]>(&v[8]));
          float a = fabsf(v[0]);
#pragma unroll
          for (int e = 1; e < 16; ++e) a = fmax_nan(a, fabsf(v[e]));
          float rawscale = __fdiv_rn(a, six_st);
          rawscale = fmin_nan(fmax_nan(rawscale, 0.015625f), 448.0f);
          const uint32_t sb = cvt_e4m3x2(rawscale, rawscale) & 0xFF;
          const float recip = __fdiv_rn(inv_st, e4m3_to_float(sb));
          uint32_t w0 = 0, w1 = 0;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            w0 |= cvt_e2m1x2(v[2 * e] * recip, v[2 * e + 1] * recip) << (8 * e);
            w1 |= cvt_e2m1x2(v[8 + 2 * e] * recip, v[8 + 2 * e + 1] * recip) << (8 * e);
          }
          const int kt = blk >> 4, b16 = blk & 15;
          const int chunk = (b16 >> 1) ^ (row & 7);
          uint8_t* a_dst = smem + kt * kFusedATile + row * kBlockKBytes + chunk * 16 + (b16 & 1) * 8;
          *reinterpret_cast<uint2*>(a_dst) = make_uint2(w0, w1);
          // scale tile (128 rows x 4 blocks = 512 bytes): byte (row % 32) * 16 + (row / 32) * 4 + block % 4
          smem[off_sfa + kt * T::kSfBytes + (b16 >> 2) * 512 + row * 16 + (b16 & 3)] =
              blk < nb_live ? static_cast<uint8_t>(sb) : 0;
        }
      }
    }
    // 4. make the generic-proxy writes visible to the tensor core's reads, then signal
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(a_ready_bar);

    // ------------------------------ epilogue (first four quantizer warps) ------------------------------
    if (warp < 6) {
    const int quad = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const int row = quad * 32 + lane;
    const bool row_ok = row < p.m;
    uint32_t local_tile = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local_tile) {
      const int win = local_tile & 1;
      if (!mbar_wait(&acc_full_bar[win], (local_tile >> 1) & 1, abort_flag)) {
        if (p.status && lane == 0) atomicCAS(p.status, 0, kStatusWaitEpilogue);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      uint32_t r0[32], r1[32];
      tmem_ld_32x32(tmem_base + lane_base + win * kSkinnyN, r0);
      tmem_ld_32x32(tmem_base + lane_base + win * kSkinnyN + 32, r1);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_free_bar[win]);
      if (!row_ok) continue;
      const int col = tile * kSkinnyN;
      __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(row) * p.ldo;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint32_t (&r)[32] = half ? r1 : r0;
#pragma unroll
        for (int v = 0; v < 32; v += 8) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(r[v + 2 * e]) * out_scale,
                                                     __uint_as_float(r[v + 2 * e + 1]) * out_scale);
            w[e] = *reinterpret_cast<uint32_t*>(&b);
          }
          store_bf16x8(out, col + 32 * half + v, p.out_cols, p.out_vec_ok != 0, w);
        }
      }
    }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, T::kTmemColsS);
  }
}

}  // namespace rtxb
