// Skinny block-scaled GEMM for M <= 128 (decode / small-batch inference): D[M,N] = A[M,K] B[N,K]^T
// with the weights B streamed from HBM exactly once.  The work is HBM bound, so the kernel is shaped
// for bandwidth rather than tensor throughput: one 128 x 64 tile per step (N / 64 tiles keep every
// SM busy even at N = 8192), a deep ring of small slots (A 16 KB from L2, B 8 KB from HBM), and two
// disjoint 64-column accumulator windows so that the epilogue of one tile never delays the next.
// Same roles as the large-tile kernel: warp 0 TMA producer, warp 1 MMA issuer (one elected lane),
// warps 2..5 epilogue.  Replaces the reference's persistent packed GEMM on decode shapes
// (rtx/kernels/mxfp8_gemm.py:1009-1045 persistence schedules; rtx/fp4.py:639-668 `_DynamicXRunner`).
#pragma once

#include "gemm_blockscaled.cuh"

namespace rtxb {

constexpr int kSkinnyN = 64;

template <int KIND>
struct SkinnyTraits {
  static constexpr int kSfChunks = KIND == kKindMxfp8 ? 1 : 4;
  static constexpr int kSfBytes = 512 * kSfChunks;          // one 128-row scale tile set per operand per K step
  static constexpr int kABytes = 128 * kBlockKBytes;
  static constexpr int kBBytes = kSkinnyN * kBlockKBytes;
  static constexpr int kSlots = KIND == kKindMxfp8 ? 8 : 7;
  static constexpr int kOffB = kSlots * kABytes;
  static constexpr int kOffSfa = kOffB + kSlots * kBBytes;
  static constexpr int kOffSfb = kOffSfa + kSlots * kSfBytes;
  static constexpr int kOffBars = kOffSfb + kSlots * kSfBytes;
  static constexpr int kSmemBytes = kOffBars + 1024 + 256;
  // TMEM: accumulator windows [0,64) and [64,128); scale sets from column 128
  static constexpr int kTmemColsS = 256;
  static constexpr int kSfSetCols = 8 * kSfChunks;           // SFA 4c + SFB 4c (one 128-row tile each)
  static constexpr int kSfBase = 128;
  static constexpr uint32_t kIdesc =
      idesc_block_scaled(128, kSkinnyN, KIND == kKindMxfp8 ? 0u : 1u, KIND == kKindMxfp8 ? 1u : 0u);
};

template <int KIND, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const GemmParams p) {
  using T = SkinnyTraits<KIND>;
  constexpr int S = T::kSlots;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + T::kOffBars);
  uint64_t* full_bar = bars;                // [S]
  uint64_t* empty_bar = bars + S;           // [S]
  uint64_t* acc_full_bar = bars + 2 * S;    // [2] one per accumulator window
  uint64_t* acc_free_bar = acc_full_bar + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_tiles = p.n_tiles;   // one 128-row block of A; n_tiles counts 64-wide tiles

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(&acc_full_bar[w], 1);
      mbar_init(&acc_free_bar[w], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, T::kTmemColsS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    const bool leader = elect_one_sync();
    if (leader) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
    }
    int slot = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int b_row0 = tile * kSkinnyN;
      const uint8_t* sfb_src = p.sfb + static_cast<size_t>(b_row0 >> 7) * p.sf_k_chunks * 512;
      for (int kt = 0; kt < p.k_tiles; ++kt) {
        if (!mbar_wait(&empty_bar[slot], phase ^ 1, abort_flag)) {
          if (p.status && leader) atomicCAS(p.status, 0, kStatusWaitProducer);
          *abort_flag = 1;
          ok = false;
          break;
        }
        if (leader) {
          mbar_expect_tx(&full_bar[slot], T::kABytes + T::kBBytes + 2 * T::kSfBytes);
          tma_load_2d(smem + slot * T::kABytes, &map_a, &full_bar[slot], kt * kBlockKBytes, 0);
          tma_load_2d(smem + T::kOffB + slot * T::kBBytes, &map_b, &full_bar[slot], kt * kBlockKBytes, b_row0);
          const size_t sf_off = static_cast<size_t>(kt) * T::kSfBytes;
          bulk_load_1d(smem + T::kOffSfa + slot * T::kSfBytes, p.sfa + sf_off, T::kSfBytes, &full_bar[slot]);
          bulk_load_1d(smem + T::kOffSfb + slot * T::kSfBytes, sfb_src + sf_off, T::kSfBytes, &full_bar[slot]);
        }
        __syncwarp();
        if (++slot == S) { slot = 0; phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    const bool leader = elect_one_sync();
    const uint32_t smem_base = smem_u32(smem);
    int slot = 0;
    uint32_t phase = 0, local_tile = 0, step = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local_tile) {
      const int win = local_tile & 1;
      // the 64 B rows of this tile are rows (tile & 1) * 64 .. of their 128-row scale tile:
      // their scale columns start 2 columns into the copied set
      const uint32_t sfb_shift = 2 * (tile & 1);
      if (local_tile >= 2) {
        // window `win` was last used by tile local_tile - 2: its epilogue must have drained it
        if (!mbar_wait(&acc_free_bar[win], ((local_tile >> 1) - 1) & 1, abort_flag)) {
          if (p.status && leader) atomicCAS(p.status, 0, kStatusWaitMma);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
      }
      bool ok = true;
      for (int kt = 0; kt < p.k_tiles; ++kt, ++step) {
        if (!mbar_wait(&full_bar[slot], phase, abort_flag)) {
          if (p.status && leader) atomicCAS(p.status, 0, kStatusWaitMma);
          *abort_flag = 1;
          ok = false;
          break;
        }
        if (leader) {
          const int set = step & 1;
          const uint32_t ta = tmem_base + T::kSfBase + set * T::kSfSetCols;
          const uint32_t tb = ta + 4 * T::kSfChunks;
          const uint32_t ssfa = smem_base + T::kOffSfa + slot * T::kSfBytes;
          const uint32_t ssfb = smem_base + T::kOffSfb + slot * T::kSfBytes;
#pragma unroll
          for (int c = 0; c < T::kSfChunks; ++c) {
            tc_cp_32x128b_warpx4(ta + 4 * c, umma_desc_sf(ssfa + 512 * c));
            tc_cp_32x128b_warpx4(tb + 4 * c, umma_desc_sf(ssfb + 512 * c));
          }
          const uint64_t da = umma_desc_sw128(smem_base + slot * T::kABytes);
          const uint64_t db = umma_desc_sw128(smem_base + T::kOffB + slot * T::kBBytes);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t acc = (kt > 0 || j > 0) ? 1u : 0u;
            if (KIND == kKindMxfp8)
              tc_mma_mxf8f6f4(tmem_base + win * kSkinnyN, da + 2 * j, db + 2 * j, idesc_with_sf_ids(T::kIdesc, j, j), ta,
                              tb + sfb_shift, acc);
            else
              tc_mma_mxf4nvf4(tmem_base + win * kSkinnyN, da + 2 * j, db + 2 * j, T::kIdesc, ta + 4 * j,
                              tb + 4 * j + sfb_shift, acc);
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
    // ------------------------------ epilogue ------------------------------
    const int quad = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const float out_scale = p.out_scale ? __ldg(p.out_scale) : 1.0f;
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
      if (lane == 0) mbar_arrive(&acc_free_bar[win]);   // window drained into registers
      if (!row_ok) continue;
      const int col = tile * kSkinnyN;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint32_t (&r)[32] = half ? r1 : r0;
        if (EPI == kEpiBf16) {
          __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(row) * p.ldo;
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
        } else {
          float* out = reinterpret_cast<float*>(p.out) + static_cast<int64_t>(row) * p.ldo;
          for (int v = 0; v < 32; ++v)
            if (col + 32 * half + v < p.out_cols) out[col + 32 * half + v] = __uint_as_float(r[v]) * out_scale;
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
