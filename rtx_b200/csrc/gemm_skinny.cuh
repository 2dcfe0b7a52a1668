// Streaming block-scaled GEMM for M <= 128 (decode / small-batch inference): D[M,N] = A[M,K] B[N,K]^T
// with the weights B read from HBM exactly once.  The work is HBM bound, so the kernel is shaped
// for bytes in flight rather than tensor throughput:
//   * one 128 x 64 tile per step (N / 64 tiles keep every SM busy even at N = 8192) and two disjoint
//     64-column accumulator windows, so the epilogue of one tile never delays the next;
//   * only the live rows of A are fetched: the TMA box of A is M rounded up to 8 rows (one 1 KB
//     swizzle atom per 8 rows).  The MMA still reads 128 rows from the slot; rows past the box are
//     whatever shared memory holds and only reach accumulator rows that are never stored;
//   * the ring depth is chosen at launch from what fits shared memory with that A box (up to
//     kSkinnyMaxSlots K steps of 8 KB of B in flight per SM);
//   * the producer starts the weight loads of the first ring pass before it waits for the grid it
//     depends on (programmatic dependent launch): when the launch is marked as such, the weights
//     stream while the kernel that quantizes the activations is still running.
// Same roles as the large-tile kernel: warp 0 TMA producer, warp 1 MMA issuer (warp-uniform loop,
// one elected lane issues), warps 2..5 epilogue.  Replaces the reference's persistent packed GEMM on
// decode shapes (rtx/kernels/mxfp8_gemm.py:1009-1045 persistence schedules; rtx/fp4.py:639-668
// `_DynamicXRunner`).
#pragma once

#include "gemm_blockscaled.cuh"

namespace rtxb {

constexpr int kSkinnyN = 64;
constexpr int kSkinnyMaxSlots = 24;
constexpr int kSkinnySmemBudget = 227 * 1024;

template <int KIND>
struct SkinnyTraits {
  static constexpr int kSfChunks = KIND == kKindMxfp8 ? 1 : 4;
  static constexpr int kSfBytes = 512 * kSfChunks;          // one 128-row scale tile set per operand per K step
  static constexpr int kBBytes = kSkinnyN * kBlockKBytes;
  static constexpr int kBarBytes = (2 * kSkinnyMaxSlots + 4) * 8 + 16;
  // TMEM: accumulator windows [0,64) and [64,128); scale sets from column 128
  static constexpr int kTmemColsS = 256;
  static constexpr int kSfSetCols = 8 * kSfChunks;           // SFA 4c + SFB 4c (one 128-row tile each)
  static constexpr int kSfBase = 128;
  static constexpr uint32_t kIdesc =
      idesc_block_scaled(128, kSkinnyN, KIND == kKindMxfp8 ? 0u : 1u, KIND == kKindMxfp8 ? 1u : 0u);

  // a ring slot holds `ks` consecutive K steps
  __host__ __device__ static constexpr int slot_bytes(int a_box_rows, int ks) {
    return ks * (a_box_rows * kBlockKBytes + kBBytes + 2 * kSfBytes);
  }
  // ring slots for an A box of `a_box_rows` rows (1 KB of slack for the 1024-byte alignment of the ring)
  __host__ __device__ static constexpr int slots_for(int a_box_rows, int ks) {
    const int s = (kSkinnySmemBudget - 1024 - kBarBytes) / slot_bytes(a_box_rows, ks);
    return s > kSkinnyMaxSlots ? kSkinnyMaxSlots : s;
  }
  __host__ __device__ static constexpr int smem_bytes(int a_box_rows, int ks, int slots) {
    return 1024 + slots * slot_bytes(a_box_rows, ks) + kBarBytes;
  }
};

// Loads of one ring slot.  With a 3-D tensor map one instruction fetches all `ks` K steps of an
// operand (issuing a TMA instruction costs the issuing thread on the order of 100 clocks, which at
// four instructions per 8 KB K step is what bounded the streaming rate); payloads whose rows are not
// 128-byte multiples use one 2-D instruction per K step.
template <int KIND>
struct SkinnySlotLoader {
  using T = SkinnyTraits<KIND>;
  const CUtensorMap* map_a;
  const CUtensorMap* map_b;
  const GemmParams& p;
  uint8_t* smem;
  int a_bytes, off_b, off_sfa, off_sfb, ks;

  // K steps of group `kg` that lie inside K
  __device__ __forceinline__ int live_steps(int kg) const { return min(ks, p.k_tiles - kg * ks); }
  __device__ __forceinline__ uint32_t tx_bytes(int kg) const {
    const int live = live_steps(kg);
    // a 3-D box always delivers its full size (chunks past K read as zeros); 2-D loads are issued per live step
    const int payload_steps = p.map3d ? ks : live;
    return static_cast<uint32_t>(payload_steps * (a_bytes + T::kBBytes) + 2 * live * T::kSfBytes);
  }
  __device__ __forceinline__ void weights(int slot, int tile, int kg, uint64_t* bar) const {
    const int b_row0 = tile * kSkinnyN;
    const int kt0 = kg * ks, live = live_steps(kg);
    uint8_t* sb = smem + off_b + slot * ks * T::kBBytes;
    if (p.map3d) {
      tma_load_3d(sb, map_b, bar, 0, b_row0, kt0);
    } else {
      for (int i = 0; i < live; ++i) tma_load_2d(sb + i * T::kBBytes, map_b, bar, (kt0 + i) * kBlockKBytes, b_row0);
    }
    const uint8_t* sfb_src = p.sfb + (static_cast<size_t>(b_row0 >> 7) * p.sf_k_chunks + static_cast<size_t>(kt0) * T::kSfChunks) * 512;
    bulk_load_1d(smem + off_sfb + slot * ks * T::kSfBytes, sfb_src, live * T::kSfBytes, bar);
  }
  __device__ __forceinline__ void activations(int slot, int kg, uint64_t* bar) const {
    const int kt0 = kg * ks, live = live_steps(kg);
    uint8_t* sa = smem + slot * ks * a_bytes;
    if (p.map3d) {
      tma_load_3d(sa, map_a, bar, 0, 0, kt0);
    } else {
      for (int i = 0; i < live; ++i) tma_load_2d(sa + i * a_bytes, map_a, bar, (kt0 + i) * kBlockKBytes, 0);
    }
    bulk_load_1d(smem + off_sfa + slot * ks * T::kSfBytes, p.sfa + static_cast<size_t>(kt0) * T::kSfBytes,
                 live * T::kSfBytes, bar);
  }
};

template <int KIND, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const GemmParams p) {
  using T = SkinnyTraits<KIND>;
  const int S = p.slots;
  const int KS = p.ks;
  const int a_bytes = p.a_box_rows * kBlockKBytes;
  // ring: [A x S][B x S][SFA x S][SFB x S][barriers], each slot KS K steps.  The MMA reads 16 KB from
  // an A tile whatever the box height: for the last tiles that range runs into the B slots, which is
  // inside the allocation because S * KS * 8 KB >= 16 KB.
  const int off_b = S * KS * a_bytes;
  const int off_sfa = off_b + S * KS * T::kBBytes;
  const int off_sfb = off_sfa + S * KS * T::kSfBytes;
  const int off_bars = off_sfb + S * KS * T::kSfBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + off_bars);
  uint64_t* full_bar = bars;                // [S]
  uint64_t* empty_bar = bars + S;           // [S]
  uint64_t* acc_full_bar = bars + 2 * S;    // [2] one per accumulator window
  uint64_t* acc_free_bar = acc_full_bar + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_tiles = p.n_tiles;   // one 128-row block of A; n_tiles counts 64-wide tiles
  const int k_groups = (p.k_tiles + KS - 1) / KS;

  // A grid launched as a programmatic dependent of this one may start its own prologue now; it
  // orders its memory accesses against this grid with griddepcontrol.wait.
  griddep_launch_dependents();

  // The producer warp initialises the ring barriers itself and starts the first ring pass before
  // the block-wide barrier below, so the first loads are in flight while TMEM is being allocated.
  const SkinnySlotLoader<KIND> loader{&map_a, &map_b, p, smem, a_bytes, off_b, off_sfa, off_sfb, KS};
  const int my_tiles = (total_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                       static_cast<int>(gridDim.x);
  const int total_groups = my_tiles * k_groups;
  const int first_pass = total_groups < S ? total_groups : S;
  if (warp == 0) {
    // one lane per ring slot initialises its two barriers (S <= 24), so the first load is not behind 2 S serial inits
    if (lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
    }
    if (lane < S) {
      mbar_init(&full_bar[lane], 1);
      mbar_init(&empty_bar[lane], 1);
    }
    fence_barrier_init();
    __syncwarp();
    if (lane == 0) {
      // First ring pass (every slot is free).  The weights B / SFB never depend on the grid launched
      // just before this one, the activations A / SFA may: when the launch is marked as overlapping
      // its predecessor, all weight loads of the pass go first, then the wait, then the activations.
      int tile = blockIdx.x, kg = 0;
      for (int i = 0; i < first_pass; ++i) {
        mbar_expect_tx(&full_bar[i], loader.tx_bytes(kg));
        loader.weights(i, tile, kg, &full_bar[i]);
        if (!p.overlap_previous) loader.activations(i, kg, &full_bar[i]);
        if (++kg == k_groups) { kg = 0; tile += gridDim.x; }
      }
    }
    __syncwarp();
    if (p.overlap_previous) griddep_wait();
    if (lane == 0) {
      if (p.overlap_previous) {
        int kg = 0;
        for (int i = 0; i < first_pass; ++i) {
          loader.activations(i, kg, &full_bar[i]);
          if (++kg == k_groups) kg = 0;
        }
      }
    }
    __syncwarp();
  } else if (threadIdx.x == 32) {
    for (int w = 0; w < 2; ++w) {
      mbar_init(&acc_full_bar[w], 1);
      mbar_init(&acc_free_bar[w], 4);
    }
    *abort_flag = 0;
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
    // ------------------------------ TMA producer ------------------------------
    const bool leader = elect_one_sync();
    // Remaining groups: wait for the slot, then all loads.
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
      if (leader) {
        mbar_expect_tx(&full_bar[slot], loader.tx_bytes(kg));
        loader.weights(slot, tile, kg, &full_bar[slot]);
        loader.activations(slot, kg, &full_bar[slot]);
      }
      __syncwarp();
      if (++slot == S) { slot = 0; phase ^= 1; }
      if (++kg == k_groups) { kg = 0; tile += gridDim.x; }
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
            const int set = step & 1;
            const uint32_t ta = tmem_base + T::kSfBase + set * T::kSfSetCols;
            const uint32_t tb = ta + 4 * T::kSfChunks;
            const uint32_t ssfa = smem_base + off_sfa + (slot * KS + sub) * T::kSfBytes;
            const uint32_t ssfb = smem_base + off_sfb + (slot * KS + sub) * T::kSfBytes;
#pragma unroll
            for (int c = 0; c < T::kSfChunks; ++c) {
              tc_cp_32x128b_warpx4(ta + 4 * c, umma_desc_sf(ssfa + 512 * c));
              tc_cp_32x128b_warpx4(tb + 4 * c, umma_desc_sf(ssfb + 512 * c));
            }
            const uint64_t da = umma_desc_sw128(smem_base + (slot * KS + sub) * a_bytes);
            const uint64_t db = umma_desc_sw128(smem_base + off_b + (slot * KS + sub) * T::kBBytes);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t acc = (kg > 0 || sub > 0 || j > 0) ? 1u : 0u;
              if (KIND == kKindMxfp8)
                tc_mma_mxf8f6f4(tmem_base + win * kSkinnyN, da + 2 * j, db + 2 * j, idesc_with_sf_ids(T::kIdesc, j, j),
                                ta, tb + sfb_shift, acc);
              else
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
    // ------------------------------ epilogue ------------------------------
    griddep_wait();   // the output scale may come from the grid launched just before this one
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
