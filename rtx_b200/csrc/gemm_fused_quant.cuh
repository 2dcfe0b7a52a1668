// MXFP8 GEMM whose A operand is quantized inside the kernel (BF16 activations in, no quantizer
// launch, no packed copy of X in memory):  D[M,N] = epilogue( deq(quant(X[M,K])) * deq(B[N,K])^T ).
// The counterpart of the reference's fused forward MXFP8FusedLinearKernel
// (rtx/kernels/mxfp8_fwd.py:936-2934; roles :1189-1214, :1653-1667; in-kernel scale rule :754-789;
// encode :2266-2308) for the operand state "dynamic X, prequantized W" (rtx/fp8.py:1269-1302).
//
// Built on the CTA-pair kernel (cluster of two, tcgen05 cta_group::2, 256 x 256 pair tiles) with a
// third role:
//   warp 0       TMA producer: B payload and B scale tiles only
//   warp 1       MMA issuer (rank 0 of the pair), scale copies shared -> TMEM
//   warps 2..5   epilogue
//   warps 6..13  quantizers: global BF16 -> registers -> per-32 |max| by two shuffles -> E8M0 rule ->
//                cvt.rn.satfinite.e4m3x2 -> the ring slot's A tile (128-byte swizzle written by hand)
//                and its 512-byte scale tile -> fence.proxy.async -> arrive on the pair's `full`
//                barrier (the rank-1 CTA's warps arrive remotely).
// The bits are those of the row quantizer followed by the packed GEMM: same scale rule, same
// converter, same K order.  Every CTA quantizes its 128 rows of X once per column tile it visits,
// so X is re-quantized N / 256 times; this is the cost the quantize-once pipeline avoids, and why
// this kernel is a candidate only where few column tiles exist.
#pragma once

#include "gemm_blockscaled.cuh"
#include "quant.cuh"

namespace rtxb {

constexpr int kFusedQuantWarps = 8;
constexpr int kFusedQuantThreads = kGemmThreads + 32 * kFusedQuantWarps;   // 448

struct FusedAParams {
  const __nv_bfloat16* x;   // [m, k] BF16, row pitch ldx elements
  int64_t ldx;
  int k;                    // logical K (values)
  int vec_ok;               // x and its pitch allow 16-byte loads
  int round_to_infinity;
};

__device__ __forceinline__ void mbar_arrive_release_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kFusedQuantThreads, 1)
gemm_mxfp8_fused_a_pair_kernel(const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_sfb,
                               const GemmParams p, const FusedAParams fa) {
  constexpr int KIND = kKindMxfp8;
  using T = PairTraits<KIND>;
  using TP = TmemPlan<KIND>;
  constexpr int S = T::kStagesP;
  constexpr int KS = T::kStepsPerBarrierP;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + T::kOffBars);
  uint64_t* full_bar = bars;              // [S] rank 0: B loads of both CTAs landed AND both CTAs' A tiles written
  uint64_t* empty_bar = bars + S;         // [S] each CTA: slots free again
  uint64_t* acc_full_bar = bars + 2 * S;
  uint64_t* acc_overlap_bar = acc_full_bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_overlap_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int m_pairs = (p.m_tiles + 1) >> 1;
  const int total_tiles = m_pairs * p.n_tiles;
  const int k_groups = (p.k_tiles + KS - 1) / KS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full_bar[s], 1 + 2 * kFusedQuantWarps);   // the producer's expect_tx + one arrival per quantizer warp
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full_bar, 1);
    mbar_init(acc_overlap_bar, 8);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer: B and its scales ------------------------------
    const bool leader = elect_one_sync();
    if (leader) {
      prefetch_tensormap(&map_b);
      prefetch_tensormap(&map_sfb);
    }
    int group = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = pair_id; tile < total_tiles && ok; tile += num_pairs) {
      int mp_idx, n_idx;
      tile_coords(tile, m_pairs, p.n_tiles, p.group_m, mp_idx, n_idx);
      int b_blk0, b_blk1;
      if (epi_is_glu(EPI)) {
        b_blk0 = n_idx;
        b_blk1 = (p.glu_inter >> 7) + n_idx;
      } else {
        b_blk0 = n_idx * 2;
        b_blk1 = b_blk0 + 1;
      }
      const int b_mine = rank == 0 ? b_blk0 : b_blk1;
      for (int kg = 0; kg < k_groups; ++kg) {
        if (!mbar_wait(&empty_bar[group], phase ^ 1, abort_flag)) {
          if (p.status && leader) atomicCAS(p.status, 0, kStatusWaitProducer);
          *abort_flag = 1;
          ok = false;
          break;
        }
        if (leader) {
          const uint32_t full_addr = mapa_shared(smem_u32(&full_bar[group]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[group], 2 * KS * (T::kBBytes + T::kSfbBytes));
          const int slot0 = group * KS;
          const int kt0 = kg * KS;
          if (p.map3d) {
            tma_load_3d_pair(smem + T::kOffB + slot0 * T::kBBytes, &map_b, full_addr, 0, b_mine * 128, kt0);
          } else {
#pragma unroll
            for (int sub = 0; sub < KS; ++sub)
              tma_load_2d_pair(smem + T::kOffB + (slot0 + sub) * T::kBBytes, &map_b, full_addr,
                               (kt0 + sub) * kBlockKBytes, b_mine * 128);
          }
          const int sf_col = kt0 * T::kSfChunks;
          if (p.sfb3d) {
            tma_load_3d_pair(smem + T::kOffSfb + slot0 * T::kSfbBytes, &map_sfb, full_addr, 0,
                             b_blk0 * p.sf_k_chunks + sf_col, 0);
          } else {
            tma_load_2d_pair(smem + T::kOffSfb + slot0 * T::kSfbBytes, &map_sfb, full_addr, 0,
                             b_blk0 * p.sf_k_chunks + sf_col);
            tma_load_2d_pair(smem + T::kOffSfb + slot0 * T::kSfbBytes + KS * T::kSfaBytes, &map_sfb, full_addr, 0,
                             b_blk1 * p.sf_k_chunks + sf_col);
          }
        }
        __syncwarp();
        if (++group == S / KS) { group = 0; phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (rank 0 only) ------------------------------
    if (rank == 0) {
      mma_issuer_loop<KIND, true, S, KS, T::kABytes, T::kBBytes, T::kOffB, T::kOffSfa, T::kOffSfb, T::kSfaBytes,
                      T::kSfbBytes>(p, smem, full_bar, empty_bar, acc_full_bar, acc_overlap_bar, abort_flag, tmem_base,
                                    T::kIdesc, pair_id, num_pairs, total_tiles);
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    const int quad = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const float out_scale = p.out_scale ? __ldg(p.out_scale) : 1.0f;
    const uint32_t overlap_addr = mapa_shared(smem_u32(acc_overlap_bar), 0);
    uint32_t local_tile = 0;
    for (int tile = pair_id; tile < total_tiles; tile += num_pairs, ++local_tile) {
      int mp_idx, n_idx;
      tile_coords(tile, m_pairs, p.n_tiles, p.group_m, mp_idx, n_idx);
      const int row = (mp_idx * 2 + static_cast<int>(rank)) * 128 + quad * 32 + lane;
      const bool row_ok = row < p.m;
      const uint32_t acc_col = (local_tile & 1) ? TP::kAccWindow1 : 0;
      if (!mbar_wait(acc_full_bar, local_tile & 1, abort_flag)) {
        if (p.status && lane == 0) atomicCAS(p.status, 0, kStatusWaitEpilogue);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      epilogue_drain<KIND, EPI>(p, tmem_base + lane_base + acc_col, row, row_ok, n_idx, (local_tile & 1) != 0,
                                overlap_addr, out_scale, lane);
    }
  } else {
    // ------------------------------ quantizers (both CTAs) ------------------------------
    // One K step of this CTA's A tile is 128 rows x 128 values.  Sixteen lanes cover a row (eight values
    // = one 16-byte load each, four lanes per MX block), a warp covers two rows per pass, the eight
    // warps sixteen; eight passes per K step, all eight loads of a thread in flight before the first
    // is used.
    const int qwarp = warp - 6;
    const int half = lane >> 4;          // which of the warp's two rows
    const int l16 = lane & 15;           // 16-byte column chunk within the K step
    const uint32_t full_remote = mapa_shared(smem_u32(&full_bar[0]), 0);
    const bool rti = fa.round_to_infinity != 0;
    int group = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = pair_id; tile < total_tiles && ok; tile += num_pairs) {
      int mp_idx, n_idx;
      tile_coords(tile, m_pairs, p.n_tiles, p.group_m, mp_idx, n_idx);
      const int row0 = (mp_idx * 2 + static_cast<int>(rank)) * 128;
      for (int kg = 0; kg < k_groups; ++kg) {
        if (!mbar_wait(&empty_bar[group], phase ^ 1, abort_flag)) {
          if (p.status && lane == 0) atomicCAS(p.status, 0, kStatusWaitQuant);
          *abort_flag = 1;
          ok = false;
          break;
        }
#pragma unroll 1
        for (int sub = 0; sub < KS; ++sub) {
          const int kt = kg * KS + sub;
          if (kt >= p.k_tiles) break;     // never issued by the MMA warp either
          uint8_t* a_tile = smem + (group * KS + sub) * T::kABytes;
          uint8_t* sf_tile = smem + T::kOffSfa + (group * KS + sub) * T::kSfaBytes;
          const int col = kt * 128 + l16 * 8;
          uint4 raw[8];
#pragma unroll
          for (int pass = 0; pass < 8; ++pass) {
            const int r = pass * 16 + qwarp * 2 + half;
            const int row = row0 + r;
            raw[pass] = row < p.m ? load8_raw(fa.x + static_cast<int64_t>(row) * fa.ldx, col, fa.k, fa.vec_ok != 0)
                                  : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int pass = 0; pass < 8; ++pass) {
            const int r = pass * 16 + qwarp * 2 + half;
            float v[8];
            unpack8(raw[pass], v);
            float a = amax8(v);
            a = fmax_nan(a, __shfl_xor_sync(0xffffffffu, a, 1));
            a = fmax_nan(a, __shfl_xor_sync(0xffffffffu, a, 2));
            const uint32_t code = e8m0_from_amax(a, rti);
            const float recip = e8m0_reciprocal(code);
            const uint32_t w0 = cvt_e4m3x2(v[0] * recip, v[1] * recip) | (cvt_e4m3x2(v[2] * recip, v[3] * recip) << 16);
            const uint32_t w1 = cvt_e4m3x2(v[4] * recip, v[5] * recip) | (cvt_e4m3x2(v[6] * recip, v[7] * recip) << 16);
            // 128-byte swizzle: 16-byte chunk index XOR (row % 8); this lane's 8 bytes are half a chunk
            const int chunk = (l16 >> 1) ^ (r & 7);
            *reinterpret_cast<uint2*>(a_tile + r * kBlockKBytes + chunk * 16 + (l16 & 1) * 8) = make_uint2(w0, w1);
            // scale tile of the K step: byte (row % 32) * 16 + (row / 32) * 4 + block
            if ((l16 & 3) == 0) sf_tile[(r & 31) * 16 + (r >> 5) * 4 + (l16 >> 2)] = static_cast<uint8_t>(code);
          }
        }
        // generic-proxy writes -> visible to the tensor core's (async proxy) reads, then one arrival per warp
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive_release_cluster(full_remote + static_cast<uint32_t>(group) * 8u);
        if (++group == S / KS) { group = 0; phase ^= 1; }
      }
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace rtxb
