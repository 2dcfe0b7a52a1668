// Block-scaled GEMM on packed operands for sm_100a:
//   D[M,N] = epilogue( sum_k deq(A[M,K]) * deq(B[N,K]) )
// A, B are K-major payloads (MXFP8: one E4M3 byte per value, E8M0 scale per 32
// values; NVFP4: two E2M1 codes per byte, E4M3 scale per 16 values) with their
// scale factors in 128-row tiles.  Replaces the reference's warp-level
// mma.sync kernels MXFP8GemmKernel (rtx/kernels/mxfp8_gemm.py:45-2033) and
// NVFP4GemmKernel (rtx/kernels/nvfp4_gemm.py:22-64).
//
// One persistent CTA per SM, 192 threads:
//   warp 0      TMA producer: payload tiles (128-byte swizzled boxes) and
//               scale-factor tiles (1-D bulk copies) into a 4-stage ring
//   warp 1      owns TMEM; one lane copies scale factors shared->TMEM
//               (tcgen05.cp) and issues tcgen05.mma ... block_scale
//   warps 2..5  epilogue: tcgen05.ld the FP32 accumulators, apply the output
//               scale / SwiGLU, round once to BF16 (or keep FP32), store
// The 128x256 FP32 accumulator lives in TMEM.  Two accumulator windows
// [0,256) and [192,448) overlap by 64 columns; the epilogue drains the shared
// 64 columns of a tile first and then lets the next tile's MMAs start, so the
// rest of the drain overlaps the next main loop.  Scale factors use columns
// [448,512).
#pragma once

#include "common.cuh"

namespace rtxb {

enum GemmKind : int { kKindMxfp8 = 0, kKindNvfp4 = 1 };
enum GemmEpilogue : int {
  kEpiBf16 = 0,   // D bf16 = acc * out_scale
  kEpiF32 = 1,    // D f32  = acc * out_scale
  kEpiGluBf16 = 2 // D bf16[M, N/2] = silu(acc[:, gate]) * acc[:, up]
};

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kBlockKBytes = 128;  // one swizzle row: 128 E4M3 values or 256 E2M1 values
constexpr int kStages = 4;
constexpr int kGemmThreads = 192;
constexpr int kAccCols = 256;
constexpr int kAccWindow1 = 192;   // second accumulator window starts here
constexpr int kOverlapCols = 64;   // columns shared by both windows: [192,256)
constexpr int kSfColBase = 448;
constexpr int kTmemCols = 512;

template <int KIND>
struct GemmTraits {
  // bytes of scale factors per 128 rows per K tile: MXFP8 4 blocks of 32,
  // NVFP4 16 blocks of 16 -> 1 or 4 tiles of 512 bytes
  static constexpr int kSfChunks = KIND == kKindMxfp8 ? 1 : 4;
  static constexpr int kSfaBytes = 512 * kSfChunks;
  static constexpr int kSfbBytes = 2 * kSfaBytes;
  static constexpr int kABytes = kBlockM * kBlockKBytes;
  static constexpr int kBBytes = kBlockN * kBlockKBytes;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  // ring layout: [A x stages][B x stages][SFA x stages][SFB x stages][barriers];
  // payload tiles stay 1024-byte aligned (swizzle atoms), scale tiles 16-byte aligned
  static constexpr int kOffB = kStages * kABytes;
  static constexpr int kOffSfa = kOffB + kStages * kBBytes;
  static constexpr int kOffSfb = kOffSfa + kStages * kSfaBytes;
  static constexpr int kOffBars = kOffSfb + kStages * kSfbBytes;
  static constexpr int kSmemBytes = kOffBars + 1024 /*align slack*/ + 256 /*barriers*/;
  static constexpr int kSfaCol = kSfColBase;                 // 4 (MX) or 16 (NV) columns
  static constexpr int kSfbCol = kSfColBase + 4 * kSfChunks; // 8 (MX) or 32 (NV) columns
  static constexpr uint32_t kIdesc =
      idesc_block_scaled(kBlockM, kBlockN, KIND == kKindMxfp8 ? 0u : 1u, KIND == kKindMxfp8 ? 1u : 0u);
};

struct GemmParams {
  int m, n, k_tiles;      // n = rows of B (for GLU: 2 * inter); k_tiles = ceil(Kbytes / 128)
  int m_tiles, n_tiles;   // n_tiles counts 256-wide accumulator tiles
  int glu_inter;          // GLU: rows of the gate half of B (= output columns); else 0
  const uint8_t* sfa;     // [ceil(M/128)][sf_k_chunks][512]
  const uint8_t* sfb;     // [ceil(N/128)][sf_k_chunks][512]
  int sf_k_chunks;        // 512-byte tiles per 128 rows along K (whole tensor)
  void* out;              // bf16 or f32, row pitch ldo elements
  int64_t ldo;
  int out_cols;           // n, or inter for GLU
  int out_vec_ok;         // 1 when out and its row pitch are 16-byte aligned (vector stores allowed)
  const float* out_scale; // device scalar or nullptr (= 1)
  int* status;            // device status word or nullptr
};

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }

template <int KIND, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_blockscaled_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const GemmParams p) {
  using T = GemmTraits<KIND>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + T::kOffBars);
  uint64_t* full_bar = bars;                  // [kStages] TMA -> MMA
  uint64_t* empty_bar = bars + kStages;       // [kStages] MMA -> TMA
  uint64_t* acc_full_bar = bars + 2 * kStages;     // MMA -> epilogue (tile accumulated)
  uint64_t* acc_overlap_bar = acc_full_bar + 1;    // epilogue -> MMA (shared columns drained)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_overlap_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_tiles = p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full_bar, 1);
    mbar_init(acc_overlap_bar, 4);  // one arrival per epilogue warp
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int m_idx = tile % p.m_tiles, n_idx = tile / p.m_tiles;
        const int m0 = m_idx * kBlockM;
        // rows of B feeding accumulator columns [0,128) and [128,256)
        int b_row0, b_row1;
        if (EPI == kEpiGluBf16) {
          b_row0 = n_idx * 128;
          b_row1 = p.glu_inter + n_idx * 128;
        } else {
          b_row0 = n_idx * kBlockN;
          b_row1 = b_row0 + 128;
        }
        const uint8_t* sfa_src = p.sfa + static_cast<size_t>(m_idx) * p.sf_k_chunks * 512;
        const uint8_t* sfb_src0 = p.sfb + static_cast<size_t>(b_row0 >> 7) * p.sf_k_chunks * 512;
        const uint8_t* sfb_src1 = p.sfb + static_cast<size_t>(b_row1 >> 7) * p.sf_k_chunks * 512;
        const bool b1_valid = b_row1 < p.n;  // second half may lie past the last row of B
        for (int kt = 0; kt < p.k_tiles; ++kt) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            if (p.status) atomicCAS(p.status, 0, kStatusWaitProducer);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * T::kABytes;
          uint8_t* sb = smem + T::kOffB + stage * T::kBBytes;
          uint8_t* ssfa = smem + T::kOffSfa + stage * T::kSfaBytes;
          uint8_t* ssfb = smem + T::kOffSfb + stage * T::kSfbBytes;
          mbar_expect_tx(&full_bar[stage], T::kABytes + T::kBBytes + T::kSfaBytes +
                                               (b1_valid ? T::kSfbBytes : T::kSfaBytes));
          tma_load_2d(sa, &map_a, &full_bar[stage], kt * kBlockKBytes, m0);
          tma_load_2d(sb, &map_b, &full_bar[stage], kt * kBlockKBytes, b_row0);
          tma_load_2d(sb + 128 * kBlockKBytes, &map_b, &full_bar[stage], kt * kBlockKBytes, b_row1);
          const size_t sf_off = static_cast<size_t>(kt) * T::kSfaBytes;
          bulk_load_1d(ssfa, sfa_src + sf_off, T::kSfaBytes, &full_bar[stage]);
          bulk_load_1d(ssfb, sfb_src0 + sf_off, T::kSfaBytes, &full_bar[stage]);
          if (b1_valid) bulk_load_1d(ssfb + T::kSfaBytes, sfb_src1 + sf_off, T::kSfaBytes, &full_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local_tile) {
        const uint32_t acc_col = (local_tile & 1) ? kAccWindow1 : 0;
        if (local_tile > 0) {
          // previous tile's epilogue has drained the columns both windows share
          if (!mbar_wait(acc_overlap_bar, (local_tile - 1) & 1, abort_flag)) {
            if (p.status) atomicCAS(p.status, 0, kStatusWaitMma);
            *abort_flag = 1;
            break;
          }
          tc_fence_after_sync();
        }
        for (int kt = 0; kt < p.k_tiles; ++kt) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            if (p.status) atomicCAS(p.status, 0, kStatusWaitMma);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * T::kABytes);
          const uint32_t sb = smem_u32(smem + T::kOffB + stage * T::kBBytes);
          const uint32_t ssfa = smem_u32(smem + T::kOffSfa + stage * T::kSfaBytes);
          const uint32_t ssfb = smem_u32(smem + T::kOffSfb + stage * T::kSfbBytes);
          // scale factors: each 512-byte tile -> 4 TMEM columns.
          // SFA tile c -> columns kSfaCol + 4c; SFB (row block nb, tile c) -> kSfbCol + 8c + 4nb.
#pragma unroll
          for (int c = 0; c < T::kSfChunks; ++c) {
            tc_cp_32x128b_warpx4(tmem_base + T::kSfaCol + 4 * c, umma_desc_sf(ssfa + 512 * c));
            tc_cp_32x128b_warpx4(tmem_base + T::kSfbCol + 8 * c, umma_desc_sf(ssfb + 512 * c));
            tc_cp_32x128b_warpx4(tmem_base + T::kSfbCol + 8 * c + 4, umma_desc_sf(ssfb + T::kSfaBytes + 512 * c));
          }
          const uint64_t da = umma_desc_sw128(sa);
          const uint64_t db = umma_desc_sw128(sb);
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // four MMAs of 32 bytes of K each
            const uint32_t acc = (kt > 0 || j > 0) ? 1u : 0u;
            if (KIND == kKindMxfp8) {
              // one scale byte per row per MMA: byte j of the 32-bit column
              tc_mma_mxf8f6f4(tmem_base + acc_col, da + 2 * j, db + 2 * j, idesc_with_sf_ids(T::kIdesc, j, j),
                              tmem_base + T::kSfaCol, tmem_base + T::kSfbCol, acc);
            } else {
              // four scale bytes per row per MMA: a whole column group per MMA
              tc_mma_mxf4nvf4(tmem_base + acc_col, da + 2 * j, db + 2 * j, T::kIdesc,
                              tmem_base + T::kSfaCol + 4 * j, tmem_base + T::kSfbCol + 8 * j, acc);
            }
          }
          tc_commit(&empty_bar[stage]);  // stage reusable once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(acc_full_bar);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const float out_scale = p.out_scale ? __ldg(p.out_scale) : 1.0f;
    uint32_t local_tile = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local_tile) {
      const int m_idx = tile % p.m_tiles, n_idx = tile / p.m_tiles;
      const int row = m_idx * kBlockM + quad * 32 + lane;
      const bool row_ok = row < p.m;
      const uint32_t acc_col = (local_tile & 1) ? kAccWindow1 : 0;
      // local column where the shared 64 columns start for this window
      const int shared0 = (local_tile & 1) ? 0 : kAccWindow1;
      if (!mbar_wait(acc_full_bar, local_tile & 1, abort_flag)) {
        if (p.status && lane == 0) atomicCAS(p.status, 0, kStatusWaitEpilogue);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      const uint32_t tacc = tmem_base + lane_base + acc_col;

      if (EPI == kEpiGluBf16) {
        // accumulator columns [0,128) = gate, [128,256) = up, same output columns
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(row) * p.ldo;
        const int col0 = n_idx * 128;
        uint32_t held[2][32];
        // 1) read the shared columns first and release them
        //    window 0: up columns 64..127 (local 192..255); window 1: gate columns 0..63
        tmem_ld_32x32(tacc + shared0, held[0]);
        tmem_ld_32x32(tacc + shared0 + 32, held[1]);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_overlap_bar);
        const int c_first = (local_tile & 1) ? 0 : 64;  // gate/up column pair index of the held data
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t other[32];
          const int c = c_first + 32 * h;
          tmem_ld_32x32(tacc + ((local_tile & 1) ? 128 + c : c), other);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 32; v += 8) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float g0 = __uint_as_float((local_tile & 1) ? held[h][v + 2 * e] : other[v + 2 * e]);
                float u0 = __uint_as_float((local_tile & 1) ? other[v + 2 * e] : held[h][v + 2 * e]);
                float g1 = __uint_as_float((local_tile & 1) ? held[h][v + 2 * e + 1] : other[v + 2 * e + 1]);
                float u1 = __uint_as_float((local_tile & 1) ? other[v + 2 * e + 1] : held[h][v + 2 * e + 1]);
                __nv_bfloat162 b = __floats2bfloat162_rn(silu_mul(g0, u0), silu_mul(g1, u1));
                w[e] = *reinterpret_cast<uint32_t*>(&b);
              }
              const int col = col0 + c + v;
              if (p.out_vec_ok && col + 8 <= p.out_cols) {
                *reinterpret_cast<uint4*>(out + col) = make_uint4(w[0], w[1], w[2], w[3]);
              } else {
                for (int e = 0; e < 8; ++e)
                  if (col + e < p.out_cols)
                    out[col + e] = reinterpret_cast<__nv_bfloat16*>(w)[e];
              }
            }
          }
        }
        // 2) the remaining 64 column pairs
        const int c_rest = (local_tile & 1) ? 64 : 0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t g[32], u[32];
          const int c = c_rest + 32 * h;
          tmem_ld_32x32(tacc + c, g);
          tmem_ld_32x32(tacc + 128 + c, u);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 32; v += 8) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                __nv_bfloat162 b = __floats2bfloat162_rn(
                    silu_mul(__uint_as_float(g[v + 2 * e]), __uint_as_float(u[v + 2 * e])),
                    silu_mul(__uint_as_float(g[v + 2 * e + 1]), __uint_as_float(u[v + 2 * e + 1])));
                w[e] = *reinterpret_cast<uint32_t*>(&b);
              }
              const int col = col0 + c + v;
              if (p.out_vec_ok && col + 8 <= p.out_cols) {
                *reinterpret_cast<uint4*>(out + col) = make_uint4(w[0], w[1], w[2], w[3]);
              } else {
                for (int e = 0; e < 8; ++e)
                  if (col + e < p.out_cols)
                    out[col + e] = reinterpret_cast<__nv_bfloat16*>(w)[e];
              }
            }
          }
        }
      } else {
        const int col_base = n_idx * kBlockN;
#pragma unroll 1
        for (int i = 0; i < kAccCols / 32; ++i) {
          // visit the two shared 32-column groups first, then the rest in order
          const int c = (shared0 + 32 * i) % kAccCols;
          uint32_t r[32];
          tmem_ld_32x32(tacc + c, r);
          tmem_ld_wait();
          if (i == 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_overlap_bar);
          }
          if (!row_ok) continue;
          const int col = col_base + c;
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
              if (p.out_vec_ok && col + v + 8 <= p.out_cols) {
                *reinterpret_cast<uint4*>(out + col + v) = make_uint4(w[0], w[1], w[2], w[3]);
              } else {
                for (int e = 0; e < 8; ++e)
                  if (col + v + e < p.out_cols)
                    out[col + v + e] = reinterpret_cast<__nv_bfloat16*>(w)[e];
              }
            }
          } else {
            float* out = reinterpret_cast<float*>(p.out) + static_cast<int64_t>(row) * p.ldo;
#pragma unroll
            for (int v = 0; v < 32; v += 4) {
              if (p.out_vec_ok && col + v + 4 <= p.out_cols) {
                *reinterpret_cast<float4*>(out + col + v) =
                    make_float4(__uint_as_float(r[v]) * out_scale, __uint_as_float(r[v + 1]) * out_scale,
                                __uint_as_float(r[v + 2]) * out_scale, __uint_as_float(r[v + 3]) * out_scale);
              } else {
                for (int e = 0; e < 4; ++e)
                  if (col + v + e < p.out_cols) out[col + v + e] = __uint_as_float(r[v + e]) * out_scale;
              }
            }
          }
        }
      }
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace rtxb
