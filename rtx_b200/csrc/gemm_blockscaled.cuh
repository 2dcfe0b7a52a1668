// Block-scaled GEMM on packed operands for sm_100a:
//   D[M,N] = epilogue( sum_k deq(A[M,K]) * deq(B[N,K]) )
// A, B are K-major payloads (MXFP8: one E4M3 byte per value, E8M0 scale per 32
// values; NVFP4: two E2M1 codes per byte, E4M3 scale per 16 values) with their
// scale factors in 128-row tiles.  Replaces the reference's warp-level
// mma.sync kernels MXFP8GemmKernel (rtx/kernels/mxfp8_gemm.py:45-2033) and
// NVFP4GemmKernel (rtx/kernels/nvfp4_gemm.py:22-64).
//
// Two kernels share the roles, the TMEM plan and the epilogue:
//   gemm_blockscaled_kernel       one CTA per 128 x 256 tile (tcgen05 cta_group::1)
//   gemm_blockscaled_pair_kernel  a cluster of two CTAs per 256 x 256 tile (cta_group::2)
// Persistent CTAs, 192 threads:
//   warp 0      TMA producer: payload tiles (128-byte swizzled boxes) and
//               scale-factor tiles into a multi-stage ring
//   warp 1      owns TMEM; one lane copies scale factors shared->TMEM
//               (tcgen05.cp) and issues tcgen05.mma ... block_scale
//   warps 2..5  epilogue: tcgen05.ld the FP32 accumulators, apply the output
//               scale / SwiGLU, round once to BF16 (or keep FP32), store
//
// TMEM plan (512 columns): scale factors sit at the top in two sets that
// alternate per K step (so the copy for step i+1 never overwrites what the MMAs
// of step i read); the 128 x 256 FP32 accumulator uses one of two windows,
// [0,256) and [W1, W1+256), that alternate per tile and overlap by 256-W1
// columns.  The epilogue drains the shared columns of a tile first and then lets
// the next tile's MMAs start, so the rest of the drain overlaps the next main loop.
#pragma once

#include "common.cuh"

namespace rtxb {

enum GemmKind : int { kKindMxfp8 = 0, kKindNvfp4 = 1 };
enum GemmEpilogue : int {
  kEpiBf16 = 0,   // D bf16 = acc * out_scale
  kEpiF32 = 1,    // D f32  = acc * out_scale
  kEpiGluBf16 = 2, // D bf16[M, N/2] = silu(acc[:, gate]) * acc[:, up]
  kEpiGluMx = 3,   // the same H, also (or only) emitted as MXFP8: E4M3 payload + E8M0 scale tiles
  kEpiRegionBf16 = 4  // D bf16 = acc * (x_region_scale[row / Rx] * w_region_scale[col / Rw])  (NVFP4 row-region policy)
};
__host__ __device__ constexpr bool epi_is_glu(int epi) { return epi == kEpiGluBf16 || epi == kEpiGluMx; }

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kBlockKBytes = 128;  // one swizzle row: 128 E4M3 values or 256 E2M1 values
constexpr int kStages = 4;        // ring slots (one K step each) of the single-CTA kernel
// K steps handed over per full/empty barrier and ring slots of the pair kernel, per operand format
constexpr int kSingleStepsMx = 2, kSingleStepsNv = 1;
constexpr int kPairStepsMx = 2, kPairStepsNv = 1;
constexpr int kPairSlotsMx = 6, kPairSlotsNv = 5;
constexpr int kGemmThreads = 192;
// Output staging for the TMA-store epilogue: per epilogue warp two buffers of 32 rows x 64 bytes
// (64-byte swizzle), so one 32-column BF16 chunk is in flight to global memory while the next is written.
constexpr int kEpiStageBufBytes = 32 * 64;
constexpr int kEpiStageBytes = 4 * 2 * kEpiStageBufBytes;   // 16 KB
constexpr int kMaxOutBlocks = 8;
struct OutMaps {
  CUtensorMap m[kMaxOutBlocks];   // m[0]: the whole output, or one map per block of rows (GemmParams::out_block_rows)
};
__device__ __forceinline__ int rotate_tile(int tile, int shift, int total) {
  tile += shift;
  return tile >= total ? tile - total : tile;
}
constexpr int kAccCols = 256;
constexpr int kTmemCols = 512;

template <int KIND>
struct TmemPlan {
  // 512-byte scale tiles per 128 rows per K step: MXFP8 4 blocks of 32 -> 1, NVFP4 16 blocks of 16 -> 4
  static constexpr int kSfChunks = KIND == kKindMxfp8 ? 1 : 4;
  static constexpr int kSfSetCols = KIND == kKindMxfp8 ? 16 : 48;  // SFA 4c + SFB 8c columns (c = chunks), padded
  static constexpr int kSfBase = kTmemCols - 2 * kSfSetCols;       // 480 / 416
  static constexpr int kAccWindow1 = kSfBase - kAccCols;           // 224 / 160
  static constexpr int kOverlapChunks = (kAccCols - kAccWindow1) / 32;  // 1 / 3 groups of 32 shared columns
  __device__ static constexpr int sfa_col(int set) { return kSfBase + set * kSfSetCols; }
  __device__ static constexpr int sfb_col(int set) { return kSfBase + set * kSfSetCols + 4 * kSfChunks; }
};

template <int KIND>
struct GemmTraits {
  static constexpr int kSfChunks = TmemPlan<KIND>::kSfChunks;
  static constexpr int kSfaBytes = 512 * kSfChunks;
  static constexpr int kSfbBytes = 2 * kSfaBytes;
  static constexpr int kABytes = kBlockM * kBlockKBytes;
  static constexpr int kBBytes = kBlockN * kBlockKBytes;
  // ring layout: [A x stages][B x stages][SFA x stages][SFB x stages][barriers];
  // payload tiles stay 1024-byte aligned (swizzle atoms), scale tiles 16-byte aligned
  static constexpr int kOffB = kStages * kABytes;
  static constexpr int kOffSfa = kOffB + kStages * kBBytes;
  static constexpr int kOffSfb = kOffSfa + kStages * kSfaBytes;
  static constexpr int kOffBars = kOffSfb + kStages * kSfbBytes;
  // no output staging here: with four ring slots of 48 KB the NVFP4 form already fills shared memory, and this
  // kernel serves single row blocks (M <= 128), whose output is small; it keeps the direct stores
  static constexpr int kSmemBytes = kOffBars + 1024 /*align slack*/ + 256 /*barriers*/;
  static constexpr int kStepsPerBarrier = KIND == kKindMxfp8 ? kSingleStepsMx : kSingleStepsNv;
  static constexpr uint32_t kIdesc =
      idesc_block_scaled(kBlockM, kBlockN, KIND == kKindMxfp8 ? 0u : 1u, KIND == kKindMxfp8 ? 1u : 0u);
};

struct GemmParams {
  int m, n, k_tiles;      // n = rows of B (for GLU: 2 * inter); k_tiles = ceil(Kbytes / 128)
  int m_tiles, n_tiles;   // 128-row blocks of A; 256-wide accumulator tiles
  int group_m;            // raster: M blocks (pairs) per group; a group's A panel stays L2 resident while
                          // the group walks every N tile
  int glu_inter;          // GLU: rows of the gate half of B (= output columns); else 0
  const uint8_t* sfa;     // [ceil(M/128)][sf_k_chunks][512]
  const uint8_t* sfb;     // [ceil(N/128)][sf_k_chunks][512]
  int sf_k_chunks;        // 512-byte tiles per 128 rows along K (whole tensor)
  void* out;              // bf16 or f32, row pitch ldo elements
  int64_t ldo;
  int out_cols;           // n, or inter for GLU
  int out_vec_ok;         // 1 when out and its row pitch are 16-byte aligned (vector stores allowed)
  int tma_out;            // 1: BF16 / FP32 outputs leave through shared memory and TMA stores (needs out_vec_ok)
  int out_block_rows;     // pair kernel, TMA outputs: > 0 = the output is split into blocks of this many rows (a
                          // multiple of 256), block j described by output map j (e.g. buffers on different GPUs)
  int tile_shift;         // pair kernel: the tile order is rotated by this many tiles (ranks that write blocks to
                          // one another start at different owners)
  const float* out_scale; // device scalar or nullptr (= 1)
  const float* x_region_scales;  // kEpiRegionBf16: FP32 outer scale per x_region_rows rows of A
  const float* w_region_scales;  // kEpiRegionBf16: FP32 outer scale per w_region_rows rows of B (output columns)
  int x_region_rows, w_region_rows;
  uint8_t* q_out;         // kEpiGluMx: E4M3 payload of H, [M, out_cols] (out may then be nullptr)
  uint8_t* sf_out;        // kEpiGluMx: E8M0 scales of H in 128-row tiles, sf_out_chunks tiles per row block
  int sf_out_chunks;
  int* status;            // device status word or nullptr
  int a_box_rows;         // kernels for one row block (M <= 128): rows of A fetched per K step (M rounded up to 8)
  int slots;              // streaming kernel: ring slots that fit shared memory with that A box
  int ks;                 // streaming kernel: K steps per ring slot
  int map3d;              // streaming and pair kernels: payload maps are [K/128][rows][128] views (one load per
                          // operand brings all K steps of a ring slot / barrier group)
  int b_box256;           // single-CTA kernel: the map of B has 256-row boxes (both halves of a tile in one load)
  int sfb3d;              // pair kernel: the scale map of B is 3-D, third coordinate = half of the 256-wide tile
  int overlap_previous;   // streaming kernel: launched as a programmatic dependent; A / SFA / out_scale may
                          // come from the grid before it, B / SFB do not
};

// Tile order: groups of `group_m` M blocks; inside a group M runs fastest, then N.  CTAs that run at
// the same time then share one or two B tiles and a group-sized A panel that fits L2.
__device__ __forceinline__ void tile_coords(int tile, int m_count, int n_tiles, int group_m, int& m_idx, int& n_idx) {
  const int per_group = group_m * n_tiles;
  const int g = tile / per_group;
  const int r = tile - g * per_group;
  const int m_in_group = min(group_m, m_count - g * group_m);
  n_idx = r / m_in_group;
  m_idx = g * group_m + (r - n_idx * m_in_group);
}

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }

__device__ __forceinline__ void store_bf16x8(__nv_bfloat16* out, int col, int out_cols, bool vec_ok,
                                             const uint32_t (&w)[4]) {
  if (vec_ok && col + 8 <= out_cols) {
    *reinterpret_cast<uint4*>(out + col) = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
    for (int e = 0; e < 8; ++e)
      if (col + e < out_cols) out[col + e] = reinterpret_cast<const __nv_bfloat16*>(w)[e];
  }
}

// Drains one 128 x 256 accumulator window of this warp's 32 TMEM lanes.  `tacc` already holds the
// lane quadrant and the window's first column.  The columns the two windows share are at the top of
// the even window and at the bottom of the odd one; they are read first and `overlap_bar_addr` is
// signalled as soon as they are in registers.
template <int KIND, int EPI>
__device__ __forceinline__ void epilogue_drain(const GemmParams& p, uint32_t tacc, int row, bool row_ok, int n_idx,
                                               bool odd, uint32_t overlap_bar_addr, float out_scale, int lane,
                                               const CUtensorMap* map_out = nullptr, uint8_t* stage = nullptr,
                                               int out_row0 = 0) {
  // out_row0: first row of the output block `map_out` describes (0 when it describes the whole output)
  using TP = TmemPlan<KIND>;
  if (epi_is_glu(EPI)) {
    // accumulator columns [0,128) = gate, [128,256) = up of the same 128 output columns; pairs of
    // 32-column groups (gate c, up 128+c).  Shared columns: up group 96 (even window) or gate
    // group 0 (odd window) -- the first pair visited holds them.
    static_assert(!epi_is_glu(EPI) || TP::kOverlapChunks == 1, "GLU epilogue assumes a 32-column overlap");
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(row) * p.ldo;
    const int col0 = n_idx * 128;
    const int c_first = odd ? 0 : 96;
    uint32_t scale_word = 0;  // kEpiGluMx: the four E8M0 codes of this row's blocks col0/32 .. col0/32+3
#pragma unroll 1
    for (int i = 0; i < 4; ++i) {
      const int c = (c_first + 32 * i) & 127;
      uint32_t g[32], u[32];
      if (i == 0) {
        // only one of the two groups lies in the columns the windows share (up for the even window, gate for
        // the odd one): fetch it alone, release the next tile's MMAs, then fetch the other
        if (odd) tmem_ld_32x32(tacc + c, g);
        else tmem_ld_32x32(tacc + 128 + c, u);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(overlap_bar_addr);
        if (odd) tmem_ld_32x32(tacc + 128 + c, u);
        else tmem_ld_32x32(tacc + c, g);
        tmem_ld_wait();
      } else {
        tmem_ld_32x32(tacc + c, g);
        tmem_ld_32x32(tacc + 128 + c, u);
        tmem_ld_wait();
      }
      if (!row_ok) continue;
      // H in BF16 (one rounding of the FP32 result), packed two per word
      uint32_t hw[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        __nv_bfloat162 b = __floats2bfloat162_rn(silu_mul(__uint_as_float(g[2 * e]), __uint_as_float(u[2 * e])),
                                                 silu_mul(__uint_as_float(g[2 * e + 1]), __uint_as_float(u[2 * e + 1])));
        hw[e] = *reinterpret_cast<uint32_t*>(&b);
      }
      if (EPI == kEpiGluBf16 || p.out != nullptr) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint32_t w[4] = {hw[4 * v], hw[4 * v + 1], hw[4 * v + 2], hw[4 * v + 3]};
          store_bf16x8(out, col0 + c + 8 * v, p.out_cols, p.out_vec_ok != 0, w);
        }
      }
      if (EPI == kEpiGluMx) {
        // these 32 columns are exactly one MX block of H's row: quantize the BF16 values as the
        // row quantizer would (same scale rule, same converter)
        float a = 0.0f;
#pragma unroll
        for (int e = 0; e < 16; ++e) a = fmax_nan(a, fmax_nan(fabsf(bf16_lo(hw[e])), fabsf(bf16_hi(hw[e]))));
        const uint32_t code = e8m0_from_amax(a, true);
        const float recip = e8m0_reciprocal(code);
        scale_word |= code << (8 * (c >> 5));
        uint32_t q[8];
#pragma unroll
        for (int e = 0; e < 8; ++e)
          q[e] = cvt_e4m3x2(bf16_lo(hw[2 * e]) * recip, bf16_hi(hw[2 * e]) * recip) |
                 (cvt_e4m3x2(bf16_lo(hw[2 * e + 1]) * recip, bf16_hi(hw[2 * e + 1]) * recip) << 16);
        uint4* dst = reinterpret_cast<uint4*>(p.q_out + static_cast<int64_t>(row) * p.out_cols + col0 + c);
        dst[0] = make_uint4(q[0], q[1], q[2], q[3]);
        dst[1] = make_uint4(q[4], q[5], q[6], q[7]);
      }
    }
    if (EPI == kEpiGluMx) {
      // rows past M inside the last 128-row tile get zero scales (their payload is never read as non-zero)
      const int tile_row = row & 127;
      uint8_t* tile = p.sf_out + (static_cast<size_t>(row >> 7) * p.sf_out_chunks + n_idx) * 512;
      if ((row >> 7) < p.m_tiles)
        *reinterpret_cast<uint32_t*>(tile + (tile_row & 31) * 16 + (tile_row >> 5) * 4) = row_ok ? scale_word : 0u;
    }
  } else {
    const int shared0 = odd ? 0 : TP::kAccWindow1;  // local column where the shared columns start
    const int col_base = n_idx * kBlockN;
    const bool staged = p.tma_out != 0;
    // The 32-column groups both windows share are read into registers first, all of them, and the next
    // tile's MMAs are released before any of this tile's values is converted or stored.
    uint32_t held[TP::kOverlapChunks][32];
#pragma unroll
    for (int i = 0; i < TP::kOverlapChunks; ++i) tmem_ld_32x32(tacc + (shared0 + 32 * i) % kAccCols, held[i]);
    tmem_ld_wait();
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster(overlap_bar_addr);
    const int last_region = EPI == kEpiRegionBf16 ? (p.out_cols - 1) / p.w_region_rows : 0;
    // converts and stores one 32-column group `r` (local column c, i-th group visited)
    auto emit = [&](const int c, const int i, const uint32_t (&r)[32]) {
      if (!staged && !row_ok) return;
      const int col = col_base + c;
      // per-column factors: the launch-wide (or this row's) scale, times the column's region scale for the
      // NVFP4 row-region policy (the product of the two outer scales is formed first, then applied:
      // rtx/kernels/mxfp8_gemm.py:1720-1760; column scales are warp-uniform loads)
      float v[32];
      if (EPI == kEpiRegionBf16) {
        if (p.w_region_rows == 4) {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const float f = out_scale * __ldg(p.w_region_scales + min((col >> 2) + g, last_region));
#pragma unroll
            for (int e = 0; e < 4; ++e) v[4 * g + e] = __uint_as_float(r[4 * g + e]) * f;
          }
        } else {
          int widx = col / p.w_region_rows, wrem = col - widx * p.w_region_rows;
          float f = out_scale * __ldg(p.w_region_scales + min(widx, last_region));
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            v[e] = __uint_as_float(r[e]) * f;
            if (++wrem == p.w_region_rows) {
              wrem = 0;
              ++widx;
              f = out_scale * __ldg(p.w_region_scales + min(widx, last_region));
            }
          }
        }
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(r[e]) * out_scale;
      }
      if (EPI == kEpiF32) {
        if (staged) {
          // 32 rows x 128 bytes = both staging buffers as one box (128-byte swizzle: 16-byte chunk j of row r at
          // chunk j ^ (r % 8)), one store: whole 128-byte lines leave the SM, which is what a write over NVLink wants
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(stage + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(map_out, stage, col, row - lane - out_row0);
            tma_store_commit();
          }
        } else {
          float* out = reinterpret_cast<float*>(p.out) + static_cast<int64_t>(row) * p.ldo;
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            if (p.out_vec_ok && col + e + 4 <= p.out_cols) {
              *reinterpret_cast<float4*>(out + col + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
            } else {
              for (int q = 0; q < 4; ++q)
                if (col + e + q < p.out_cols) out[col + e + q] = v[e + q];
            }
          }
        }
      } else {
        uint32_t w[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
          w[e] = *reinterpret_cast<uint32_t*>(&b);
        }
        if (staged) {
          // this chunk's 32 rows x 64 bytes go to buffer i & 1; the store that read it two chunks ago is done
          uint8_t* buf = stage + (i & 1) * kEpiStageBufBytes;
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(buf + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) =
                make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(map_out, buf, col, row - lane - out_row0);
            tma_store_commit();
          }
        } else {
          __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(row) * p.ldo;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint32_t ww[4] = {w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]};
            store_bf16x8(out, col + 8 * q, p.out_cols, p.out_vec_ok != 0, ww);
          }
        }
      }
    };
    // the shared groups first (already in registers), then the rest in order
#pragma unroll
    for (int i = 0; i < TP::kOverlapChunks; ++i) emit((shared0 + 32 * i) % kAccCols, i, held[i]);
#pragma unroll 1
    for (int i = TP::kOverlapChunks; i < kAccCols / 32; ++i) {
      const int c = (shared0 + 32 * i) % kAccCols;
      uint32_t r[32];
      tmem_ld_32x32(tacc + c, r);
      tmem_ld_wait();
      emit(c, i, r);
    }
  }
}

// shared -> TMEM copy of one K step's scale factors into scale set `set`.
// SFA tile c -> columns sfa + 4c; SFB (row block nb, tile c) -> sfb + 8c + 4nb.
template <int KIND, bool PAIR>
__device__ __forceinline__ void issue_scale_copy(uint32_t tmem_base, uint32_t ssfa, uint32_t ssfb0, uint32_t ssfb1,
                                                 int set) {
  // ssfb0 / ssfb1: scale tiles of the B rows behind accumulator columns [0,128) and [128,256)
  using TP = TmemPlan<KIND>;
  const uint32_t ta = tmem_base + TP::sfa_col(set), tb = tmem_base + TP::sfb_col(set);
#pragma unroll
  for (int c = 0; c < TP::kSfChunks; ++c) {
    if (PAIR) {
      tc_cp_32x128b_warpx4_pair(ta + 4 * c, umma_desc_sf(ssfa + 512 * c));
      tc_cp_32x128b_warpx4_pair(tb + 8 * c, umma_desc_sf(ssfb0 + 512 * c));
      tc_cp_32x128b_warpx4_pair(tb + 8 * c + 4, umma_desc_sf(ssfb1 + 512 * c));
    } else {
      tc_cp_32x128b_warpx4(ta + 4 * c, umma_desc_sf(ssfa + 512 * c));
      tc_cp_32x128b_warpx4(tb + 8 * c, umma_desc_sf(ssfb0 + 512 * c));
      tc_cp_32x128b_warpx4(tb + 8 * c + 4, umma_desc_sf(ssfb1 + 512 * c));
    }
  }
}

// the four MMAs (32 bytes of K each) of one K step
template <int KIND, bool PAIR>
__device__ __forceinline__ void issue_k_step(uint32_t tmem_base, uint32_t acc_col, uint32_t sa, uint32_t sb, int set,
                                             uint32_t idesc, bool first_step) {
  using TP = TmemPlan<KIND>;
  const uint64_t da = umma_desc_sw128(sa);
  const uint64_t db = umma_desc_sw128(sb);
  const uint32_t ta = tmem_base + TP::sfa_col(set), tb = tmem_base + TP::sfb_col(set);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t acc = (!first_step || j > 0) ? 1u : 0u;
    if (KIND == kKindMxfp8) {
      // one scale byte per row per MMA: byte j of the 32-bit column
      if (PAIR)
        tc_mma_mxf8f6f4_pair(tmem_base + acc_col, da + 2 * j, db + 2 * j, idesc_with_sf_ids(idesc, j, j), ta, tb, acc);
      else
        tc_mma_mxf8f6f4(tmem_base + acc_col, da + 2 * j, db + 2 * j, idesc_with_sf_ids(idesc, j, j), ta, tb, acc);
    } else {
      // four scale bytes per row per MMA: a whole column group per MMA
      if (PAIR)
        tc_mma_mxf4nvf4_pair(tmem_base + acc_col, da + 2 * j, db + 2 * j, idesc, ta + 4 * j, tb + 8 * j, acc);
      else
        tc_mma_mxf4nvf4(tmem_base + acc_col, da + 2 * j, db + 2 * j, idesc, ta + 4 * j, tb + 8 * j, acc);
    }
  }
}

// The MMA issuer's loop over this CTA's (or pair's) tiles; the integer parameters describe the ring:
// SLOTS slots of one K step each (A, B, SFA, SFB), handed over in groups of KS slots per barrier,
// so one wait and one commit cover KS K steps (4 KS MMAs).
// All 32 lanes of the warp run it with identical control flow -- addresses, descriptors and loop
// state then stay in uniform registers, which is what keeps the issue cost of a tcgen05
// instruction low -- and one elected lane (always the same one) issues the tcgen05 instructions.
template <int KIND, bool PAIR, int SLOTS, int KS, int A_BYTES, int B_BYTES, int OFF_B, int OFF_SFA, int OFF_SFB,
          int SFA_BYTES, int SFB_BYTES>
__device__ __forceinline__ void mma_issuer_loop(const GemmParams& p, uint8_t* smem, uint64_t* full_bar,
                                                uint64_t* empty_bar, uint64_t* acc_full_bar, uint64_t* acc_overlap_bar,
                                                volatile int* abort_flag, uint32_t tmem_base, uint32_t idesc,
                                                int first_tile, int tile_stride, int total_tiles) {
  using TP = TmemPlan<KIND>;
  constexpr int GROUPS = SLOTS / KS;
  static_assert(SLOTS % KS == 0, "ring slots must split evenly into barrier groups");
  const uint32_t smem_base = smem_u32(smem);
  const int k_groups = (p.k_tiles + KS - 1) / KS;
  int group = 0;
  uint32_t phase = 0;
  uint32_t local_tile = 0;
  uint32_t step = 0;  // global K-step counter: picks the scale set
  const bool leader = elect_one_sync();
  for (int tile = first_tile; tile < total_tiles; tile += tile_stride, ++local_tile) {
    const uint32_t acc_col = (local_tile & 1) ? TP::kAccWindow1 : 0;
    if (local_tile > 0) {
      // previous tile's epilogue has drained the columns both windows share
      if (!mbar_wait(acc_overlap_bar, (local_tile - 1) & 1, abort_flag)) {
        if (p.status) atomicCAS(p.status, 0, kStatusWaitMma);
        *abort_flag = 1;
        return;
      }
      tc_fence_after_sync();
    }
    for (int kg = 0; kg < k_groups; ++kg) {
      if (!mbar_wait(&full_bar[group], phase, abort_flag)) {
        if (p.status) atomicCAS(p.status, 0, kStatusWaitMma);
        *abort_flag = 1;
        return;
      }
      if (leader) {
#pragma unroll
        for (int sub = 0; sub < KS; ++sub) {
          // A barrier group may reach past the end of K.  Those steps are loaded (zero payload) but
          // never issued: the scale bytes beside them belong to the next row block or to an earlier
          // use of the slot, and a NaN scale (E8M0 0xFF) against a zero payload would still give NaN.
          if (kg * KS + sub >= p.k_tiles) break;
          const int slot = group * KS + sub;
          const int set = step & 1;
          ++step;
          // SFB in the ring: per slot [half 0 | half 1] (single-CTA kernel), or per barrier group
          // [half 0 of its KS steps | half 1 of its KS steps] (pair kernel: one load brings a group's halves)
          const uint32_t ssfb0 = PAIR ? smem_base + OFF_SFB + group * KS * SFB_BYTES + sub * SFA_BYTES
                                      : smem_base + OFF_SFB + slot * SFB_BYTES;
          const uint32_t ssfb1 = ssfb0 + (PAIR ? KS * SFA_BYTES : SFA_BYTES);
          issue_scale_copy<KIND, PAIR>(tmem_base, smem_base + OFF_SFA + slot * SFA_BYTES, ssfb0, ssfb1, set);
          issue_k_step<KIND, PAIR>(tmem_base, acc_col, smem_base + slot * A_BYTES, smem_base + OFF_B + slot * B_BYTES,
                                   set, idesc, kg == 0 && sub == 0);
        }
        // slots reusable once these MMAs (and the copies before them) have read them
        if (PAIR) tc_commit_pair(&empty_bar[group], 3);
        else tc_commit(&empty_bar[group]);
      }
      __syncwarp();
      if (++group == GROUPS) { group = 0; phase ^= 1; }
    }
    if (leader) {
      if (PAIR) tc_commit_pair(acc_full_bar, 3);
      else tc_commit(acc_full_bar);
    }
    __syncwarp();
  }
}

template <int KIND, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_blockscaled_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const GemmParams p) {
  using T = GemmTraits<KIND>;
  using TP = TmemPlan<KIND>;
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
    // all lanes run the loop (uniform control flow); one elected lane issues the copies
    {
      const bool leader = elect_one_sync();
      if (leader) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
      }
      griddep_wait();   // operands may come from the kernel launched just before this one
      constexpr int KS = T::kStepsPerBarrier;
      const int k_groups = (p.k_tiles + KS - 1) / KS;
      int group = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int m_idx, n_idx;
        tile_coords(tile, p.m_tiles, p.n_tiles, p.group_m, m_idx, n_idx);
        const int m0 = m_idx * kBlockM;
        // rows of B feeding accumulator columns [0,128) and [128,256)
        int b_row0, b_row1;
        if (epi_is_glu(EPI)) {
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
        for (int kg = 0; kg < k_groups; ++kg) {
          if (!mbar_wait(&empty_bar[group], phase ^ 1, abort_flag)) {
            if (p.status && leader) atomicCAS(p.status, 0, kStatusWaitProducer);
            *abort_flag = 1;
            ok = false;
            break;
          }
          if (leader) {
            // K steps past the end of K fetch zero payload (TMA fill) and no scale tiles
            const int live = min(KS, p.k_tiles - kg * KS);
            // A: only the live rows are fetched when there is a single row block (box of a_box_rows rows; the
            // MMA reads 128 rows of the slot, the rest only reaches accumulator rows that are never stored)
            mbar_expect_tx(&full_bar[group], KS * (p.a_box_rows * kBlockKBytes + T::kBBytes) +
                                                 live * (T::kSfaBytes + (b1_valid ? T::kSfbBytes : T::kSfaBytes)));
#pragma unroll
            for (int sub = 0; sub < KS; ++sub) {
              const int slot = group * KS + sub;
              const int kt = kg * KS + sub;
              uint8_t* sa = smem + slot * T::kABytes;
              uint8_t* sb = smem + T::kOffB + slot * T::kBBytes;
              uint8_t* ssfa = smem + T::kOffSfa + slot * T::kSfaBytes;
              uint8_t* ssfb = smem + T::kOffSfb + slot * T::kSfbBytes;
              tma_load_2d(sa, &map_a, &full_bar[group], kt * kBlockKBytes, m0);
              if (p.b_box256) {
                // the two halves are 256 consecutive rows of B: one box
                tma_load_2d(sb, &map_b, &full_bar[group], kt * kBlockKBytes, b_row0);
              } else {
                tma_load_2d(sb, &map_b, &full_bar[group], kt * kBlockKBytes, b_row0);
                tma_load_2d(sb + 128 * kBlockKBytes, &map_b, &full_bar[group], kt * kBlockKBytes, b_row1);
              }
              if (sub < live) {
                const size_t sf_off = static_cast<size_t>(kt) * T::kSfaBytes;
                bulk_load_1d(ssfa, sfa_src + sf_off, T::kSfaBytes, &full_bar[group]);
                bulk_load_1d(ssfb, sfb_src0 + sf_off, T::kSfaBytes, &full_bar[group]);
                if (b1_valid) bulk_load_1d(ssfb + T::kSfaBytes, sfb_src1 + sf_off, T::kSfaBytes, &full_bar[group]);
              }
            }
          }
          __syncwarp();
          if (++group == kStages / KS) { group = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    {
      mma_issuer_loop<KIND, false, kStages, T::kStepsPerBarrier, T::kABytes, T::kBBytes, T::kOffB, T::kOffSfa, T::kOffSfb, T::kSfaBytes,
                      T::kSfbBytes>(p, smem, full_bar, empty_bar, acc_full_bar, acc_overlap_bar, abort_flag, tmem_base,
                                    T::kIdesc, blockIdx.x, gridDim.x, total_tiles);
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue ------------------------------
    griddep_wait();   // the output scale may come from the kernel launched just before this one
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const float out_scale = p.out_scale ? __ldg(p.out_scale) : 1.0f;
    uint32_t local_tile = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local_tile) {
      int m_idx, n_idx;
      tile_coords(tile, p.m_tiles, p.n_tiles, p.group_m, m_idx, n_idx);
      const int row = m_idx * kBlockM + quad * 32 + lane;
      const bool row_ok = row < p.m;
      const uint32_t acc_col = (local_tile & 1) ? TP::kAccWindow1 : 0;
      if (!mbar_wait(acc_full_bar, local_tile & 1, abort_flag)) {
        if (p.status && lane == 0) atomicCAS(p.status, 0, kStatusWaitEpilogue);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      // row-region policy: the row's own outer scale takes the place of the launch-wide output scale
      const float row_scale = (EPI == kEpiRegionBf16 && row_ok) ? __ldg(p.x_region_scales + row / p.x_region_rows)
                                                                : out_scale;
      epilogue_drain<KIND, EPI>(p, tmem_base + lane_base + acc_col, row, row_ok, n_idx, (local_tile & 1) != 0,
                                smem_u32(acc_overlap_bar), row_scale, lane);
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

// ===========================================================================
// CTA-pair variant (cluster of two CTAs, tcgen05 cta_group::2): pair tile 256 x 256.
//
// Each CTA of the pair owns 128 rows of A and 128 of the 256 rows of B (for the GLU epilogue:
// rank 0 the gate rows, rank 1 the up rows) and fetches only those, so an SM pulls 32 KB per
// 128-byte K step from L2 instead of 48 KB; the MMA issued by the rank-0 CTA reads A and B from
// both CTAs' shared memory and writes a 128 x 256 accumulator into each CTA's TMEM.  No TMA
// multicast is used.  Scale factors: each CTA loads its own SFA tile and the SFB tiles of all 256
// B rows.  All TMA loads of both CTAs signal the rank-0 CTA's `full` barrier; the MMA's commits
// arrive on the `empty` / `acc_full` barriers of both CTAs.  Epilogue as in the single-CTA kernel.
// ===========================================================================
template <int KIND>
struct PairTraits {
  static constexpr int kStagesP = KIND == kKindMxfp8 ? kPairSlotsMx : kPairSlotsNv;   // ring slots
  static constexpr int kStepsPerBarrierP = KIND == kKindMxfp8 ? kPairStepsMx : kPairStepsNv;
  static constexpr int kSfChunks = TmemPlan<KIND>::kSfChunks;
  static constexpr int kSfaBytes = 512 * kSfChunks;
  static constexpr int kSfbBytes = 2 * kSfaBytes;
  static constexpr int kABytes = 128 * kBlockKBytes;
  static constexpr int kBBytes = 128 * kBlockKBytes;   // this CTA's half of the 256 B rows
  static constexpr int kOffB = kStagesP * kABytes;
  static constexpr int kOffSfa = kOffB + kStagesP * kBBytes;
  static constexpr int kOffSfb = kOffSfa + kStagesP * kSfaBytes;
  static constexpr int kOffBars = kOffSfb + kStagesP * kSfbBytes;
  static constexpr int kOffStage = kOffBars + 1024;
  static constexpr int kSmemBytes = kOffStage + kEpiStageBytes + 1024;
  static constexpr int kTxBytesPerCta = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr uint32_t kIdesc =
      idesc_block_scaled(256, 256, KIND == kKindMxfp8 ? 0u : 1u, KIND == kKindMxfp8 ? 1u : 0u);
};

template <int KIND, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_blockscaled_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                             const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                             const __grid_constant__ OutMaps maps_out, const GemmParams p) {
  using T = PairTraits<KIND>;
  using TP = TmemPlan<KIND>;
  constexpr int S = T::kStagesP;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + T::kOffBars);
  uint64_t* full_bar = bars;              // [S] used in the rank-0 CTA: both CTAs' loads land
  uint64_t* empty_bar = bars + S;         // [S] in each CTA: stage free again
  uint64_t* acc_full_bar = bars + 2 * S;  // in each CTA: tile accumulated
  uint64_t* acc_overlap_bar = acc_full_bar + 1;  // rank 0: shared columns drained by all 8 epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_overlap_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int m_pairs = (p.m_tiles + 1) >> 1;
  const int total_tiles = m_pairs * p.n_tiles;

  griddep_launch_dependents();   // a kernel launched as a programmatic dependent may run beside this one

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full_bar[s], 1);
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
  cluster_sync_all();   // the peer's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    {
      const bool leader = elect_one_sync();
      if (leader) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        prefetch_tensormap(&map_sfa);
        prefetch_tensormap(&map_sfb);
      }
      constexpr int KS = T::kStepsPerBarrierP;
      const int k_groups = (p.k_tiles + KS - 1) / KS;
      int group = 0;
      uint32_t phase = 0;
      bool ok = true;
      // launched as a programmatic dependent (composite forwards): the operands come from the quantizer launched just
      // before this kernel; everything above ran beside its tail.  Returns at once for an ordinary launch.
      griddep_wait();
      for (int tile = pair_id; tile < total_tiles && ok; tile += num_pairs) {
        int mp_idx, n_idx;
        tile_coords(rotate_tile(tile, p.tile_shift, total_tiles), m_pairs, p.n_tiles, p.group_m, mp_idx, n_idx);
        const int m_blk = mp_idx * 2 + static_cast<int>(rank);   // 128-row block of A this CTA owns
        int b_blk0, b_blk1;                                      // 128-row blocks of B behind columns [0,128), [128,256)
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
            // One instruction per operand and barrier group where the layout allows it: issuing a TMA
            // instruction costs the issuing thread on the order of 100 clocks, and one K step of MMAs
            // lasts 512.  Payloads: [K/128][rows][128] views (KS steps per load) when rows are 128-byte
            // multiples.  Scale tiles: KS steps of a row block are consecutive rows of the scale maps, and
            // the two B halves are one 3-D box (third coordinate = half).
            const uint32_t full_addr = mapa_shared(smem_u32(&full_bar[group]), 0);
            if (rank == 0) mbar_expect_tx(&full_bar[group], 2 * KS * T::kTxBytesPerCta);
            const int slot0 = group * KS;
            const int kt0 = kg * KS;   // steps past the end of K are loaded (zero fill) but never issued
            if (p.map3d) {
              tma_load_3d_pair(smem + slot0 * T::kABytes, &map_a, full_addr, 0, m_blk * 128, kt0);
              tma_load_3d_pair(smem + T::kOffB + slot0 * T::kBBytes, &map_b, full_addr, 0, b_mine * 128, kt0);
            } else {
#pragma unroll
              for (int sub = 0; sub < KS; ++sub) {
                tma_load_2d_pair(smem + (slot0 + sub) * T::kABytes, &map_a, full_addr, (kt0 + sub) * kBlockKBytes,
                                 m_blk * 128);
                tma_load_2d_pair(smem + T::kOffB + (slot0 + sub) * T::kBBytes, &map_b, full_addr,
                                 (kt0 + sub) * kBlockKBytes, b_mine * 128);
              }
            }
            // scale tiles: rows of the maps are 512-byte tiles, [row block][K tile]
            const int sf_col = kt0 * T::kSfChunks;
            tma_load_2d_pair(smem + T::kOffSfa + slot0 * T::kSfaBytes, &map_sfa, full_addr, 0,
                             m_blk * p.sf_k_chunks + sf_col);
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
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (rank 0 only) ------------------------------
    if (rank == 0) {
      mma_issuer_loop<KIND, true, S, T::kStepsPerBarrierP, T::kABytes, T::kBBytes, T::kOffB, T::kOffSfa, T::kOffSfb, T::kSfaBytes,
                      T::kSfbBytes>(p, smem, full_bar, empty_bar, acc_full_bar, acc_overlap_bar, abort_flag, tmem_base,
                                    T::kIdesc, pair_id, num_pairs, total_tiles);
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    const int quad = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    griddep_wait();   // the output scale (and, for the region epilogue, the scale arrays) may come from the grid before
    const float out_scale = p.out_scale ? __ldg(p.out_scale) : 1.0f;
    const uint32_t overlap_addr = mapa_shared(smem_u32(acc_overlap_bar), 0);
    uint32_t local_tile = 0;
    for (int tile = pair_id; tile < total_tiles; tile += num_pairs, ++local_tile) {
      int mp_idx, n_idx;
      tile_coords(rotate_tile(tile, p.tile_shift, total_tiles), m_pairs, p.n_tiles, p.group_m, mp_idx, n_idx);
      const int row = (mp_idx * 2 + static_cast<int>(rank)) * 128 + quad * 32 + lane;
      const bool row_ok = row < p.m;
      const uint32_t acc_col = (local_tile & 1) ? TP::kAccWindow1 : 0;
      if (!mbar_wait(acc_full_bar, local_tile & 1, abort_flag)) {
        if (p.status && lane == 0) atomicCAS(p.status, 0, kStatusWaitEpilogue);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      const float row_scale = (EPI == kEpiRegionBf16 && row_ok) ? __ldg(p.x_region_scales + row / p.x_region_rows)
                                                                : out_scale;
      // the output block this 256-row pair tile belongs to (whole tiles never straddle blocks)
      const int out_blk = p.out_block_rows > 0 ? (mp_idx * 256) / p.out_block_rows : 0;
      epilogue_drain<KIND, EPI>(p, tmem_base + lane_base + acc_col, row, row_ok, n_idx, (local_tile & 1) != 0,
                                overlap_addr, row_scale, lane, &maps_out.m[out_blk],
                                smem + T::kOffStage + quad * 2 * kEpiStageBufBytes, out_blk * p.out_block_rows);
    }
    if (p.tma_out && lane == 0) tma_store_wait_all<0>();   // shared memory outlives the last store's reads
    __syncwarp();
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // neither CTA frees TMEM or leaves while the pair may still touch it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace rtxb
