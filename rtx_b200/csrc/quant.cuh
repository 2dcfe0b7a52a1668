// HBM-bound quantizers for sm_100a: BF16 -> MXFP8 (rows and transposed) and
// BF16 -> NVFP4, plus the per-tensor |max| reduction that feeds the NVFP4
// outer scale.  They replace the reference's MXFP8QuantKernel /
// MXFP8TransposedQuantKernel (rtx/kernels/mxfp8_quant.py:52-395, :526-1019)
// and NVFP4QuantKernel (rtx/kernels/nvfp4_quant.py:32-349).
//
// Every kernel walks 128-row tiles with a grid-stride loop, reads 16 bytes per
// thread per load, and stages the tile's scale factors in shared memory so
// that the 128-row scale tiles (the layout tcgen05.cp consumes) leave the SM
// as whole 16-byte segments.
#pragma once

#include "common.cuh"

namespace rtxb {

enum ScaleLayout : int { kScaleRowMajor = 0, kScaleMma64 = 1, kScaleMma128 = 2 };

constexpr int kQuantThreads = 256;

// ---------------------------------------------------------------------------
// MXFP8 rows: src bf16 [rows, k] (pitch ld elements) -> q e4m3 [rows, kp],
// scales e8m0.
// ---------------------------------------------------------------------------
struct QuantMxParams {
  const __nv_bfloat16* src;
  uint8_t* q;
  uint8_t* scales;
  int rows, k, kp;       // kp = k rounded up to 32
  int64_t ld;            // source row pitch (elements)
  int nb;                // kp / 32 scale blocks per row
  int sf_chunks;         // 512-byte scale tiles per 128 rows (ceil(nb / 4))
  int layout;            // ScaleLayout
  int round_to_infinity; // 1 = default, 0 = OCP floor ablation
};

__device__ __forceinline__ void load8_bf16(const __nv_bfloat16* row_ptr, int col, int k, bool vec_ok, float (&v)[8]) {
  if (vec_ok && col + 8 <= k) {
    uint4 raw = __ldg(reinterpret_cast<const uint4*>(row_ptr + col));
    v[0] = bf16_lo(raw.x); v[1] = bf16_hi(raw.x); v[2] = bf16_lo(raw.y); v[3] = bf16_hi(raw.y);
    v[4] = bf16_lo(raw.z); v[5] = bf16_hi(raw.z); v[6] = bf16_lo(raw.w); v[7] = bf16_hi(raw.w);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = (col + e < k) ? __bfloat162float(row_ptr[col + e]) : 0.0f;
  }
}

__device__ __forceinline__ float amax8(const float (&v)[8]) {
  float a = fabsf(v[0]);
#pragma unroll
  for (int e = 1; e < 8; ++e) a = fmax_nan(a, fabsf(v[e]));
  return a;
}

// write one 128-row x (4*chunks) block tile of scale bytes held in shared
// memory as tile[row][blocks_in_tile] to global in the requested layout
template <int BLOCKS>
__device__ __forceinline__ void store_scale_tile(const uint8_t (*tile)[BLOCKS], uint8_t* scales, int layout, int row0,
                                                 int blk0, int rows, int nb, int sf_chunks) {
  if (layout == kScaleMma128) {
    // BLOCKS/4 tiles of 512 bytes; one 16-byte segment per (tile, row % 32)
    for (int t = threadIdx.x; t < (BLOCKS / 4) * 32; t += blockDim.x) {
      const int chunk = t >> 5, r32 = t & 31;
      if ((blk0 >> 2) + chunk >= sf_chunks) continue;
      uint32_t w[4];
#pragma unroll
      for (int rg = 0; rg < 4; ++rg) {
        const uint8_t* s = tile[rg * 32 + r32] + chunk * 4;
        w[rg] = s[0] | (s[1] << 8) | (s[2] << 16) | (static_cast<uint32_t>(s[3]) << 24);
      }
      uint8_t* dst = scales + (static_cast<size_t>(row0 >> 7) * sf_chunks + (blk0 >> 2) + chunk) * 512 + r32 * 16;
      *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else {
    for (int t = threadIdx.x; t < 128 * BLOCKS; t += blockDim.x) {
      const int r = t / BLOCKS, b = t % BLOCKS;
      if (row0 + r < rows && blk0 + b < nb) scales[static_cast<size_t>(row0 + r) * nb + blk0 + b] = tile[r][b];
    }
  }
}

// raw 16-byte load of 8 BF16 values (zero beyond k); scalar path for ragged or unaligned rows
__device__ __forceinline__ uint4 load8_raw(const __nv_bfloat16* row_ptr, int col, int k, bool vec_ok) {
  if (vec_ok && col + 8 <= k) return __ldg(reinterpret_cast<const uint4*>(row_ptr + col));
  const uint16_t* s = reinterpret_cast<const uint16_t*>(row_ptr);
  uint32_t w[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const uint32_t lo = (col + 2 * e < k) ? s[col + 2 * e] : 0u;
    const uint32_t hi = (col + 2 * e + 1 < k) ? s[col + 2 * e + 1] : 0u;
    w[e] = lo | (hi << 16);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ void unpack8(const uint4 raw, float (&v)[8]) {
  v[0] = bf16_lo(raw.x); v[1] = bf16_hi(raw.x); v[2] = bf16_lo(raw.y); v[3] = bf16_hi(raw.y);
  v[4] = bf16_lo(raw.z); v[5] = bf16_hi(raw.z); v[6] = bf16_lo(raw.w); v[7] = bf16_hi(raw.w);
}

// One 128 x 128 tile of the row quantizer (see quant_mxfp8_rows_kernel); ends with a block-wide barrier.
__device__ __forceinline__ void quant_mxfp8_rows_tile(const QuantMxParams& p, int tile, uint8_t (*tile_scales)[4]) {
  const int sub = threadIdx.x & 15, rsel = threadIdx.x >> 4;
  const int col_tiles = (p.kp + 127) / 128;
  const bool vec_ok = (p.ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.src) & 15) == 0);
  const bool q_vec_ok = (reinterpret_cast<uintptr_t>(p.q) & 7) == 0;  // kp % 32 == 0 keeps rows 8-byte aligned
  const bool rinf = p.round_to_infinity != 0;
  const int row0 = (tile / col_tiles) * 128;
  const int col = (tile % col_tiles) * 128 + sub * 8;
  const bool col_ok = col < p.kp;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    uint4 raw[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int row = row0 + rsel + 16 * (half * 4 + j);
      raw[j] = (row < p.rows && col_ok) ? load8_raw(p.src + static_cast<int64_t>(row) * p.ld, col, p.k, vec_ok)
                                        : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = rsel + 16 * (half * 4 + j);
      const int row = row0 + r;
      const bool live = row < p.rows && col_ok;
      float v[8];
      unpack8(raw[j], v);
      float a = amax8(v);
      a = fmax_nan(a, __shfl_xor_sync(0xffffffffu, a, 1));
      a = fmax_nan(a, __shfl_xor_sync(0xffffffffu, a, 2));
      const uint32_t code = e8m0_from_amax(a, rinf);
      const float recip = e8m0_reciprocal(code);
      if ((sub & 3) == 0) tile_scales[r][sub >> 2] = live ? static_cast<uint8_t>(code) : 0;
      if (live) {
        const uint32_t lo = cvt_e4m3x2(v[0] * recip, v[1] * recip) | (cvt_e4m3x2(v[2] * recip, v[3] * recip) << 16);
        const uint32_t hi = cvt_e4m3x2(v[4] * recip, v[5] * recip) | (cvt_e4m3x2(v[6] * recip, v[7] * recip) << 16);
        uint8_t* dst = p.q + static_cast<int64_t>(row) * p.kp + col;
        if (q_vec_ok) {
          *reinterpret_cast<uint2*>(dst) = make_uint2(lo, hi);
        } else {
          for (int e = 0; e < 4; ++e) { dst[e] = lo >> (8 * e); dst[4 + e] = hi >> (8 * e); }
        }
      }
    }
  }
  __syncthreads();
  store_scale_tile<4>(tile_scales, p.scales, p.layout, row0, (tile % col_tiles) * 4, p.rows, p.nb, p.sf_chunks);
  __syncthreads();
}

// Tile = 128 rows x 128 columns (exactly one 512-byte scale tile).  Thread t owns 8 columns
// (t & 15) of row (t >> 4) + 16 i; four neighbouring lanes share a block of 32.  Four row loads
// are issued before any is consumed so that each thread keeps 64 bytes in flight.
__global__ void __launch_bounds__(kQuantThreads, 6) quant_mxfp8_rows_kernel(const QuantMxParams p) {
  __shared__ __align__(16) uint8_t tile_scales[128][4];
  const int tiles = ((p.kp + 127) / 128) * ((p.rows + 127) / 128);
  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) quant_mxfp8_rows_tile(p, tile, tile_scales);
}

// Two tensors in one launch (the reference's dual quantizer, rtx/kernels/mxfp8_quant.py:398-1399: activations and
// weight of a dynamic forward): the tiles of `a`, then the tiles of `b`.  On small layers a launch costs more than
// the quantization, and the GEMM launched behind this kernel as a programmatic dependent can set up meanwhile.
__global__ void __launch_bounds__(kQuantThreads, 6) quant_mxfp8_rows2_kernel(const QuantMxParams a, const QuantMxParams b) {
  __shared__ __align__(16) uint8_t tile_scales[128][4];
  griddep_launch_dependents();
  const int tiles_a = ((a.kp + 127) / 128) * ((a.rows + 127) / 128);
  const int tiles_b = ((b.kp + 127) / 128) * ((b.rows + 127) / 128);
  for (int tile = blockIdx.x; tile < tiles_a + tiles_b; tile += gridDim.x) {
    if (tile < tiles_a) quant_mxfp8_rows_tile(a, tile, tile_scales);
    else quant_mxfp8_rows_tile(b, tile - tiles_a, tile_scales);
  }
}

// ---------------------------------------------------------------------------
// MXFP8 transposed: src bf16 stored [k, rows] (pitch ld) -> q e4m3 [rows, kp]
// K-major with blocks of 32 along the stored row index k; equal to quantising
// src^T.contiguous() by rows.  Tile = 128 output rows x 128 k: the CTA reads
// 128 source rows of 128 values (coalesced), keeps them in shared memory and
// each thread then walks one output row's 32-value blocks down a column.
// ---------------------------------------------------------------------------
struct QuantMxTParams {
  const __nv_bfloat16* src;  // [k, rows]
  uint8_t* q;                // [rows, kp]
  uint8_t* scales;
  int rows, k, kp;
  int64_t ld;
  int nb, sf_chunks, layout, round_to_infinity;
  // dual form: the same staged tile is also quantized along the source rows (blocks of 32 source columns),
  // i.e. the plain row quantization of src, so that src is read from memory once for both
  uint8_t* q_rows;           // [k, np], np = source columns rounded up to 32
  uint8_t* s_rows;
  int np, nb_rows, chunks_rows;
};

// Staged tile: [k_local][row_local] BF16 bits, pitch 136 halfwords (272 bytes: 16-byte aligned rows for the
// asynchronous 16-byte copies; a warp reading one k with 32 consecutive row pairs is conflict free).
constexpr int kQtPitch = 136;
constexpr int kQtTileBytes = 128 * kQtPitch * 2;
constexpr int kQtSmemBytes = 2 * kQtTileBytes;   // two tiles: the next one is fetched while this one is quantized

// Pitch of the output staging rows (128 payload bytes + 16): the staged input tile is re-used, once every
// thread has read it, to collect the tile's output bytes so that they leave the SM as whole 128-byte rows.
constexpr int kQtOutPitch = 144;

// Column pass over a staged 128 x 128 tile `tile[k_local][row_local]` (BF16 bits, pitch kQtPitch halfwords):
// thread -> two adjacent output rows (source columns) x one block of 32 along k, so every
// shared-memory read is one 32-bit word holding both rows' values; consecutive lanes read consecutive
// words (conflict free).  Returns the two rows' 32 payload bytes in `o` (o[h][0..7]) and writes the
// 128 x 4 scale codes to `tile_scales`; the payload is stored by quant_mxfp8_tile_columns_store.
__device__ __forceinline__ void quant_mxfp8_tile_columns(const uint16_t (*tile)[kQtPitch], uint8_t (*tile_scales)[4],
                                                         uint32_t (&o)[2][8], int kp, int rows, int row0, int k0,
                                                         bool round_to_infinity) {
  const int rp = threadIdx.x & 63, j = threadIdx.x >> 6;   // 64 row pairs x 4 blocks = 256 threads
  uint32_t w[32];
#pragma unroll
  for (int e = 0; e < 32; ++e) w[e] = *reinterpret_cast<const uint32_t*>(&tile[j * 32 + e][2 * rp]);
  const int kcol = k0 + j * 32;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float a = 0.0f;
#pragma unroll
    for (int e = 0; e < 32; ++e) a = fmax_nan(a, fabsf(h ? bf16_hi(w[e]) : bf16_lo(w[e])));
    const uint32_t code = e8m0_from_amax(a, round_to_infinity);
    const float recip = e8m0_reciprocal(code);
    const int r = 2 * rp + h, row = row0 + r;
    const bool live = row < rows && kcol < kp;
    tile_scales[r][j] = live ? static_cast<uint8_t>(code) : 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float v0 = h ? bf16_hi(w[4 * e]) : bf16_lo(w[4 * e]), v1 = h ? bf16_hi(w[4 * e + 1]) : bf16_lo(w[4 * e + 1]);
      const float v2 = h ? bf16_hi(w[4 * e + 2]) : bf16_lo(w[4 * e + 2]), v3 = h ? bf16_hi(w[4 * e + 3]) : bf16_lo(w[4 * e + 3]);
      o[h][e] = cvt_e4m3x2(v0 * recip, v1 * recip) | (cvt_e4m3x2(v2 * recip, v3 * recip) << 16);
    }
  }
}

// Second half of the column pass, after every thread has finished reading the staged tile: the payload goes
// into the tile's own storage as [row_local][128 bytes] and leaves as whole rows — eight lanes write one
// 128-byte row of q, a warp four rows per instruction (the direct form wrote 16 bytes to 32 different rows
// per instruction).
__device__ __forceinline__ void quant_mxfp8_tile_columns_store(uint8_t* stage, const uint32_t (&o)[2][8], uint8_t* q,
                                                               int kp, int rows, int row0, int k0) {
  const int rp = threadIdx.x & 63, j = threadIdx.x >> 6;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint4* dst = reinterpret_cast<uint4*>(stage + (2 * rp + h) * kQtOutPitch + j * 32);
    dst[0] = make_uint4(o[h][0], o[h][1], o[h][2], o[h][3]);
    dst[1] = make_uint4(o[h][4], o[h][5], o[h][6], o[h][7]);
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = threadIdx.x + kQuantThreads * i;
    const int r = c >> 3, part = c & 7;
    const int row = row0 + r, col = k0 + part * 16;
    if (row < rows && col < kp)
      *reinterpret_cast<uint4*>(q + static_cast<int64_t>(row) * kp + col) =
          *reinterpret_cast<const uint4*>(stage + r * kQtOutPitch + part * 16);
  }
}

// Row pass over the same staged tile (dual form): eight lanes cover one source row of the tile (16 values each,
// two lanes per MX block), so a warp writes four whole 128-byte rows of the row-quantized payload per pass.
__device__ __forceinline__ void quant_mxfp8_tile_rows(const uint16_t (*tile)[kQtPitch], uint8_t (*tile_scales)[4],
                                                      uint8_t* q, int np, int k_rows, int cols, int k0, int col0,
                                                      bool round_to_infinity) {
  const int part = threadIdx.x & 7;
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int r = (threadIdx.x >> 3) + 32 * pass;
    uint32_t w[8];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const uint4 v = *reinterpret_cast<const uint4*>(&tile[r][part * 16 + 8 * c]);
      w[4 * c] = v.x; w[4 * c + 1] = v.y; w[4 * c + 2] = v.z; w[4 * c + 3] = v.w;
    }
    float a = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) a = fmax_nan(a, fmax_nan(fabsf(bf16_lo(w[e])), fabsf(bf16_hi(w[e]))));
    a = fmax_nan(a, __shfl_xor_sync(0xffffffffu, a, 1));
    const uint32_t code = e8m0_from_amax(a, round_to_infinity);
    const float recip = e8m0_reciprocal(code);
    const int row = k0 + r, col = col0 + part * 16;
    const bool live = row < k_rows && col < np;
    if ((part & 1) == 0) tile_scales[r][part >> 1] = live ? static_cast<uint8_t>(code) : 0;
    if (live) {
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        o[e] = cvt_e4m3x2(bf16_lo(w[2 * e]) * recip, bf16_hi(w[2 * e]) * recip) |
               (cvt_e4m3x2(bf16_lo(w[2 * e + 1]) * recip, bf16_hi(w[2 * e + 1]) * recip) << 16);
      *reinterpret_cast<uint4*>(q + static_cast<int64_t>(row) * np + col) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

constexpr int kQtOccupancy = 3;   // resident CTAs per SM the transposed quantizer is compiled for (registers, 70 KB of tiles)
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src, bool valid) {
  // copies 16 bytes, or writes 16 zero bytes when !valid (source size 0)
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src),
               "r"(valid ? 16 : 0)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// fetch tile t (128 source rows x 128 source columns) into `tile`; aligned full-width tiles asynchronously
__device__ __forceinline__ void quant_mxfp8_t_fetch(const QuantMxTParams& p, uint16_t (*tile)[kQtPitch], int row0, int k0,
                                                    bool vec_ok) {
  const uint16_t* src = reinterpret_cast<const uint16_t*>(p.src);
  if (vec_ok && row0 + 128 <= p.rows) {
    const int c8 = (threadIdx.x & 15) * 8, kr = threadIdx.x >> 4;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int gk = k0 + kr + 16 * j;
      const bool valid = gk < p.k;
      cp_async_16(&tile[kr + 16 * j][c8], src + static_cast<int64_t>(valid ? gk : 0) * p.ld + row0 + c8, valid);
    }
  } else {
    for (int i = threadIdx.x; i < 128 * 64; i += kQuantThreads) {
      const int kk = i >> 6, c2 = (i & 63) * 2;
      const int gk = k0 + kk, gc = row0 + c2;
      uint16_t a = 0, b = 0;
      if (gk < p.k) {
        const uint16_t* rp = src + static_cast<int64_t>(gk) * p.ld;
        if (gc < p.rows) a = rp[gc];
        if (gc + 1 < p.rows) b = rp[gc + 1];
      }
      tile[kk][c2] = a;
      tile[kk][c2 + 1] = b;
    }
  }
  cp_async_commit();
}

template <bool DUAL>
__global__ void __launch_bounds__(kQuantThreads, kQtOccupancy) quant_mxfp8_transposed_kernel(const QuantMxTParams p) {
  extern __shared__ __align__(16) uint8_t qt_smem[];
  uint16_t (*tiles[2])[kQtPitch] = {reinterpret_cast<uint16_t (*)[kQtPitch]>(qt_smem),
                                    reinterpret_cast<uint16_t (*)[kQtPitch]>(qt_smem + kQtTileBytes)};
  __shared__ __align__(16) uint8_t tile_scales[128][4];
  __shared__ __align__(16) uint8_t tile_scales_rows[DUAL ? 128 : 1][4];
  const int row_tiles = (p.rows + 127) / 128;
  const int k_tiles = (p.kp + 127) / 128;
  const int total = row_tiles * k_tiles;
  const bool vec_ok = (p.ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.src) & 15) == 0);
  int buf = 0;
  if (static_cast<int>(blockIdx.x) < total)
    quant_mxfp8_t_fetch(p, tiles[0], (blockIdx.x % row_tiles) * 128, (blockIdx.x / row_tiles) * 128, vec_ok);
  for (int t = blockIdx.x; t < total; t += gridDim.x) {
    const int row0 = (t % row_tiles) * 128;  // output rows = source columns
    const int k0 = (t / row_tiles) * 128;
    const int tn = t + gridDim.x;
    if (tn < total) {
      quant_mxfp8_t_fetch(p, tiles[buf ^ 1], (tn % row_tiles) * 128, (tn / row_tiles) * 128, vec_ok);
      cp_async_wait<1>();   // everything but the newest group (the next tile) has landed
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    uint32_t o[2][8];
    quant_mxfp8_tile_columns(tiles[buf], tile_scales, o, p.kp, p.rows, row0, k0, p.round_to_infinity != 0);
    if (DUAL)
      quant_mxfp8_tile_rows(tiles[buf], tile_scales_rows, p.q_rows, p.np, p.k, p.rows, k0, row0,
                            p.round_to_infinity != 0);
    __syncthreads();   // every thread has read the staged tile: its storage now collects the transposed payload
    quant_mxfp8_tile_columns_store(reinterpret_cast<uint8_t*>(tiles[buf]), o, p.q, p.kp, p.rows, row0, k0);
    store_scale_tile<4>(tile_scales, p.scales, p.layout, row0, k0 / 32, p.rows, p.nb, p.sf_chunks);
    if (DUAL) store_scale_tile<4>(tile_scales_rows, p.s_rows, p.layout, k0, row0 / 32, p.k, p.nb_rows, p.chunks_rows);
    __syncthreads();   // the scale tiles and this buffer are free again
    buf ^= 1;
  }
}

// ---------------------------------------------------------------------------
// per-tensor |max| (NaN-propagating) of a BF16 matrix, accumulated with an
// integer atomic max on the FP32 bit pattern (non-negative floats order like
// integers and every NaN pattern is larger than infinity)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) amax_bf16_kernel(const __nv_bfloat16* src, int64_t rows, int64_t k, int64_t ld,
                                                        uint32_t* amax_bits) {
  uint32_t m = 0;
  const bool vec_ok = (ld % 8 == 0) && (k % 8 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
  if (vec_ok && ld == k) {
    // contiguous tensor: plain linear indexing (no division per load), eight 16-byte loads in flight per thread
    const uint4* base = reinterpret_cast<const uint4*>(src);
    const int64_t total = rows * (k / 8);
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i0 = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i0 < total; i0 += 8 * stride) {
      uint4 raw[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) raw[j] = i0 + j * stride < total ? __ldg(base + i0 + j * stride) : make_uint4(0, 0, 0, 0);
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
  } else if (vec_ok) {
    // four 16-byte loads in flight per thread
    const int64_t vec_per_row = k / 8;
    const int64_t total = rows * vec_per_row;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i0 = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i0 < total; i0 += 4 * stride) {
      uint4 raw[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int64_t i = i0 + j * stride;
        raw[j] = i < total ? __ldg(reinterpret_cast<const uint4*>(src + (i / vec_per_row) * ld + (i % vec_per_row) * 8))
                           : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t w[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          m = max(m, (w[e] << 16) & 0x7FFFFFFFu);
          m = max(m, w[e] & 0x7FFF0000u);
        }
      }
    }
  } else {
    const int64_t total = rows * k;
    const uint16_t* s = reinterpret_cast<const uint16_t*>(src);
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
      m = max(m, (static_cast<uint32_t>(s[(i / k) * ld + (i % k)]) << 16) & 0x7FFFFFFFu);
    }
  }
  m = __reduce_max_sync(0xffffffffu, m);
  if ((threadIdx.x & 31) == 0 && m != 0) atomicMax(amax_bits, m);
}

// Outer (per tensor / per region) decode scale from a |max| given as FP32 bits.
// mode 0: exact amax / (448 * 6); mode 1: the power of two 2^ceil(log2(max(amax / 2688, 2^-126))).
// 1.0 when amax is zero or NaN (the reference selects with `amax > 0`, rtx/fp4.py:343-365).
// The reference forms the quotient in two ways and both are kept bit for bit:
//   kernel_form = false  division, as its PyTorch functions do for the `current` policy and for
//                        quantize_nvfp4 (rtx/fp4.py:346, 361);
//   kernel_form = true   multiplication by the FP32 constant 1/2688, as its quantizer kernels do for
//                        the delayed and row-region policies (rtx/kernels/nvfp4_quant.py:117-143).
// The power of two comes from the exponent-bump rule of those kernels; on every BF16 magnitude it
// equals the PyTorch exp2(ceil(log2(t))) form (checked exhaustively against the reference's function).
__device__ __forceinline__ float nvfp4_scale_from_amax_bits(uint32_t amax_bits, int mode, bool kernel_form = false) {
  const float amax = __uint_as_float(amax_bits);
  const float quotient = kernel_form ? __fmul_rn(amax, 1.0f / 2688.0f) : __fdiv_rn(amax, 2688.0f);
  float s;
  if (mode == 0) {
    s = quotient;
  } else {
    const float target = fmax_nan(quotient, 1.17549435e-38f);
    const uint32_t bits = __float_as_uint(target);
    uint32_t ebits = bits & 0x7F800000u;
    if (bits & 0x007FFFFFu) ebits += 1u << 23;
    s = __uint_as_float(ebits);
  }
  if (!(amax > 0.0f)) s = 1.0f;
  return s;
}

__global__ void nvfp4_tensor_scale_kernel(const uint32_t* amax_bits, int mode, float* scale, const float* other_scale,
                                          float* out_scale, bool kernel_form) {
  const float s = nvfp4_scale_from_amax_bits(*amax_bits, mode, kernel_form);
  *scale = s;
  if (out_scale) *out_scale = s * *other_scale;
}

// ---------------------------------------------------------------------------
// NVFP4: src bf16 [rows, k] -> packed e2m1 [rows, kp/2] (kp = k rounded up to
// 32), E4M3 block scale per 16 values; a thread owns one whole block of 16
// values (two 16-byte loads, one 8-byte store).
// ---------------------------------------------------------------------------
struct QuantNvParams {
  const __nv_bfloat16* src;
  uint8_t* q;
  uint8_t* scales;
  const float* tensor_scale;  // device scalar, nullptr = 1.0 (block policy)
  const float* region_scales; // row-region policy: outer scale of rows [i * region_rows, (i + 1) * region_rows)
  int region_rows;            // 0 = one scale for the tensor (tensor_scale)
  int rows, k, kp;
  int64_t ld;
  int nb;         // kp / 16
  int sf_chunks;  // 512-byte tiles per 128 rows
  int layout;
};

// Tile = 128 rows x 256 columns (16 blocks = four 512-byte scale tiles).  Thread t owns the
// block (t & 15) of row (t >> 4) + 16 i; the loads of two rows (four 16-byte loads) are issued
// before the first is consumed.
struct QuantNvTileCtx {
  int sub, rsel, col_tiles, row_bytes;
  bool vec_ok;
  float six_st, inv_st;
};

__device__ __forceinline__ QuantNvTileCtx quant_nvfp4_ctx(const QuantNvParams& p, float st) {
  QuantNvTileCtx c;
  c.sub = threadIdx.x & 15;
  c.rsel = threadIdx.x >> 4;
  c.col_tiles = (p.kp + 255) / 256;
  c.row_bytes = p.kp / 2;
  c.vec_ok = (p.ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.src) & 15) == 0);
  c.six_st = 6.0f * st;
  c.inv_st = __fdiv_rn(1.0f, st);
  return c;
}

// one 128 x 256 tile: payload bytes and the tile's scale bytes (block-wide: ends with a barrier).
// REGION: the outer scale is looked up per row (row-region policy) instead of being one per tensor.
template <bool REGION = false, bool OBSERVE = false>
__device__ __forceinline__ void quant_nvfp4_tile(const QuantNvParams& p, const QuantNvTileCtx& c, int tile,
                                                 uint8_t (*tile_scales)[16], const float2* row_factors = nullptr,
                                                 float* observed = nullptr) {
  // OBSERVE: *observed accumulates the |max| of everything this thread quantizes (delayed policy)
  // row_factors (REGION): per row of the tile {6 * scale, 1 / scale} of the row's region, in shared memory
  const int row0 = (tile / c.col_tiles) * 128;
  const int col = (tile % c.col_tiles) * 256 + c.sub * 16;
  const bool col_ok = col < p.kp;
#pragma unroll
  for (int pair = 0; pair < 4; ++pair) {
    uint4 raw[2][2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int row = row0 + c.rsel + 16 * (pair * 2 + j);
      if (row < p.rows && col_ok) {
        const __nv_bfloat16* rp = p.src + static_cast<int64_t>(row) * p.ld;
        raw[j][0] = load8_raw(rp, col, p.k, c.vec_ok);
        raw[j][1] = load8_raw(rp, col + 8, p.k, c.vec_ok);
      } else {
        raw[j][0] = raw[j][1] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int r = c.rsel + 16 * (pair * 2 + j);
      const int row = row0 + r;
      const bool live = row < p.rows && col_ok;
      float v[16];
      unpack8(raw[j][0], *reinterpret_cast<float(*)[8]>(&v[0]));
      unpack8(raw[j][1], *reinterpret_cast<float(*)[8]>(&v[8]));
      float a = fabsf(v[0]);
#pragma unroll
      for (int e = 1; e < 16; ++e) a = fmax_nan(a, fabsf(v[e]));
      if (OBSERVE) *observed = fmax_nan(*observed, a);
      float six_st = c.six_st, inv_st = c.inv_st;
      if (REGION) {
        const float2 f = row_factors[r];
        six_st = f.x;
        inv_st = f.y;
      }
      float rawscale = __fdiv_rn(a, six_st);
      rawscale = fmin_nan(fmax_nan(rawscale, 0.015625f), 448.0f);
      const uint32_t sb = cvt_e4m3x2(rawscale, rawscale) & 0xFF;
      const float recip = __fdiv_rn(inv_st, e4m3_to_float(sb));
      tile_scales[r][c.sub] = live ? static_cast<uint8_t>(sb) : 0;
      if (live) {
        uint32_t w0 = 0, w1 = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          w0 |= cvt_e2m1x2(v[2 * e] * recip, v[2 * e + 1] * recip) << (8 * e);
          w1 |= cvt_e2m1x2(v[8 + 2 * e] * recip, v[8 + 2 * e + 1] * recip) << (8 * e);
        }
        *reinterpret_cast<uint2*>(p.q + static_cast<int64_t>(row) * c.row_bytes + col / 2) = make_uint2(w0, w1);
      }
    }
  }
  __syncthreads();
  store_scale_tile<16>(tile_scales, p.scales, p.layout, row0, (tile % c.col_tiles) * 16, p.rows, p.nb, p.sf_chunks);
  __syncthreads();
}

__global__ void __launch_bounds__(kQuantThreads, 4) quant_nvfp4_rows_kernel(const QuantNvParams p) {
  __shared__ __align__(16) uint8_t tile_scales[128][16];
  const float st = p.tensor_scale ? __ldg(p.tensor_scale) : 1.0f;
  const QuantNvTileCtx c = quant_nvfp4_ctx(p, st);
  const int row_tiles = (p.rows + 127) / 128;
  for (int tile = blockIdx.x; tile < c.col_tiles * row_tiles; tile += gridDim.x) quant_nvfp4_tile(p, c, tile, tile_scales);
}

// ---------------------------------------------------------------------------
// Delayed policy (NVFP4DelayedDualQuantKernel, rtx/kernels/nvfp4_quant.py:473-664): the outer scale
// comes from the |max| history of earlier steps (history[0] = most recent; the window maximum or only
// the most recent entry), and the same single read of the tensor both quantizes it with that scale
// and observes its |max|, published as next_history[0]; next_history[i] = history[i - 1].  No
// reduction over the current tensor stands before the quantization.  next_history[0] must be zero
// when the kernel starts (the entry point clears it).
// ---------------------------------------------------------------------------
struct QuantNvDelayedParams {
  QuantNvParams q;            // q.tensor_scale / region fields are not read
  const float* history;       // [history_len]
  float* next_history;        // [history_len]
  int history_len, entries;   // entries read for the scale: history_len (window_max) or 1 (most_recent)
  int mode;
  float* scale_out;           // [1] the scale used
  const float* other_scale;   // nullptr or [1]
  float* out_scale;           // nullptr or [1] = scale * other_scale
};

__global__ void __launch_bounds__(kQuantThreads, 4) quant_nvfp4_delayed_kernel(const QuantNvDelayedParams dp) {
  __shared__ __align__(16) uint8_t tile_scales[128][16];
  __shared__ uint32_t prior_bits;
  const QuantNvParams& p = dp.q;
  if (threadIdx.x < 32) {
    uint32_t m = 0;
    for (int i = threadIdx.x; i < dp.entries; i += 32) m = max(m, __float_as_uint(__ldg(dp.history + i)) & 0x7FFFFFFFu);
    m = __reduce_max_sync(0xffffffffu, m);
    if (threadIdx.x == 0) prior_bits = m;
    if (blockIdx.x == 0) {
      for (int i = threadIdx.x + 1; i < dp.history_len; i += 32) dp.next_history[i] = __ldg(dp.history + i - 1);
    }
  }
  __syncthreads();
  const float st = nvfp4_scale_from_amax_bits(prior_bits, dp.mode, true);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    *dp.scale_out = st;
    if (dp.out_scale) *dp.out_scale = st * *dp.other_scale;
  }
  const QuantNvTileCtx c = quant_nvfp4_ctx(p, st);
  const int row_tiles = (p.rows + 127) / 128;
  float observed = 0.0f;
  for (int tile = blockIdx.x; tile < c.col_tiles * row_tiles; tile += gridDim.x)
    quant_nvfp4_tile<false, true>(p, c, tile, tile_scales, nullptr, &observed);
  uint32_t obs = __float_as_uint(observed) & 0x7FFFFFFFu;   // NaN keeps a pattern above infinity
  obs = __reduce_max_sync(0xffffffffu, obs);
  if ((threadIdx.x & 31) == 0 && obs != 0) atomicMax(reinterpret_cast<uint32_t*>(dp.next_history), obs);
}

// ---------------------------------------------------------------------------
// Row-region policy (the reference's default NVFP4 scaling, NVFP4JITRegionDualQuantKernel,
// rtx/kernels/nvfp4_quant.py:667-1000): one FP32 outer scale per region of `region_rows` consecutive
// rows, from the region's current |max|.  Here: one warp reduces a region and applies the scale rule
// (amax_regions_kernel), then the tiled quantizer looks the scale up per row.
// ---------------------------------------------------------------------------
// |max| bits of one region (region_rows rows of k values), reduced by one warp
__device__ __forceinline__ uint32_t amax_region_warp(const __nv_bfloat16* src, int k, int64_t ld, int region_rows, int region,
                                                     int lane, bool vec_ok) {
  uint32_t m = 0;
  if (vec_ok && ld == k) {
    // contiguous region: one flat range, eight 16-byte loads in flight per lane (a region of a small layer is a few
    // tens of kilobytes read by ONE warp: the number of dependent load rounds is its whole cost)
    const uint4* base = reinterpret_cast<const uint4*>(src + static_cast<int64_t>(region) * region_rows * ld);
    const int vecs = region_rows * (k / 8);
    for (int i0 = lane; i0 < vecs; i0 += 256) {
      uint4 raw[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) raw[j] = i0 + 32 * j < vecs ? __ldg(base + i0 + 32 * j) : make_uint4(0, 0, 0, 0);
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
    return __reduce_max_sync(0xffffffffu, m);
  }
  for (int r = 0; r < region_rows; ++r) {
    const __nv_bfloat16* rp = src + static_cast<int64_t>(region * region_rows + r) * ld;
    if (vec_ok) {
      const int vecs = k / 8;
      for (int i0 = lane; i0 < vecs; i0 += 128) {   // four 16-byte loads in flight per lane
        uint4 raw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          raw[j] = i0 + 32 * j < vecs ? __ldg(reinterpret_cast<const uint4*>(rp) + i0 + 32 * j) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t w[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            m = max(m, (w[e] << 16) & 0x7FFFFFFFu);
            m = max(m, w[e] & 0x7FFF0000u);
          }
        }
      }
    } else {
      const uint16_t* sp = reinterpret_cast<const uint16_t*>(rp);
      for (int i = lane; i < k; i += 32) m = max(m, (static_cast<uint32_t>(sp[i]) << 16) & 0x7FFFFFFFu);
    }
  }
  return __reduce_max_sync(0xffffffffu, m);
}

__global__ void __launch_bounds__(256) amax_regions_kernel(const __nv_bfloat16* src, int rows, int k, int64_t ld,
                                                           int region_rows, int mode, float* region_scales) {
  const int regions = rows / region_rows;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const bool vec_ok = (ld % 8 == 0) && (k % 8 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
  for (int region = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; region < regions; region += warps) {
    const uint32_t m = amax_region_warp(src, k, ld, region_rows, region, lane, vec_ok);
    if (lane == 0) region_scales[region] = nvfp4_scale_from_amax_bits(m, mode, true);
  }
}

// Region scales of two tensors with the same k (activations and weight of a dynamic forward) in one launch: on
// small layers the launches cost more than the reductions.
struct RegionScaleJob {
  const __nv_bfloat16* src;
  float* region_scales;
  int rows, region_rows;
  int64_t ld;
};
__global__ void __launch_bounds__(256) amax_regions2_kernel(const RegionScaleJob a, const RegionScaleJob b, int k, int mode) {
  griddep_launch_dependents();
  const int regions_a = a.rows / a.region_rows, regions_b = b.rows / b.region_rows;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int idx = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; idx < regions_a + regions_b; idx += warps) {
    const RegionScaleJob& j = idx < regions_a ? a : b;
    const int region = idx < regions_a ? idx : idx - regions_a;
    const bool vec_ok = (j.ld % 8 == 0) && (k % 8 == 0) && ((reinterpret_cast<uintptr_t>(j.src) & 15) == 0);
    const uint32_t m = amax_region_warp(j.src, k, j.ld, j.region_rows, region, lane, vec_ok);
    if (lane == 0) j.region_scales[region] = nvfp4_scale_from_amax_bits(m, mode, true);
  }
}

// The same reduction with a whole CTA per region, for regions large enough to keep 256 threads busy
// (a region is contiguous when ld == k: the threads then stride over it as one flat range).
__global__ void __launch_bounds__(256) amax_regions_cta_kernel(const __nv_bfloat16* src, int rows, int k, int64_t ld,
                                                               int region_rows, int mode, float* region_scales) {
  __shared__ uint32_t warp_max[8];
  const int regions = rows / region_rows;
  const bool flat = (ld == k) && (k % 8 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
  for (int region = blockIdx.x; region < regions; region += gridDim.x) {
    uint32_t m = 0;
    if (flat) {
      const uint4* base = reinterpret_cast<const uint4*>(src + static_cast<int64_t>(region) * region_rows * ld);
      const int vecs = region_rows * (k / 8);
      for (int i0 = threadIdx.x; i0 < vecs; i0 += 4 * 256) {
        uint4 raw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) raw[j] = i0 + 256 * j < vecs ? __ldg(base + i0 + 256 * j) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t w[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            m = max(m, (w[e] << 16) & 0x7FFFFFFFu);
            m = max(m, w[e] & 0x7FFF0000u);
          }
        }
      }
    } else {
      const uint16_t* sp = reinterpret_cast<const uint16_t*>(src);
      const int64_t total = static_cast<int64_t>(region_rows) * k;
      for (int64_t i = threadIdx.x; i < total; i += 256) {
        const int64_t row = region * static_cast<int64_t>(region_rows) + i / k;
        m = max(m, (static_cast<uint32_t>(sp[row * ld + i % k]) << 16) & 0x7FFFFFFFu);
      }
    }
    m = __reduce_max_sync(0xffffffffu, m);
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
      uint32_t v = threadIdx.x < 8 ? warp_max[threadIdx.x] : 0u;
      v = __reduce_max_sync(0xffffffffu, v);
      if (threadIdx.x == 0) region_scales[region] = nvfp4_scale_from_amax_bits(v, mode, true);
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kQuantThreads, 4) quant_nvfp4_regions_kernel(const QuantNvParams p) {
  __shared__ __align__(16) uint8_t tile_scales[128][16];
  __shared__ float2 row_factors[128];
  const QuantNvTileCtx c = quant_nvfp4_ctx(p, 1.0f);
  const int row_tiles = (p.rows + 127) / 128;
  int table_row0 = -1;
  for (int tile = blockIdx.x; tile < c.col_tiles * row_tiles; tile += gridDim.x) {
    const int row0 = (tile / c.col_tiles) * 128;
    if (row0 != table_row0) {
      // the 128 rows of this tile: look the region scale up once per row, not once per block of 16 values
      if (threadIdx.x < 128) {
        const int row = row0 + threadIdx.x;
        const float st = row < p.rows ? __ldg(p.region_scales + row / p.region_rows) : 1.0f;
        row_factors[threadIdx.x] = make_float2(6.0f * st, __fdiv_rn(1.0f, st));
      }
      table_row0 = row0;
      __syncthreads();
    }
    quant_nvfp4_tile<true>(p, c, tile, tile_scales, row_factors);   // ends with a block-wide barrier
  }
}

// Two tensors in one launch (tiles of `a`, then tiles of `b`), launched as a programmatic dependent of
// amax_regions2_kernel: it waits for that grid before it reads a region scale.
__global__ void __launch_bounds__(kQuantThreads, 4) quant_nvfp4_regions2_kernel(const QuantNvParams a, const QuantNvParams b) {
  __shared__ __align__(16) uint8_t tile_scales[128][16];
  __shared__ float2 row_factors[128];
  griddep_launch_dependents();
  const QuantNvTileCtx ca = quant_nvfp4_ctx(a, 1.0f), cb = quant_nvfp4_ctx(b, 1.0f);
  const int tiles_a = ca.col_tiles * ((a.rows + 127) / 128), tiles_b = cb.col_tiles * ((b.rows + 127) / 128);
  griddep_wait();
  int table_key = -1;
  for (int idx = blockIdx.x; idx < tiles_a + tiles_b; idx += gridDim.x) {
    const bool first = idx < tiles_a;
    const QuantNvParams& p = first ? a : b;
    const QuantNvTileCtx& c = first ? ca : cb;
    const int tile = first ? idx : idx - tiles_a;
    const int row0 = (tile / c.col_tiles) * 128;
    const int key = 2 * row0 + (first ? 0 : 1);
    if (key != table_key) {
      if (threadIdx.x < 128) {
        const int row = row0 + threadIdx.x;
        const float st = row < p.rows ? __ldg(p.region_scales + row / p.region_rows) : 1.0f;
        row_factors[threadIdx.x] = make_float2(6.0f * st, __fdiv_rn(1.0f, st));
      }
      table_key = key;
      __syncthreads();
    }
    quant_nvfp4_tile<true>(p, c, tile, tile_scales, row_factors);   // ends with a block-wide barrier
  }
}

// ---------------------------------------------------------------------------
// Small tensors (decode activations): the outer scale from the tensor's own |max| and the
// quantization as two launches chained by programmatic dependent launch, with no memset and no
// one-thread finalize launch in between:
//   amax_partials_kernel     CTA p writes the |max| bits of tiles p, p + P, ... to partials[p]
//   quant_nvfp4_dynamic_kernel  every CTA reduces the P partials itself, applies the scale rule
//                            (all CTAs get the same bits), CTA 0 publishes the scale(s), then the
//                            tiles are quantized with the code of the two-pass path.
// Both let their dependents start early (griddepcontrol.launch_dependents first thing) and wait
// for their own predecessor before touching global memory that it may still use.
// Replaces, for small M, the reference's torch reductions of `_outer_tensor_scale`
// (rtx/fp4.py:343-365) followed by compile_nvfp4_quant (rtx/kernels/nvfp4_quant.py:32-349).
// ---------------------------------------------------------------------------
constexpr int kDynamicMaxPartials = 64;

__global__ void __launch_bounds__(kQuantThreads) amax_partials_kernel(const QuantNvParams p, uint32_t* partials) {
  __shared__ uint32_t cta_amax;
  griddep_launch_dependents();
  if (threadIdx.x == 0) cta_amax = 0;
  griddep_wait();   // src may be the output of the kernel before this one; partials may still be read by it
  __syncthreads();
  const QuantNvTileCtx c = quant_nvfp4_ctx(p, 1.0f);
  const int tiles = c.col_tiles * ((p.rows + 127) / 128);
  uint32_t m = 0;
  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int row0 = (tile / c.col_tiles) * 128;
    const int col = (tile % c.col_tiles) * 256 + c.sub * 16;
    if (col >= p.kp) continue;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = row0 + c.rsel + 16 * i;
      if (row >= p.rows) continue;
      const __nv_bfloat16* rp = p.src + static_cast<int64_t>(row) * p.ld;
      const uint4 a = load8_raw(rp, col, p.k, c.vec_ok), b = load8_raw(rp, col + 8, p.k, c.vec_ok);
      const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        m = max(m, (w[e] << 16) & 0x7FFFFFFFu);
        m = max(m, w[e] & 0x7FFF0000u);
      }
    }
  }
  m = __reduce_max_sync(0xffffffffu, m);
  if ((threadIdx.x & 31) == 0 && m != 0) atomicMax(&cta_amax, m);
  __syncthreads();
  if (threadIdx.x == 0) partials[blockIdx.x] = cta_amax;
}

struct QuantNvDynamicParams {
  QuantNvParams q;           // q.tensor_scale is not read
  int mode;                  // 0 exact, 1 power of two
  const uint32_t* partials;  // [n_partials] |max| bits
  int n_partials;            // <= kDynamicMaxPartials
  float* scale_out;          // [1]
  const float* other_scale;  // nullptr or [1]
  float* out_scale;          // nullptr or [1] = scale * other_scale
};

__global__ void __launch_bounds__(kQuantThreads, 4) quant_nvfp4_dynamic_kernel(const QuantNvDynamicParams dp) {
  __shared__ __align__(16) uint8_t tile_scales[128][16];
  __shared__ uint32_t warp_amax[2];
  griddep_launch_dependents();
  griddep_wait();
  const QuantNvParams& p = dp.q;
  if (threadIdx.x < 64) {
    uint32_t v = threadIdx.x < dp.n_partials ? dp.partials[threadIdx.x] : 0u;
    v = __reduce_max_sync(0xffffffffu, v);
    if ((threadIdx.x & 31) == 0) warp_amax[threadIdx.x >> 5] = v;
  }
  __syncthreads();
  const float st = nvfp4_scale_from_amax_bits(max(warp_amax[0], warp_amax[1]), dp.mode);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    *dp.scale_out = st;
    if (dp.out_scale) *dp.out_scale = st * *dp.other_scale;
  }
  const QuantNvTileCtx c = quant_nvfp4_ctx(p, st);
  const int tiles = c.col_tiles * ((p.rows + 127) / 128);
  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) quant_nvfp4_tile(p, c, tile, tile_scales);
}

}  // namespace rtxb
